"""The scheduler's decisions against a fake executor that makes up sampled tokens
(the reference tests its scheduler against a host-allocated pool the same way,
tests/unit/scheduler_test.cc:28-78).  The behaviours are those of
scheduler_test.cc:451 (chunks), :505 (decodes first), :742 (a preempted sequence
produces the same tokens), :853 (back to the front of the queue), :903 (context
limit), :963 (a lone sequence that cannot grow), :1367 (every token of a batch has
a page)."""
import pytest

from inferx_b200.cache import CacheGroup, CacheManager
from inferx_b200.engine.scheduler import (CANCELLED, CONTEXT_LIMIT, MAX_TOKENS, OUT_OF_MEMORY,
                                          STOP_TOKEN, Scheduler, SchedulerConfig)
from inferx_b200.sampling import SamplingParams


def fake_token(rid, position):
    """What the fake model 'samples' after the token at ``position`` of request rid."""
    import zlib
    return zlib.crc32(f"{rid}:{position}".encode()) % 9973 + 3


def make(pages=64, page=4, slots=8, windows=(0,), **cfg):
    cache = CacheManager([CacheGroup(w) for w in windows], pages, page, slots)
    return Scheduler(SchedulerConfig(**cfg), cache), cache


def run(sched, cache, max_steps=10000, on_step=None):
    """Drive prepare/commit with the fake executor until nothing is left."""
    done, log = {}, []
    for _ in range(max_steps):
        if not sched.has_work():
            break
        planned = sched.prepare_step()
        for c in sched.take_completed():
            done[c.id] = c
        if not planned:
            continue
        # every token of the batch has a page behind it
        for e in planned:
            start = cache.length(e.id)
            assert cache.capacity(e.id) >= start + len(e.tokens)
            for g in range(len(cache.groups)):
                table = cache.table(e.id, g)
                for p in range(start, start + len(e.tokens)):
                    assert table[p // cache.page_size] >= 0
        log.append([(e.id, len(e.tokens), e.sample) for e in planned])
        if on_step:
            on_step(planned)
        sampled = [fake_token(e.id, cache.length(e.id) + len(e.tokens) - 1)
                   for e in planned if e.sample]
        sched.commit_step(sampled)
        cache.check_invariants()
        for c in sched.take_completed():
            done[c.id] = c
    assert not sched.has_work(), "scheduler did not finish"
    return done, log


def expected_tokens(rid, prompt_len, n):
    return [fake_token(rid, prompt_len - 1 + i) for i in range(n)]


def test_whole_prompt_then_decode_until_max_tokens():
    s, c = make()
    s.add_request("a", list(range(10)), SamplingParams(max_tokens=5))
    done, log = run(s, c)
    assert log[0] == [("a", 10, True)]
    assert all(step == [("a", 1, True)] for step in log[1:]) and len(log) == 5
    assert done["a"].reason == MAX_TOKENS
    assert done["a"].output_tokens == expected_tokens("a", 10, 5)
    assert c.free_pages() == 64 and c.free_slots() == 8


def test_prompt_is_cut_into_portions_by_budget_and_by_chunk_cap():
    s, c = make(max_batch_tokens=8)
    s.add_request("a", list(range(21)), SamplingParams(max_tokens=1))
    _, log = run(s, c)
    assert [st[0][1:] for st in log] == [(8, False), (8, False), (5, True)]
    s, c = make(max_batch_tokens=100, max_prefill_chunk=7)
    s.add_request("a", list(range(21)), SamplingParams(max_tokens=1))
    s.add_request("b", list(range(9)), SamplingParams(max_tokens=1))
    _, log = run(s, c)
    assert log[0] == [("a", 7, False), ("b", 7, False)]
    assert log[1] == [("a", 7, False), ("b", 2, True)]


def test_decodes_are_served_before_prompts():
    s, c = make(max_batch_tokens=6)
    s.add_request("a", [1, 2], SamplingParams(max_tokens=10))
    s.prepare_step(); s.commit_step([fake_token("a", 1)])      # a is decoding now
    s.add_request("b", list(range(20)), SamplingParams(max_tokens=1))
    planned = s.prepare_step()
    assert [(e.id, len(e.tokens)) for e in planned] == [("a", 1), ("b", 5)]
    # emission is in running order, the budget went to the decode first


def test_first_come_first_served_and_max_running():
    s, c = make(max_running=2)
    for rid in "abc":
        s.add_request(rid, [1, 2, 3], SamplingParams(max_tokens=2))
    done, log = run(s, c)
    assert [e[0] for e in log[0]] == ["a", "b"]
    first_c = next(i for i, st in enumerate(log) if any(e[0] == "c" for e in st))
    assert first_c >= 2          # c waits until one of a, b is finished
    assert set(done) == {"a", "b", "c"}


def test_stop_token_and_cancel_and_bad_requests():
    s, c = make()
    stop = fake_token("a", 4)
    s.add_request("a", [1, 2, 3], SamplingParams(max_tokens=50, stop_tokens=(stop,)))
    s.add_request("b", [1, 2, 3], SamplingParams(max_tokens=50))
    seen = []

    def on_step(planned):
        seen.append(1)
        if len(seen) == 2:
            s.cancel("b")
    done, _ = run(s, c, on_step=on_step)
    assert done["a"].reason == STOP_TOKEN and done["a"].output_tokens[-1] == stop
    assert done["a"].output_tokens == expected_tokens("a", 3, 3)
    assert done["b"].reason == CANCELLED and len(done["b"].output_tokens) == 2
    with pytest.raises(ValueError):
        s.add_request("x", [], SamplingParams())
    with pytest.raises(ValueError):
        s.add_request("y", [1], SamplingParams(max_tokens=0))


def test_too_long_and_never_fitting_requests_are_retired():
    s, c = make(pages=4, page=4, max_seq_len=32)
    s.add_request("long", list(range(40)), SamplingParams(max_tokens=1))      # > max_seq_len
    s.add_request("big", list(range(20)), SamplingParams(max_tokens=1))       # > the whole pool
    s.add_request("ok", list(range(5)), SamplingParams(max_tokens=2))
    done, _ = run(s, c)
    assert done["long"].reason == OUT_OF_MEMORY and done["big"].reason == OUT_OF_MEMORY
    assert done["ok"].reason == MAX_TOKENS and len(done["ok"].output_tokens) == 2


def test_admission_waits_instead_of_preempting():
    s, c = make(pages=4, page=4)
    s.add_request("a", list(range(12)), SamplingParams(max_tokens=2))     # 3 pages
    s.add_request("b", list(range(8)), SamplingParams(max_tokens=2))      # needs 2: must wait
    planned = s.prepare_step()
    assert [e.id for e in planned] == ["a"] and s.preemptions == 0
    assert [q.id for q in s.waiting] == ["b"] and not c.has("b")


def test_preemption_takes_the_newest_and_it_resumes_with_the_same_tokens():
    # 6 pages of 4: a (8 tokens) and b (8 tokens) fill 4 pages; growing forces a preemption
    s, c = make(pages=6, page=4)
    s.add_request("a", list(range(8)), SamplingParams(max_tokens=12))
    s.add_request("b", list(range(100, 108)), SamplingParams(max_tokens=12))
    victims = []
    orig = s._preempt

    def spy(index):
        victims.append(s.running[index].id)
        orig(index)
    s._preempt = spy
    done, log = run(s, c)
    assert s.preemptions >= 1 and victims[0] == "b"          # the most recently admitted
    assert done["a"].output_tokens == expected_tokens("a", 8, 12)
    assert done["b"].output_tokens == expected_tokens("b", 8, 12)   # same as without preemption
    # on re-admission b prefilled its prompt AND what it had generated
    resumed = [st for st in log if any(e[0] == "b" and e[1] > 8 for e in st)]
    assert resumed


def test_preempted_sequence_goes_to_the_front_of_the_queue():
    s, c = make(pages=6, page=4, max_running=2)
    s.add_request("a", list(range(8)), SamplingParams(max_tokens=16))
    s.add_request("b", list(range(8)), SamplingParams(max_tokens=16))
    s.add_request("z", [1, 2], SamplingParams(max_tokens=1))            # queued behind
    while s.preemptions == 0:
        planned = s.prepare_step()
        s.commit_step([fake_token(e.id, c.length(e.id) + len(e.tokens) - 1)
                       for e in planned if e.sample])
    assert [q.id for q in s.waiting][0] == "b"


def test_needy_newest_sequence_takes_from_the_next_newest():
    s, c = make(pages=5, page=4)
    s.add_request("a", list(range(6)), SamplingParams(max_tokens=30))     # 2 pages, full at 8
    s.add_request("b", list(range(11)), SamplingParams(max_tokens=30))    # 3 pages, full at 12
    s.prepare_step(); s.commit_step([5, 6])
    # b is the newest and needs a page first (position 12): a gives up its pages
    victims = []
    orig = s._preempt
    s._preempt = lambda i: (victims.append(s.running[i].id), orig(i))
    for _ in range(3):
        planned = s.prepare_step()
        s.commit_step([7] * sum(e.sample for e in planned))
    assert victims and victims[0] == "a"


def test_lone_sequence_that_cannot_grow_is_retired_out_of_memory():
    s, c = make(pages=2, page=4)
    s.add_request("a", list(range(6)), SamplingParams(max_tokens=100))
    done, _ = run(s, c)
    assert done["a"].reason == OUT_OF_MEMORY
    assert len(done["a"].output_tokens) == 3          # positions 6, 7 fit; the third has no page
    assert c.free_pages() == 2


def test_context_limit_retires_only_that_sequence():
    s, c = make(max_seq_len=10)
    s.add_request("a", list(range(7)), SamplingParams(max_tokens=100))
    s.add_request("b", [1, 2], SamplingParams(max_tokens=3))
    done, _ = run(s, c)
    assert done["a"].reason == CONTEXT_LIMIT and len(done["a"].output_tokens) == 4
    assert done["b"].reason == MAX_TOKENS


def test_row_seed_depends_on_position_not_on_batch():
    s, c = make()
    s.add_request("a", [1, 2, 3], SamplingParams(max_tokens=3, temperature=0.7, seed=99))
    e = s.prepare_step()[0]
    assert e.temperature == 0.7
    assert e.seed == 99 ^ ((0x9E3779B97F4A7C15 * 3) & ((1 << 64) - 1))
    s.commit_step([5])
    e2 = s.prepare_step()[0]
    assert e2.seed == 99 ^ ((0x9E3779B97F4A7C15 * 4) & ((1 << 64) - 1))


def test_penalty_history_masks_and_logprob_counts_of_a_row():
    """A row whose request has a penalty carries the distinct tokens generated so far with
    their counts, newest first (src/scheduler/scheduler.cc:617-645); under ``min_tokens``
    it carries its stop tokens to be masked (647-657); the count of alternatives is -1
    when log-probabilities are not wanted (659-664).  Prompt tokens are no history."""
    from inferx_b200.engine.scheduler import TokenLogprob
    s, c = make()
    s.add_request("a", [7, 7, 9], SamplingParams(max_tokens=8, repetition_penalty=1.3,
                                                presence_penalty=0.5, stop_tokens=(4, 2),
                                                min_tokens=2, want_logprobs=True,
                                                top_logprobs=50))
    s.add_request("b", [1, 2], SamplingParams(max_tokens=8))
    a, b = s.prepare_step()
    assert a.history == () and a.masked == (4, 2) and a.logprobs_k == 20
    assert b.history == () and b.masked == () and b.logprobs_k == -1
    assert (a.presence_penalty, a.repetition_penalty) == (0.0, 1.0)     # nothing generated yet
    deltas = s.commit_step([11, 3], [TokenLogprob(11, -0.5, [(11, -0.5)]), None])
    assert deltas[0].logprob.logprob == -0.5 and deltas[1].logprob is None
    for tok in (12, 11, 11):
        a, b = s.prepare_step()
        s.commit_step([tok, 3], [TokenLogprob(tok, -1.0, []), None])
    a, b = s.prepare_step()
    assert a.history == ((11, 3), (12, 1))            # newest first, counts of the whole run
    assert (a.presence_penalty, a.frequency_penalty, a.repetition_penalty) == (0.5, 0.0, 1.3)
    assert a.masked == ()                             # four generated: past min_tokens
    assert b.history == ()                            # no penalty asked: no history carried
    s.commit_step([4, 3], [TokenLogprob(4, -2.0, []), None])        # a's stop token
    done = {x.id: x for x in s.take_completed()}
    assert done["a"].reason == STOP_TOKEN and done["a"].output_tokens == [11, 12, 11, 11, 4]
    assert [lp.token for lp in done["a"].logprobs] == [11, 12, 11, 11, 4]
    with pytest.raises(ValueError):
        s.prepare_step()
        s.commit_step([3], [None, None])              # one record per sampled row
    with pytest.raises(ValueError):
        SamplingParams(repetition_penalty=0.0)
    with pytest.raises(ValueError):
        SamplingParams(min_tokens=-1)


def test_penalty_history_is_cut_to_the_newest_distinct_tokens():
    from inferx_b200.engine.scheduler import PENALTY_HISTORY_CAP
    s, c = make(pages=400, max_seq_len=2000)
    s.add_request("a", [1], SamplingParams(max_tokens=1000, frequency_penalty=0.1))
    n = PENALTY_HISTORY_CAP + 40
    for i in range(n):
        s.prepare_step()
        s.commit_step([100 + i])
    for _ in range(3):
        s.prepare_step()
        s.commit_step([100])                          # the oldest token, again
    (a,) = s.prepare_step()
    assert len(a.history) == PENALTY_HISTORY_CAP
    assert a.history[0] == (100, 4)                   # newest first, all four occurrences
    assert a.history[1] == (100 + n - 1, 1)
    assert (101, 1) not in a.history                  # the oldest distinct ones fell out


def test_commit_checks_the_number_of_samples():
    s, c = make()
    s.add_request("a", [1, 2, 3], SamplingParams())
    s.prepare_step()
    with pytest.raises(ValueError):
        s.commit_step([])


def test_windowed_groups_under_preemption_leave_nothing_behind():
    s, c = make(pages=8, page=4, windows=(0, 6))
    for i in range(5):
        s.add_request(i, list(range(3 + 5 * i)), SamplingParams(max_tokens=9))
    done, _ = run(s, c)
    assert len(done) == 5
    assert c.free_pages(0) == 8 and c.free_pages(1) == 8 and c.free_slots() == 8


def test_recorded_step_shapes_stay_bounded():
    """A serving run meets ever new (batch size, table width) shapes; the number of
    recorded steps kept must not grow with them.  The least recently used goes."""
    from inferx_b200.engine.executor import GraphCache
    cache = GraphCache(decode_graphs=5, prompt_graphs=2)
    recorded = 0
    for width in (8, 16, 32, 64):
        for batch in range(1, 40):
            key = (batch, (width,), tuple(range(batch)))
            for _ in range(3):
                if cache.get(key) is None and cache.should_record(key, True):
                    cache.put(key, object(), True)
                    recorded += 1
            assert cache.count(True) <= 5
    assert recorded == 4 * 39 and cache.evictions == recorded - 5 and len(cache) == 5
    # a shape is recorded at its second sighting (decode) or its third (prompts)
    fresh = GraphCache()
    assert not fresh.should_record("d", True) and fresh.should_record("d", True)
    assert [fresh.should_record("p", False) for _ in range(3)] == [False, False, True]
    # the one just used survives the next eviction
    lru = GraphCache(decode_graphs=2)
    lru.put("a", 1, True)
    lru.put("b", 2, True)
    assert lru.get("a") == 1
    lru.put("c", 3, True)
    assert lru.get("b") is None and lru.get("a") == 1 and lru.get("c") == 3
    # prompt shapes have a bound of their own and do not push decode shapes out
    for i in range(10):
        lru.put(((i, 5), (8,), ()), i, False)
    assert lru.count(False) == 4 and lru.count(True) == 2
