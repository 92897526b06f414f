"""The engine's host logic (cache manager, step function, replay) against the plain
model, on the CPU, with the kernels replaced by their plain statements
(tests/host_ops.py).  What this covers is bookkeeping: positions, slots, block
tables, page reuse, window release, batching.  The kernels themselves are compared
on the GPU (``-m gpu``)."""
import pytest
import torch

import host_ops
import model_cases as mc
import traces
from conftest import TINY_A, TINY_B, TINY_B_LISTED
from inferx_b200.engine.replay import ReplaySession

CASES = [("A", TINY_A, 0, [5, 9, 17, 40, 3, 70], 4), ("B", TINY_B, 1, [1, 6, 13, 31, 45, 80], 8),
         ("B-listed", TINY_B_LISTED, 2, [2, 29, 11, 52], 8)]


@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, name, cfg, seed, lengths, page, kind):
    d = mc.make_model_dir(cfg, tmp_path / "m", seed)
    reqs = mc.make_requests(cfg, lengths, seed)
    ref = mc.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, "float32", traces.peak_tokens(steps), page_size=page, max_live=4,
                         device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, steps)
    mc.compare(rows, ref, 2e-5, f"{name}/{kind}")
    if kind in ("whole", "tail", "portions"):
        assert len(rows) == sum(lengths)


def test_pool_too_small_is_reported(tmp_path):
    d = mc.make_model_dir(TINY_A, tmp_path / "m", 0)
    reqs = mc.make_requests(TINY_A, [200], 0)
    from inferx_b200.engine.replay import ReplayError
    sess = ReplaySession(d, "float32", 64, page_size=16, device="cpu", ops=host_ops)
    with pytest.raises(ReplayError, match="no page left"):
        mc.run_trace(sess, traces.whole(reqs))


def test_replayed_rows_are_tagged_with_request_and_position(tmp_path):
    import json
    from inferx_b200.engine.replay import run_stream
    d = mc.make_model_dir(TINY_A, tmp_path / "m", 0)
    reqs = mc.make_requests(TINY_A, [9, 4], 0)
    steps = traces.mixed(reqs, max_live=2, seed=1, decode_tail=3)
    sess = ReplaySession(d, "float32", traces.peak_tokens(steps), page_size=4, device="cpu",
                         ops=host_ops)
    out = tmp_path / "out"
    run_stream(sess, [json.dumps(s) for s in steps], str(out), index=True)
    pos = {}
    for st in steps:
        want = [(e["id"], pos.get(e["id"], 0) + w) for e in st["entries"] for w in e["want"]]
        for e in st["entries"]:
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
        path = out / f"{st['step']}.rows.json"
        if not want:
            assert not path.exists()
            continue
        tagged = json.loads(path.read_text())
        assert tagged["vocab"] == TINY_A["vocab_size"]
        assert [(r["id"], r["position"]) for r in tagged["rows"]] == want


def test_host_mirrors_of_a_step_are_shape_or_value(tmp_path):
    """What a part may read on the host: the step's shape always; the step's values
    (lengths, state slots, first live pages) only when the step is not recorded for
    replay, where they would be baked into the recording."""
    from inferx_b200.engine.executor import StepEntry
    d = mc.make_model_dir(TINY_B, tmp_path / "m", 1)
    sess = ReplaySession(d, "float32", 256, page_size=8, max_live=3, device="cpu", ops=host_ops)
    mgr, ex = sess.manager, sess.executor
    for rid, n in (("a", 30), ("b", 5)):
        mgr.open(rid)
        assert mgr.reserve(rid, n + 4)
        mgr.advance(rid, n)            # 'a' is 30 tokens in: its windowed group gave pages back
    entries = [StepEntry("a", [7], [0]), StepEntry("b", [1, 2, 3], [2])]
    lay = ex._layout(entries, bucket_tables=False)
    dev = ex._upload(lay)
    eager, _ = ex._context(dev, lay, static=False)
    assert eager.q_lens == [1, 3] and eager.kv_lens == [31, 8] and not eager.captured
    assert eager.state_slots == [mgr.slot("a"), mgr.slot("b")]
    assert eager.state_slot.tolist() == eager.state_slots
    windowed = [g for g in eager.groups if g.window > 0][0]
    assert windowed.first_live == [mgr.first_live("a", 1), 0] and windowed.first_live[0] >= 2
    recorded, _ = ex._context(dev, lay, static=True)
    assert recorded.captured and recorded.q_lens == [1, 3] and recorded.num_decode_seqs == 1
    assert recorded.kv_lens is None and recorded.state_slots is None
    assert all(g.first_live is None for g in recorded.groups)
    assert recorded.kv_len.tolist() == [31, 8]          # the device's copies are always there


def _check_penalised_generation(d, reqs, params, outs):
    """Every generated token against the plain model: the argmax (ties to the lower id) of
    the plain logits after the request's penalties over what it had generated so far and
    after masking its stop tokens under ``min_tokens``; and the reported log-probabilities
    against the plain ones of that same row."""
    import plain_qwen2_moe as plain
    pcfg, w = plain.read_model_folder(d)
    for toks, p, c in zip(reqs.values(), params, outs):
        lg = plain.forward(pcfg, w, list(toks) + c.output_tokens)
        scale = float(lg.abs().max())
        assert c.logprobs is None or len(c.logprobs) == len(c.output_tokens)
        for j, got in enumerate(c.output_tokens):
            generated = c.output_tokens[:j]
            masked = p.stop_tokens if j < p.min_tokens else ()
            row = plain.penalised(lg[len(toks) + j - 1], generated, p.presence_penalty,
                                  p.frequency_penalty, p.repetition_penalty, masked)
            want = plain.greedy(row)
            if got != want:        # level within the 32-bit bound, else a fault
                assert abs(float(row[got] - row[want])) <= 2e-5 * scale, (j, got, want)
            assert got not in masked
            if p.want_logprobs:
                lp = c.logprobs[j]
                ref_lp, ref_top = plain.logprobs(row, got, p.top_logprobs)
                assert lp.token == got and abs(lp.logprob - ref_lp) <= 1e-4
                assert len(lp.top) == p.top_logprobs
                for (t, v), (rt, rv) in zip(lp.top, ref_top):
                    assert abs(v - rv) <= 1e-4
                    assert t == rt or abs(float(row[t] - row[rt])) <= 2e-5 * scale


def penalty_workload(cfg):
    """Requests and sampling options for the penalty tests: greedy, so that every token
    can be checked against the plain model; one request per feature and one with all."""
    from inferx_b200 import SamplingParams
    reqs = mc.make_requests(cfg, [5, 9, 3, 14], 6)
    vocab = cfg["vocab_size"]
    stops = (vocab // 2, vocab // 3, 1)
    params = [SamplingParams(max_tokens=14, repetition_penalty=1.8),
              SamplingParams(max_tokens=14, presence_penalty=1.5, frequency_penalty=0.7,
                             want_logprobs=True, top_logprobs=3),
              SamplingParams(max_tokens=10, want_logprobs=True),
              SamplingParams(max_tokens=14, repetition_penalty=0.6, frequency_penalty=1.1,
                             presence_penalty=-0.4, stop_tokens=stops, min_tokens=14,
                             want_logprobs=True, top_logprobs=5)]
    return reqs, params


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B], ids=["A", "B"])
def test_penalties_min_tokens_and_logprobs_through_the_engine(tmp_path, cfg):
    from inferx_b200 import Engine, EngineConfig, Request
    d = mc.make_model_dir(cfg, tmp_path / "m", 9)
    reqs, params = penalty_workload(cfg)
    eng = Engine.create(EngineConfig(model=d, dtype="float32", device="cpu", block_size=4,
                                     num_gpu_blocks_override=64, max_num_seqs=3,
                                     prefill_chunk=4, max_model_len=64), ops=host_ops)
    outs = eng.generate([Request(t, p) for t, p in zip(reqs.values(), params)])
    assert [len(c.output_tokens) for c in outs] == [14, 14, 10, 14]
    assert outs[0].logprobs is None and outs[2].logprobs[0].top == []
    _check_penalised_generation(d, reqs, params, outs)
    # the penalties do something: without them some request generates other tokens
    bare = eng.generate([Request(t, type(p)(max_tokens=p.max_tokens))
                         for t, p in zip(reqs.values(), params)])
    assert any(a.output_tokens != b.output_tokens for a, b in zip(bare, outs))
