"""The engine as a whole on the GPU: long decoding (with CUDA graphs), the first
tokens of a sequence, greedy generation through the Python entry point and the
command line, temperature sampling, preemption."""
import json
import os
import subprocess
import sys

import pytest
import torch

import model_cases as mc
import plain_qwen2_moe as plain
import traces
from conftest import ROOT, TINY_A, TINY_B
from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
from inferx_b200.engine.replay import ReplaySession

pytestmark = pytest.mark.gpu



@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg,seed,page", [(TINY_A, 0, 4), (TINY_B, 1, 8)])
def test_long_decoding_with_graphs(tmp_path, dtype, cfg, seed, page):
    """300 tokens one by one after a short prompt: the block table grows through
    several captured widths, windows slide over many pages."""
    d = mc.make_model_dir(cfg, tmp_path / "m", seed,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = mc.make_requests(cfg, [330], seed)
    ref = mc.reference_rows(d, reqs)
    steps = traces.tail_decode(reqs, 300)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=page, use_graphs=True)
    rows = mc.run_trace(sess, steps)
    assert len(rows) == 330
    assert sess.executor.graph_replays >= 290 and len(sess.executor._graphs) >= 3
    mc.compare(rows, ref, mc.bound_for(dtype, d, reqs), f"long decode {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_prompt_shapes_are_captured_too(tmp_path, dtype):
    """Six prompts of the same length (and a decoding neighbour from the second one on):
    from its third occurrence a prompt-carrying shape replays a CUDA graph, and every
    row still matches the plain model."""
    cfg = TINY_B
    d = mc.make_model_dir(cfg, tmp_path / "m", 4,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = mc.make_requests(cfg, [40] * 6 + [12], 7)
    ref = mc.reference_rows(d, reqs)
    long = reqs["r6"]
    steps = [{"step": 0, "entries": [{"id": "r6", "tokens": long[:5], "want": [4]}], "end": []}]
    for i in range(6):
        steps.append({"step": i + 1, "entries": [
            {"id": f"r{i}", "tokens": reqs[f"r{i}"], "want": [0, 39]},
            {"id": "r6", "tokens": [long[5 + i]], "want": [0]}],
            "end": [f"r{i}"] + (["r6"] if i == 5 else [])})
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=8, max_live=2,
                         use_graphs=True)
    rows = mc.run_trace(sess, steps)
    assert len(rows) == 1 + 6 * 3
    ex = sess.executor
    assert ex.graph_replays >= 4 and ex._graphs.count(False) >= 1
    mc.compare(rows, ref, mc.bound_for(dtype, d, reqs), f"prompt graphs {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tmp_path, dtype):
    """Positions 0, 1, 2: one-token prompts, a batch of first tokens, two-token portions."""
    cfg = TINY_B
    d = mc.make_model_dir(cfg, tmp_path / "m", 2,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = mc.make_requests(cfg, [1, 2, 3, 4], 9)
    ref = mc.reference_rows(d, reqs)
    steps = [
        {"step": 0, "entries": [{"id": r, "tokens": t[:1], "want": [0]} for r, t in reqs.items()],
         "end": ["r0"]},
        {"step": 1, "entries": [{"id": r, "tokens": reqs[r][1:3], "want": list(range(len(reqs[r][1:3])))}
                                for r in ("r1", "r2", "r3")], "end": ["r1", "r2"]},
        {"step": 2, "entries": [{"id": "r3", "tokens": reqs["r3"][3:], "want": [0]}], "end": ["r3"]},
    ]
    sess = ReplaySession(d, dtype, 256, page_size=8)
    rows = mc.run_trace(sess, steps)
    assert len(rows) == 10
    mc.compare(rows, ref, mc.bound_for(dtype, d, reqs), f"first tokens {dtype}")


def _plain_greedy(d, prompt, n):
    cfg, w = plain.read_model_folder(d)
    seq, out = list(prompt), []
    for _ in range(n):
        t = plain.greedy(plain.forward(cfg, w, seq)[-1])
        out.append(t)
        seq.append(t)
    return out


def _check_greedy_choices(d, prompt, tokens, rel):
    """Every generated token is (within the error bound) the plain model's best
    continuation of the tokens before it."""
    cfg, w = plain.read_model_folder(d)
    lg = plain.forward(cfg, w, list(prompt) + list(tokens))
    scale = float(lg.abs().max())
    for i, tok in enumerate(tokens):
        row = lg[len(prompt) - 1 + i]
        assert float(row.max() - row[tok]) <= 2 * rel * scale, (i, tok, int(row.argmax()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("eager", [False, True])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype, eager):
    cfg = TINY_B
    d = mc.make_model_dir(cfg, tmp_path / "m", 1,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = mc.make_requests(cfg, [1, 6, 13, 31], 1)
    eng = Engine.create(EngineConfig(model=d, dtype=dtype, block_size=8, max_num_seqs=4,
                                     num_gpu_blocks_override=10, prefill_chunk=7,
                                     max_model_len=64, enforce_eager=eager))
    outs = eng.generate([Request(t, SamplingParams(max_tokens=12)) for t in reqs.values()])
    assert eng.stats()["preemptions"] >= 1          # 10 pages of 8 do not hold 4 x 43 tokens
    assert all(c.reason == "max_tokens" and len(c.output_tokens) == 12 for c in outs)
    for toks, c in zip(reqs.values(), outs):
        if dtype == "float32":
            assert c.output_tokens == _plain_greedy(d, toks, 12)
        else:
            _check_greedy_choices(d, toks, c.output_tokens, mc.bf16_bound(d, {"r": list(toks) + c.output_tokens}))
    eng.runtime.manager.check_invariants()
    assert eng.stats()["pages_free"] == eng.stats()["pages_total"]


def test_preemption_does_not_change_greedy_output(tmp_path):
    cfg = TINY_A
    d = mc.make_model_dir(cfg, tmp_path / "m", 0)
    reqs = mc.make_requests(cfg, [5, 9, 17], 0)

    def run(pages):
        eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=4, max_num_seqs=3,
                                         num_gpu_blocks_override=pages, max_model_len=64))
        outs = eng.generate([Request(t, SamplingParams(max_tokens=8)) for t in reqs.values()])
        return [c.output_tokens for c in outs], eng.stats()["preemptions"]
    roomy, p0 = run(64)
    tight, p1 = run(6)
    assert p0 == 0 and p1 >= 1 and roomy == tight


def test_temperature_sampling_is_seeded_and_varied(tmp_path):
    cfg = TINY_B
    d = mc.make_model_dir(cfg, tmp_path / "m", 1)
    prompt = mc.make_requests(cfg, [13], 4)["r0"]

    def run(seed, temperature=0.7, **kw):
        eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=8,
                                         num_gpu_blocks_override=16, max_model_len=64))
        return eng.generate([Request(prompt, SamplingParams(
            max_tokens=12, temperature=temperature, seed=seed, **kw))])[0].output_tokens
    a, b, c = run(7), run(7), run(8)
    assert a == b and a != c
    assert run(7, top_k=1) == _plain_greedy(d, prompt, 12)
    # with a batch around it the draw is the same: the seed depends on the position only
    eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=8,
                                     num_gpu_blocks_override=32, max_model_len=64))
    outs = eng.generate([Request([1, 2, 3], SamplingParams(max_tokens=5)),
                         Request(prompt, SamplingParams(max_tokens=12, temperature=0.7, seed=7))])
    assert outs[1].output_tokens == a


def test_temperature_workload_draws_what_the_plain_sampler_draws(tmp_path):
    """Four requests with prompts of 1, 6, 13 and 31 tokens, portions of 7, pages of 8,
    12 tokens each at temperature 0.7, each request with a seed of its own, in 32-bit:
    every token the engine drew is the one the plain sampler draws from the plain
    model's logits with the row's seed (seed ^ golden * tokens so far,
    src/scheduler/scheduler.cc:613-615).  A draw may differ only where the uniform
    number falls on the edge between two tokens' shares, within rounding."""
    cfg = TINY_B
    d = mc.make_model_dir(cfg, tmp_path / "m", 1)
    reqs = mc.make_requests(cfg, [1, 6, 13, 31], 1)
    eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=8, max_num_seqs=4,
                                     num_gpu_blocks_override=40, prefill_chunk=7,
                                     max_model_len=64))
    seeds = [11, 22, 33, 44]
    outs = eng.generate([Request(t, SamplingParams(max_tokens=12, temperature=0.7, seed=sd))
                         for t, sd in zip(reqs.values(), seeds)])
    pcfg, w = plain.read_model_folder(d)
    mask = (1 << 64) - 1
    on_edge = 0
    for toks, sd, c in zip(reqs.values(), seeds, outs):
        assert len(c.output_tokens) == 12
        seq = list(toks)
        lg = plain.forward(pcfg, w, seq + c.output_tokens)
        for j, got in enumerate(c.output_tokens):
            n_before = len(toks) + j
            row_seed = (sd ^ ((0x9E3779B97F4A7C15 * n_before) & mask)) & mask
            want, cdf, target = plain.sample_temperature(lg[n_before - 1], 0.7, row_seed)
            if got != want:
                # only on an edge: the target within 1e-5 of the total of the boundary
                edge = min(abs(float(cdf[min(got, want)]) - target),
                           abs(float(cdf[max(got, want) - 1]) - target))
                assert abs(got - want) == 1 and edge <= 1e-5 * float(cdf[-1]), (j, got, want)
                on_edge += 1
    assert on_edge <= 1
    assert len({tuple(c.output_tokens) for c in outs}) == 4


@pytest.mark.parametrize("dtype,graphs", [("float32", True), ("float32", False),
                                          ("bfloat16", True)])
def test_penalties_min_tokens_and_logprobs(tmp_path, dtype, graphs):
    """Greedy generation with repetition, presence and frequency penalties, stop tokens
    masked under min_tokens and log-probabilities reported, against the plain model token
    by token (32-bit), portions of prompts beside decoding rows, recorded steps or not.
    In bfloat16 the same run must finish, never choose a masked token, and report
    log-probabilities that are those of its own tokens (at most 0, the chosen one among
    the alternatives when it is the most probable)."""
    from test_engine_on_host_double import _check_penalised_generation, penalty_workload
    cfg = TINY_B
    d = mc.make_model_dir(cfg, tmp_path / "m", 9,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs, params = penalty_workload(cfg)
    eng = Engine.create(EngineConfig(model=d, dtype=dtype, block_size=4,
                                     num_gpu_blocks_override=64, max_num_seqs=3,
                                     prefill_chunk=4, max_model_len=64,
                                     enforce_eager=not graphs))
    outs = eng.generate([Request(t, p) for t, p in zip(reqs.values(), params)])
    assert [len(c.output_tokens) for c in outs] == [14, 14, 10, 14]
    if dtype == "float32":
        _check_penalised_generation(d, reqs, params, outs)
    for p, c in zip(params, outs):
        assert not set(c.output_tokens[:p.min_tokens]) & set(p.stop_tokens)
        if p.want_logprobs:
            for tok, lp in zip(c.output_tokens, c.logprobs):
                assert lp.token == tok and lp.logprob <= 1e-6 and len(lp.top) == p.top_logprobs
                if lp.top:
                    assert lp.top[0][1] >= lp.logprob - 1e-6
                    assert all(a[1] >= b[1] for a, b in zip(lp.top, lp.top[1:]))
        else:
            assert c.logprobs is None


def test_rounds_of_wandering_requests_leave_nothing_behind(tmp_path):
    """Three rounds of 24 requests with prompts of wandering lengths and every sampling
    option in some of them, through one engine whose pool forces preemptions: every request
    gets exactly its tokens, every page is free again after a round, the recorded step
    shapes stay within their bounds (old ones are dropped), and the memory the process
    holds stops growing after the first round."""
    cfg = dict(TINY_B, num_hidden_layers=3)
    d = mc.make_model_dir(cfg, tmp_path / "m", 3, dtype="bfloat16")
    eng = Engine.create(EngineConfig(model=d, dtype="bfloat16", block_size=8, max_num_seqs=12,
                                     num_gpu_blocks_override=90, prefill_chunk=32,
                                     max_num_batched_tokens=96, max_model_len=400))
    vocab = cfg["vocab_size"]
    reserved = []
    for rnd in range(3):
        g = torch.Generator().manual_seed(50 + rnd)
        lens = torch.randint(1, 200, (24,), generator=g).tolist()
        prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
        params = [SamplingParams(max_tokens=int(torch.randint(1, 60, (1,), generator=g)),
                                 ignore_eos=True, temperature=0.8 if i % 3 == 0 else 0.0, seed=i,
                                 top_k=7 if i % 6 == 0 else 0, top_p=0.9 if i % 7 == 0 else 1.0,
                                 repetition_penalty=1.2 if i % 4 == 0 else 1.0,
                                 presence_penalty=0.3 if i % 8 == 0 else 0.0,
                                 want_logprobs=i % 5 == 0, top_logprobs=2) for i in range(24)]
        outs = eng.generate([Request(p, q) for p, q in zip(prompts, params)])
        torch.cuda.synchronize()
        st = eng.stats()
        assert [len(c.output_tokens) for c in outs] == [q.max_tokens for q in params]
        assert all((c.logprobs is not None) == q.want_logprobs for c, q in zip(outs, params))
        assert st["pages_free"] == st["pages_total"] and st["running"] == st["waiting"] == 0
        eng.runtime.manager.check_invariants()
        graphs = eng.runtime.executor._graphs
        assert graphs.count(True) <= graphs.limits[True] and graphs.count(False) <= graphs.limits[False]
        reserved.append(torch.cuda.memory_reserved())
    assert eng.stats()["preemptions"] >= 1 and eng.stats()["graph_replays"] > 100
    assert reserved[2] <= reserved[0] + (64 << 20), reserved


def test_a_wait_that_ran_out_is_reported(tmp_path):
    """Kernels with bounded waits write a code into a status word instead of hanging.
    The word is written from the host here (no kernel is made to wait): reading it must
    raise and name the kernel and the role, the word must be cleared, and generation must
    surface the error rather than return tokens computed from an invalid step."""
    from inferx_b200.kernels import ops
    st = ops._tc_status(torch.device("cuda:0"))
    st.fill_(22)
    with pytest.raises(ops.KernelError, match=r"paged_attention_prefill \(tcgen05 form\): the MMA "
                                              r"issuer waited past its limit \(status 22\)"):
        ops.check_async_errors()
    assert int(st.item()) == 0
    ops.check_async_errors()            # cleared: nothing to report
    d = mc.make_model_dir(TINY_A, tmp_path / "m", 0)
    eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=4,
                                     num_gpu_blocks_override=16, max_model_len=32))
    st.fill_(2)
    with pytest.raises(ops.KernelError, match="grouped_gemm_tc: the MMA issuer"):
        eng.generate([Request([1, 2, 3], SamplingParams(max_tokens=2))])
    assert int(st.item()) == 0


def test_a_step_that_fails_while_recorded_reports_itself_and_leaves_the_executor_usable(tmp_path):
    """A decode shape is recorded into a CUDA graph the second time it is seen.  If the
    model's forward pass raises during that recording, the caller gets that error (not one
    about a capture left open), the stream is out of capture mode, and the same executor
    goes on: eagerly at once, and recording the shape the next time."""
    cfg = TINY_A
    d = mc.make_model_dir(cfg, tmp_path / "m", 2, dtype="float32")
    reqs = mc.make_requests(cfg, [30], 3)
    ref = mc.reference_rows(d, reqs)
    toks = reqs["r0"]
    sess = ReplaySession(d, "float32", 64, page_size=8, max_live=1, use_graphs=True)
    ex = sess.executor
    rows = {}

    def feed(i, lo, hi):
        out = sess.run_step({"step": i, "entries": [{"id": "r0", "tokens": toks[lo:hi],
                                                     "want": [hi - lo - 1]}], "end": []})
        rows[("r0", hi - 1)] = out[0].float().cpu()

    feed(0, 0, 20)
    feed(1, 20, 21)                      # the decode shape's first sighting: eager
    orig = ex.model.forward

    def failing(ctx, caches, logit_rows):
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("this part cannot be recorded")
        return orig(ctx, caches, logit_rows)

    ex.model.forward = failing
    captures = ex.graph_captures
    with pytest.raises(RuntimeError, match="this part cannot be recorded"):
        feed(2, 21, 22)                  # second sighting: recorded, and fails there
    assert not torch.cuda.is_current_stream_capturing()
    assert ex.graph_captures == captures and len(ex._graphs) == 0
    ex.model.forward = orig
    torch.zeros(4, device="cuda").sum().item()          # the device takes ordinary work
    for i in range(22, 30):              # the token that failed was not committed: again
        feed(i, i - 1, i)
    assert ex.graph_captures == captures + 1 and ex.graph_replays >= 6
    mc.compare(rows, ref, mc.bound_for("float32", d, reqs), "after a failed recording")


def test_command_line(tmp_path):
    cfg = dict(TINY_A, eos_token_id=5)
    d = mc.make_model_dir(cfg, tmp_path / "m", 0)
    p = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "inferx-generate"), d, "--dtype", "fp32",
         "--block-size", "4", "--max-model-len", "64", "--max-num-seqs", "2",
         "--num-gpu-blocks-override", "32", "--prompt-ids", "5,17,3,200,41",
         "--prompt-ids", "9 8 7", "--max-tokens", "6", "--ignore-eos", "--log-level", "warning"],
        capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [json.loads(ln) for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert [l["index"] for l in lines] == [0, 1]
    assert lines[0]["output_ids"] == _plain_greedy(d, [5, 17, 3, 200, 41], 6)
    assert lines[1]["output_ids"] == _plain_greedy(d, [9, 8, 7], 6)
    assert lines[0]["finish_reason"] == "max_tokens"
    assert "logprobs" not in lines[0]
    # the sampling options beyond temperature: penalties, min-tokens, log-probabilities
    p = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "inferx-generate"), d, "--dtype", "fp32",
         "--block-size", "4", "--max-model-len", "64", "--num-gpu-blocks-override", "32",
         "--prompt-ids", "9 8 7", "--max-tokens", "5", "--repetition-penalty", "1.5",
         "--presence-penalty", "0.3", "--frequency-penalty", "0.2", "--min-tokens", "5",
         "--stop-token-ids", "5,6", "--logprobs", "2", "--log-json", "--log-file",
         str(tmp_path / "run.log"), "--kv-blocks", "32", "--no-cuda-graphs"],
        capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    logged = [json.loads(ln) for ln in (tmp_path / "run.log").read_text().splitlines()]
    assert [r["level"] for r in logged] == ["info", "info"] and logged[1]["steps"] >= 5
    assert logged[1]["graph_replays"] == 0            # --no-cuda-graphs
    (line,) = [json.loads(ln) for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert len(line["output_ids"]) == 5 and not set(line["output_ids"]) & {5, 6}
    assert [lp["token"] for lp in line["logprobs"]] == line["output_ids"]
    assert all(len(lp["top"]) == 2 and lp["logprob"] <= 0 for lp in line["logprobs"])
