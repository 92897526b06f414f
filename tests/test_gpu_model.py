"""The engine on the GPU against the plain implementation: each request alone and
whole; most of it in one step and the last 32 tokens one by one; portions of
changing size; mixed batches with pages used again; in 32-bit and in bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import model_cases as mc
import plain_qwen2_moe as plain
import traces
from conftest import ROOT, TINY_A, TINY_B, TINY_B_LISTED
from inferx_b200.engine.replay import ReplaySession

pytestmark = pytest.mark.gpu

CASES = [("A", TINY_A, 0, [5, 9, 17, 40, 3, 70], 4), ("B", TINY_B, 1, [1, 6, 13, 31, 45, 80], 8),
         ("B-listed", TINY_B_LISTED, 2, [2, 29, 11, 52], 8)]
# Error bounds relative to the largest logit of the request: fp32 differs from the plain
# implementation only by summation order (2e-5); the bfloat16 bound is derived per model
# from what bfloat16 storage costs the plain model itself (model_cases.bf16_bound).



@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, dtype, name, cfg, seed, lengths, page, kind):
    store = "float32" if dtype == "float32" else "bfloat16"
    d = mc.make_model_dir(cfg, tmp_path / "m", seed, dtype=store)
    reqs = mc.make_requests(cfg, lengths, seed)
    ref = mc.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=page, max_live=4)
    rows = mc.run_trace(sess, steps)
    worst = mc.compare(rows, ref, mc.bound_for(dtype, d, reqs), f"{name}/{kind}/{dtype}")
    print(f"{name}/{kind}/{dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files and
    'done <step>' lines out."""
    cfg = TINY_B
    d = mc.make_model_dir(cfg, tmp_path / "m", 5, dtype="bfloat16")
    reqs = mc.make_requests(cfg, [70, 33, 20, 9, 50], 5)
    ref = mc.reference_rows(d, reqs)
    steps = traces.mixed(reqs, max_live=4, seed=1)
    out = tmp_path / "out"
    p = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(traces.peak_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    done = [ln for ln in p.stdout.splitlines() if ln.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    outs = []
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if n == 0:
            assert not path.exists()
            outs.append(None)
        else:
            outs.append(torch.from_numpy(
                np.fromfile(path, dtype="<f4").reshape(n, cfg["vocab_size"]).copy()))
    rows = traces.collect(steps, outs)
    mc.compare(rows, ref, mc.bound_for(dtype, d, reqs), f"trace_run/{dtype}")


def test_trace_run_answers_step_by_step(tmp_path):
    """The sender writes one step, waits for its 'done' line, then writes the next;
    the files of earlier steps are complete by then."""
    cfg = TINY_A
    d = mc.make_model_dir(cfg, tmp_path / "m", 2, dtype="bfloat16")
    reqs = mc.make_requests(cfg, [21, 8], 2)
    steps = traces.portions(reqs)
    out = tmp_path / "out"
    p = subprocess.Popen(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype",
         "float32", "--out", str(out), "--max-tokens", str(traces.peak_tokens(steps))],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, bufsize=1)
    try:
        for s in steps:
            if s is steps[0]:        # an entry without tokens runs nothing and holds nothing
                s = dict(s, entries=s["entries"] + [{"id": "idle", "tokens": [], "want": []}])
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            assert p.stdout.readline().strip() == f"done {s['step']}"
            n = sum(len(e["want"]) for e in s["entries"])
            if n:
                got = np.fromfile(out / f"{s['step']}.f32", dtype="<f4")
                assert got.size == n * cfg["vocab_size"] and np.isfinite(got).all()
        p.stdin.close()
        assert p.wait(timeout=120) == 0, p.stderr.read()[-2000:]
    finally:
        if p.poll() is None:
            p.kill()


MID = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 16,
    "num_key_value_heads": 16, "head_dim": 128, "num_experts": 60, "num_experts_per_tok": 4,
    "moe_intermediate_size": 1408, "shared_expert_intermediate_size": 5632,
    "intermediate_size": 5632, "decoder_sparse_step": 2, "mlp_only_layers": [],
    "norm_topk_prob": True, "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "use_sliding_window": True, "sliding_window": 96, "max_window_layers": 1,
    "tie_word_embeddings": False, "torch_dtype": "bfloat16",
}


GQA = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 1792, "num_attention_heads": 14,
    "num_key_value_heads": 2, "head_dim": 128, "num_experts": 16, "num_experts_per_tok": 8,
    "moe_intermediate_size": 320, "shared_expert_intermediate_size": 640,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "norm_topk_prob": False,
    "vocab_size": 777, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "use_sliding_window": False, "tie_word_embeddings": True, "torch_dtype": "bfloat16",
}


HD64 = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 160, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "num_experts": 6, "num_experts_per_tok": 2,
    "moe_intermediate_size": 264, "shared_expert_intermediate_size": 96,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "norm_topk_prob": True,
    "vocab_size": 500, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "use_sliding_window": True, "sliding_window": 70, "max_window_layers": 1,
    "tie_word_embeddings": True, "torch_dtype": "bfloat16",
}


def test_head_size_64_over_page_sizes(tmp_path):
    """Head size 64 with a 70-token window on the second layer, over the page sizes the
    TMA-fed kernels take (8, 32, 64) and one they do not (12, which falls to the cp.async
    forms): prompts longer than the window, decoded on, and mixed with page reuse.  Each
    against the plain model.  (Not against one another: the number of key splits follows
    the width of the block table, so page sizes differ by rounding.)"""
    d = mc.make_model_dir(HD64, tmp_path / "m", 6, dtype="bfloat16")
    reqs = mc.make_requests(HD64, [300, 130, 64, 9], 6)
    ref = mc.reference_rows(d, reqs)
    bound = mc.bf16_bound(d, reqs)
    for kind in ("tail", "mixed"):
        steps = mc.TRACE_KINDS[kind](reqs)
        for page in (8, 32, 64, 12):
            sess = ReplaySession(d, "bfloat16", traces.peak_tokens(steps), page_size=page,
                                 max_live=4, use_graphs=(kind == "tail"))
            rows = mc.run_trace(sess, steps)
            sess.executor.poll_errors()
            worst = mc.compare(rows, ref, bound, f"hd64/page{page}/{kind}")
            print(f"hd64/page{page}/{kind}: worst relative error {worst:.3e} (bound {bound:.3e})")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_grouped_query_heads_at_width(tmp_path, dtype):
    """Seven query heads per KV head, head size 128, top-8 routing (the shape family of
    the larger Qwen2-MoE checkpoints, scaled down in width): the tensor-core attention
    kernels pack the seven heads of a group into one tile; in 32-bit the split-KV kernel
    of the single-token steps is a different one from the tiny configurations'."""
    store = "float32" if dtype == "float32" else "bfloat16"
    d = mc.make_model_dir(GQA, tmp_path / "m", 4, dtype=store)
    reqs = mc.make_requests(GQA, [200, 75, 33], 4)
    ref = mc.reference_rows(d, reqs)
    bound = mc.bound_for(dtype, d, reqs)
    for kind in ("tail", "mixed"):
        steps = mc.TRACE_KINDS[kind](reqs)
        sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=16, max_live=4,
                             use_graphs=(kind == "tail"))
        rows = mc.run_trace(sess, steps)
        worst = mc.compare(rows, ref, bound, f"gqa/{kind}/{dtype}")
        print(f"gqa/{kind}/{dtype}: worst relative error {worst:.3e} (bound {bound:.3e})")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_layer_sizes_of_the_benchmark_model(tmp_path, dtype):
    """Two layers at the widths the benchmark runs (hidden 2048, 16 heads of 128, 60
    experts of 1408, shared 5632, dense 5632, a 96-token window): the tuned kernels see
    their real shapes, prompt-sized and decode-sized, against the plain model; in 32-bit
    through all four ways of cutting the same requests, at the 32-bit bound."""
    store = "float32" if dtype == "float32" else "bfloat16"
    d = mc.make_model_dir(MID, tmp_path / "m", 3, dtype=store)
    reqs = mc.make_requests(MID, [330, 150, 40], 3)
    ref = mc.reference_rows(d, reqs)
    bound = mc.bound_for(dtype, d, reqs)
    for kind in (("tail", "mixed") if dtype == "bfloat16" else tuple(mc.TRACE_KINDS)):
        steps = mc.TRACE_KINDS[kind](reqs)
        sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=16, max_live=4,
                             use_graphs=True)
        rows = mc.run_trace(sess, steps)
        worst = mc.compare(rows, ref, bound, f"mid/{kind}/{dtype}")
        print(f"mid/{kind}/{dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("graphs", [False, True])
def test_dependent_launch_changes_no_bit(tmp_path, graphs):
    """Decode steps of a few tokens are launched so that a kernel may come onto the device
    while its predecessor drains, and some kernels read what was written two launches back
    (the experts' row offsets) or ask for their first weights before they wait.  If one of
    them ever read something too early, a result would differ from the run without such
    launches; the two runs use the same kernels in the same order, so every logit must be
    the same bit for bit.  Four mixture layers at the benchmark's widths, 48 steps of four
    sequences, eagerly and from recorded steps."""
    from inferx_b200.kernels import ops
    cfg = dict(MID, num_hidden_layers=4, decoder_sparse_step=1, max_window_layers=2)
    d = mc.make_model_dir(cfg, tmp_path / "m", 5, dtype="bfloat16")
    new = 48
    reqs = mc.make_requests(cfg, [new + 41, new + 33, new + 20, new + 9], 5)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:len(t) - new], "want": [len(t) - new - 1]}
                                     for r, t in reqs.items()], "end": []}]
    for i in range(new):
        steps.append({"step": i + 1, "entries": [{"id": r, "tokens": [t[len(t) - new + i]],
                                                   "want": [0]} for r, t in reqs.items()],
                      "end": list(reqs) if i == new - 1 else []})

    def run():
        sess = ReplaySession(d, "bfloat16", traces.peak_tokens(steps), page_size=16, max_live=4,
                             use_graphs=graphs)
        return [sess.run_step(s).float().cpu() for s in steps]

    limit = ops.DEPENDENT_LAUNCH_MAX_TOKENS
    assert limit >= 4
    overlapped = run()
    try:
        ops.DEPENDENT_LAUNCH_MAX_TOKENS = 0
        plain_launches = run()
    finally:
        ops.DEPENDENT_LAUNCH_MAX_TOKENS = limit
    for i, (a, b) in enumerate(zip(overlapped, plain_launches)):
        assert torch.isfinite(a).all()
        assert torch.equal(a, b), f"step {i}: dependent launches changed a logit"


LONG = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 1024, "num_attention_heads": 8,
    "num_key_value_heads": 2, "head_dim": 128, "num_experts": 8, "num_experts_per_tok": 2,
    "moe_intermediate_size": 128, "shared_expert_intermediate_size": 256,
    "decoder_sparse_step": 1, "mlp_only_layers": [], "norm_topk_prob": True,
    "vocab_size": 300, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "use_sliding_window": True, "sliding_window": 3000, "max_window_layers": 1,
    "tie_word_embeddings": True, "torch_dtype": "bfloat16",
}


def far_key_stands_out(name, t):
    """With some 8,000 random keys every attention weight is about 1/8,000 and a kernel
    that skipped a run of keys would hardly move the logits; sharper queries and keys
    let single far keys carry weight."""
    if name.endswith(("q_proj.weight", "k_proj.weight")):
        return t * 2.5
    if name.endswith("mlp.gate.weight"):
        return t * 2.0
    return t


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_long_context_inside_a_trace(tmp_path, dtype):
    """Contexts at which both attention kernels cut a query's keys into runs that are
    merged afterwards (a 512-token portion after 4,096 cached tokens; single tokens
    beyond 8,192), inside a replayed trace with a second request decoding beside the
    long one, one layer with all keys and one with a 3,000-token window whose pages are
    given back as it moves: against the plain model's one pass over the whole
    sequence."""
    from inferx_b200.weights.random_model import write_random_model
    store = "float32" if dtype == "float32" else "bfloat16"
    d = str(tmp_path / "m")
    write_random_model(LONG, d, seed=12, dtype=store, adjust=far_key_stands_out)
    reqs = mc.make_requests(LONG, [8260, 90], 12)
    big, small = reqs["r0"], reqs["r1"]
    cfg, w = plain.read_model_folder(d)
    ref_big = plain.forward(cfg, w, big)
    ref_small = plain.forward(cfg, w, small)
    ref = {("r0", p): ref_big[p] for p in range(len(big))}
    ref.update({("r1", p): ref_small[p] for p in range(len(small))})
    steps = [
        {"entries": [{"id": "r0", "tokens": big[:4096], "want": [0, 2047, 4095]}]},
        {"entries": [{"id": "r0", "tokens": big[4096:4608], "want": [0, 255, 511]},
                     {"id": "r1", "tokens": small[:40], "want": [39]}]},
        {"entries": [{"id": "r0", "tokens": big[4608:8200], "want": [0, 3591]},
                     {"id": "r1", "tokens": [small[40]], "want": [0]}]},
    ]
    for i in range(60):     # single tokens at 8,200 and beyond, beside the short request
        entries = [{"id": "r0", "tokens": [big[8200 + i]], "want": [0]}]
        if 41 + i < len(small):
            entries.append({"id": "r1", "tokens": [small[41 + i]], "want": [0]})
        steps.append({"entries": entries})
    for n, st in enumerate(steps):
        st["step"] = n
        st.setdefault("end", [])
    steps[-1]["end"] = ["r0"]
    steps[3 + len(small) - 42]["end"] = ["r1"]     # the step that brings r1's last token
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=16, max_live=2,
                         use_graphs=True)
    outs = []
    for st in steps:
        lg = sess.run_step(st)
        outs.append(None if lg is None else lg.detach().float().cpu())
    sess.executor.poll_errors()
    sess.manager.check_invariants()
    rows = traces.collect(steps, outs)
    if dtype == "float32":
        bound = 2e-5
    else:
        a = plain.forward(cfg, w, big[:2100], plain.round_bf16)
        bound = max(5e-3, 3.0 * float((a - ref_big[:2100]).abs().max()) / float(ref_big.abs().max()))
    worst = mc.compare(rows, ref, bound, f"long/{dtype}")
    print(f"long/{dtype}: worst relative error {worst:.3e} (bound {bound:.3e})")
