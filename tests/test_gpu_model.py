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


def test_grouped_query_heads_at_width(tmp_path):
    """Seven query heads per KV head, head size 128, top-8 routing (the shape family of
    the larger Qwen2-MoE checkpoints, scaled down in width): the tensor-core attention
    kernels pack the seven heads of a group into one tile."""
    d = mc.make_model_dir(GQA, tmp_path / "m", 4, dtype="bfloat16")
    reqs = mc.make_requests(GQA, [200, 75, 33], 4)
    ref = mc.reference_rows(d, reqs)
    bound = mc.bf16_bound(d, reqs)
    for kind in ("tail", "mixed"):
        steps = mc.TRACE_KINDS[kind](reqs)
        sess = ReplaySession(d, "bfloat16", traces.peak_tokens(steps), page_size=16, max_live=4,
                             use_graphs=(kind == "tail"))
        rows = mc.run_trace(sess, steps)
        worst = mc.compare(rows, ref, bound, f"gqa/{kind}")
        print(f"gqa/{kind}: worst relative error {worst:.3e} (bound {bound:.3e})")


def test_layer_sizes_of_the_benchmark_model(tmp_path):
    """Two layers at the widths the benchmark runs (hidden 2048, 16 heads of 128, 60
    experts of 1408, shared 5632, dense 5632, a 96-token window): the tuned kernels see
    their real shapes, prompt-sized and decode-sized, against the plain model."""
    d = mc.make_model_dir(MID, tmp_path / "m", 3, dtype="bfloat16")
    reqs = mc.make_requests(MID, [330, 150, 40], 3)
    ref = mc.reference_rows(d, reqs)
    bound = mc.bf16_bound(d, reqs)
    for kind in ("tail", "mixed"):
        steps = mc.TRACE_KINDS[kind](reqs)
        sess = ReplaySession(d, "bfloat16", traces.peak_tokens(steps), page_size=16, max_live=4,
                             use_graphs=True)
        rows = mc.run_trace(sess, steps)
        worst = mc.compare(rows, ref, bound, f"mid/{kind}")
        print(f"mid/{kind}: worst relative error {worst:.3e}")
