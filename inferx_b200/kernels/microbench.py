"""Kernel-level timings with achieved bandwidth or FLOP rate.

    python -m inferx_b200.kernels.microbench attn_decode --batch 8 --context 4096 [--form tma|mma|scalar]
    python -m inferx_b200.kernels.microbench grouped --tokens 8
    python -m inferx_b200.kernels.microbench dense --rows 8 --n 6144 --k 2048
    python -m inferx_b200.kernels.microbench attn_prefill --tokens 2048 [--form tc|mma]
    python -m inferx_b200.kernels.microbench attn_prefill --tokens 512 --context 8192 [--splits N]
    python -m inferx_b200.kernels.microbench router --tokens 2048
    python -m inferx_b200.kernels.microbench qkv --rows 8 [--separate]
    python -m inferx_b200.kernels.microbench grouped --tokens 2048

Each case runs one kernel face at Qwen1.5-MoE-A2.7B sizes (or the sizes given),
cycling through enough copies of its inputs that consecutive iterations do not
find them in the 126 MB L2, timed with CUDA events after warm-up.  One JSON line
per case: microseconds per call, bytes (or FLOP) per call by the algorithm, and the
achieved rate.  The reference's counterpart is its per-kernel bench harness
(bench/cuda_timer.h:1-40, bench/decode_step_bench.cc).
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import types

import torch

L2_BYTES = 126 << 20


EAGER = [False]   # --eager: no graph capture (for profilers that want plain launches)


def _time(fn, n_variants, iters, warmup=5):
    """Microseconds per call.  The calls are captured into one CUDA graph and the
    graph is replayed, so the host's launch cost does not hide a short kernel."""
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    if EAGER[0]:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(iters):
            fn(i % n_variants)
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) * 1e3 / iters
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i % n_variants)
    graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / iters


def _copies(bytes_per_copy):
    return max(2, int(math.ceil(2 * L2_BYTES / max(1, bytes_per_copy))))


def attn_decode(args):
    from . import ops
    B, C, heads, kvh, hd, page = args.batch, args.context, args.heads, args.kv_heads, \
        args.head_dim, args.page
    dt = torch.bfloat16
    pages_per_seq = -(-C // page)
    per_copy = B * pages_per_seq * page * kvh * hd * 2 * 2
    n = min(_copies(per_copy), 8)
    P = B * pages_per_seq
    kcs = [torch.randn(P, kvh, page, hd, device="cuda", dtype=dt) for _ in range(n)]
    vcs = [torch.randn(P, kvh, page, hd, device="cuda", dtype=dt) for _ in range(n)]
    bt = torch.randperm(P, device="cuda").to(torch.int32).view(B, pages_per_seq)
    q = torch.randn(B, heads, hd, device="cuda", dtype=dt)
    kv_len = torch.full((B,), C, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(hd)

    def fn(i):
        ops.paged_attention_decode(q, kcs[i], vcs[i], bt, kv_len, C, args.window, scale,
                                   splits=args.splits or None, kernel=args.form or None)
    us = _time(fn, n, args.iters)
    span = min(C, args.window) if args.window else C
    nbytes = B * span * kvh * hd * 2 * 2
    return {"case": "attn_decode", "batch": B, "context": C, "heads": heads, "kv_heads": kvh,
            "head_dim": hd, "splits": args.splits, "form": args.form or "auto", "us": round(us, 2), "bytes": nbytes,
            "GBps": round(nbytes / us / 1e3, 1)}


def grouped(args):
    from . import ops
    T, H, I, E, k = args.tokens, args.hidden, args.inter, args.experts, args.top_k
    dt = torch.bfloat16
    per_copy = E * 3 * I * H * 2
    n = _copies(per_copy)
    wgu = [torch.randn(E, 2 * I, H, device="cuda", dtype=dt) * 0.02 for _ in range(n)]
    wd = [torch.randn(E, H, I, device="cuda", dtype=dt) * 0.02 for _ in range(n)]
    x = torch.randn(T, H, device="cuda", dtype=dt)
    g = torch.Generator(device="cuda").manual_seed(0)
    idx = torch.stack([torch.randperm(E, device="cuda", generator=g)[:k] for _ in range(T)]
                      ).to(torch.int32)
    offsets, rows, dest = ops.moe_dispatch(idx, E)
    touched = int(torch.unique(idx).numel())
    act = ops.grouped_gate_up_swiglu(x, rows, offsets, wgu[0])

    def f1(i):
        ops.grouped_gate_up_swiglu(x, rows, offsets, wgu[i])

    def f2(i):
        ops.grouped_down(act, offsets, wd[i])
    us1 = _time(f1, n, args.iters)
    us2 = _time(f2, n, args.iters)
    b1, b2 = touched * 2 * I * H * 2, touched * I * H * 2
    fl1, fl2 = 2 * T * k * 2 * I * H, 2 * T * k * I * H
    return {"case": "grouped", "tokens": T, "experts_touched": touched,
            "gate_up_us": round(us1, 2), "gate_up_GBps": round(b1 / us1 / 1e3, 1),
            "gate_up_TFLOPs": round(fl1 / us1 / 1e6, 1),
            "down_us": round(us2, 2), "down_GBps": round(b2 / us2 / 1e3, 1),
            "down_TFLOPs": round(fl2 / us2 / 1e6, 1)}


def dense(args):
    from . import ops
    M, N, K = args.rows, args.n, args.k
    dt = torch.float32 if args.dtype == "float32" else torch.bfloat16
    n = _copies(N * K * 2)
    ws = [torch.randn(N, K, device="cuda", dtype=dt) * 0.02 for _ in range(n)]
    x = torch.randn(M, K, device="cuda", dtype=dt)

    def fn(i):
        if args.swiglu:
            ops.gate_up_swiglu(x, ws[i])
        else:
            ops.linear(x, ws[i])
    us = _time(fn, n, args.iters)
    nbytes = N * K * (4 if dt == torch.float32 else 2)
    return {"case": "dense", "rows": M, "n": N, "k": K, "swiglu": bool(args.swiglu),
            "dtype": args.dtype,
            "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
            "TFLOPs": round(2 * M * N * K / us / 1e6, 2)}


def qkv(args):
    """The QKV projection of a few-token step with bias, rotation and cache write: the one
    fused kernel, or (--separate) the product followed by the rotation kernel."""
    from . import ops
    T, H, heads, kvh, hd, page = args.rows, args.hidden, args.heads, args.kv_heads, args.head_dim, args.page
    dt = torch.bfloat16
    width = (heads + 2 * kvh) * hd
    n = _copies(width * H * 2)
    ws = [torch.randn(width, H, device="cuda", dtype=dt) * 0.02 for _ in range(n)]
    bias = torch.randn(width, device="cuda") * 0.1
    x = torch.randn(T, H, device="cuda", dtype=dt)
    positions = torch.arange(4000, 4000 + T, dtype=torch.int32, device="cuda")
    inv = (10000.0 ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().cuda()
    kc = torch.zeros(T + 1, kvh, page, hd, device="cuda", dtype=dt)
    vc = torch.zeros_like(kc)
    slots = (torch.arange(T, dtype=torch.int32, device="cuda") * page)
    ops.set_dependent_launch(True)

    def fused(i):
        ops.qkv_project_rope_append(x, ws[i], bias, positions, inv, hd, heads, kvh, hd, kc, vc, slots)

    def separate(i):
        ops.qkv_rope_append(ops.linear(x, ws[i]), bias, positions, inv, hd, heads, kvh, hd, kc, vc,
                            slots)
    us = _time(separate if args.separate else fused, n, args.iters)
    nbytes = width * H * 2
    return {"case": "qkv", "rows": T, "width": width, "k": H, "fused": not args.separate,
            "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}


def router(args):
    from . import ops
    T, H, E, k = args.tokens, args.hidden, args.experts, args.top_k
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, H, device="cuda", dtype=torch.float32) * 0.02
    extra = torch.randn(H, device="cuda", dtype=torch.float32) * 0.02

    def fn(i):
        ops.router_topk(x, w, k, False, 1.0, extra_w=extra)
    us = _time(fn, 1, args.iters)
    idx = ops.router_topk(x, w, k, False, 1.0, extra_w=extra)[1]

    def fd(i):
        ops.moe_dispatch(idx, E)
    return {"case": "router", "tokens": T, "router_us": round(us, 2),
            "dispatch_us": round(_time(fd, 1, args.iters), 2)}


def attn_prefill(args):
    from . import ops
    T, heads, kvh, hd, page = args.tokens, args.heads, args.kv_heads, args.head_dim, args.page
    dt = torch.float32 if args.dtype == "float32" else torch.bfloat16
    C = max(args.context if args.context_given else T, T)   # keys: the portion ends the context
    pages = -(-C // page)
    kc = torch.randn(pages, kvh, page, hd, device="cuda", dtype=dt)
    vc = torch.randn(pages, kvh, page, hd, device="cuda", dtype=dt)
    bt = torch.randperm(pages, device="cuda").to(torch.int32).view(1, pages)
    q = torch.randn(T, heads, hd, device="cuda", dtype=dt)
    step = types.SimpleNamespace(
        seq_of_token=torch.zeros(T, dtype=torch.int32, device="cuda"),
        positions=torch.arange(T, dtype=torch.int32, device="cuda"),
        cu_q=torch.tensor([0, T], dtype=torch.int32, device="cuda"),
        q_pos0=torch.full((1,), C - T, dtype=torch.int32, device="cuda"),
        kv_len=torch.full((1,), C, dtype=torch.int32, device="cuda"),
        max_q_len=T, max_kv_len=C, all_decode=False, num_seqs=1, num_tokens=T)
    scale = 1.0 / math.sqrt(hd)

    def fn(i):
        if args.form == "tiled":      # the CUDA-core kernel (any element type)
            ops.paged_attention_tiled(q, kc, vc, bt, step.cu_q, step.q_pos0, args.window, scale)
        else:
            ops.paged_attention_prefill(q, kc, vc, bt, step.cu_q, step.q_pos0, args.window, scale,
                                        kernel=args.form or None, splits=args.splits or None)
    us = _time(fn, 1, args.iters)
    flops = 4 * heads * hd * (T * T / 2 + T * (C - T))
    return {"case": "attn_prefill", "tokens": T, "context": C, "heads": heads, "head_dim": hd,
            "splits": args.splits or "auto",
            "form": args.form or "auto",
            "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=["attn_decode", "grouped", "dense", "attn_prefill", "router",
                                     "qkv"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--form", default="", help="attn_decode: tma, mma or scalar; attn_prefill: tc, mma or tiled (default: auto)")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=1408)
    ap.add_argument("--experts", type=int, default=60)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="dense, attn_prefill --form tiled: the element type")
    ap.add_argument("--separate", action="store_true",
                    help="qkv: the product and the rotation as two kernels")
    ap.add_argument("--eager", action="store_true", help="plain launches, no graph capture")
    args = ap.parse_args(argv)
    args.context_given = any(a == "--context" or a.startswith("--context=") for a in (argv or sys.argv[1:]))
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 3
    EAGER[0] = args.eager
    print(json.dumps(globals()[args.case](args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
