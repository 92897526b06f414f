"""Times this repository's kernels at the shapes reference_kernel_times.cu times the
reference's own kernels at (the benchmark model's sizes; 8 tokens and 2048 tokens).

Each call is recorded ten times into one CUDA graph, so that the host's share of a launch is
not part of the figure; the graph is replayed twice untimed and then nine times between CUDA
events, and the median, divided by ten, is printed, one JSON object a line.  Where a kernel
here does more than its counterpart (the gather and SwiGLU in the gate/up product, the router
product before the choice, the residual sum before the norm) the name says so.

    python tests/golden/kernel_times.py
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from inferx_b200.kernels import ops  # noqa: E402

E, H, I, TOP_K = 60, 2048, 1408, 4
CALLS = 10


def time_us(call) -> float:
    call()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(CALLS):
            call()
    times = []
    for i in range(11):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(a.elapsed_time(b) * 1000 / CALLS)
    times.sort()
    return times[len(times) // 2]


def report(name: str, us: float) -> None:
    print(json.dumps({"kernel": name, "us": round(us, 1)}), flush=True)


def main() -> None:
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)

    def rand(*shape, scale=1.0, dtype=torch.bfloat16):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(dtype)

    w_gate_up, w_down = rand(E, 2 * I, H, scale=0.05), rand(E, H, I, scale=0.05)
    for tokens in (8, 2048):
        experts = (torch.arange(tokens * TOP_K, device=dev) * 7 % E).int().view(tokens, TOP_K)
        offsets, rows, _ = ops.moe_dispatch(experts, E)
        x = rand(tokens, H)
        act = ops.grouped_gate_up_swiglu(x, rows, offsets, w_gate_up)
        report(f"grouped_gate_up_t{tokens} (with gather and SwiGLU)",
               time_us(lambda: ops.grouped_gate_up_swiglu(x, rows, offsets, w_gate_up)))
        report(f"grouped_down_t{tokens}", time_us(lambda: ops.grouped_down(act, offsets, w_down)))
    for tokens in (8, 2048):
        x, w_router = rand(tokens, H), rand(E, H, scale=0.05, dtype=torch.float32)
        report(f"route_topk_t{tokens} (with the router product)",
               time_us(lambda: ops.router_topk(x, w_router, TOP_K, False, 1.0)))
    for tokens in (8, 2048):
        resid, delta = rand(tokens, H, dtype=torch.float32), rand(tokens, H)
        gain = torch.ones(H, device=dev)
        report(f"rmsnorm_t{tokens} (with the residual sum)",
               time_us(lambda: ops.add_rmsnorm(resid, delta, gain, 1e-6, torch.bfloat16)))
    seqs, context, page, heads, head_dim = 8, 4096, 16, 16, 128
    pages = seqs * context // page
    k_cache, v_cache = rand(pages, heads, page, head_dim), rand(pages, heads, page, head_dim)
    table = torch.arange(pages, device=dev, dtype=torch.int32).view(seqs, context // page)
    kv_len = torch.full((seqs,), context, device=dev, dtype=torch.int32)
    q = rand(seqs, heads, head_dim)
    report("paged_attention_decode_b8_ctx4096",
           time_us(lambda: ops.paged_attention_decode(q, k_cache, v_cache, table, kv_len,
                                                      context, 0, head_dim ** -0.5)))
    logits = rand(8, 151936, scale=4.0, dtype=torch.float32)
    report("argmax_b8_vocab151936", time_us(lambda: ops.sample(logits)))


if __name__ == "__main__":
    main()
