#!/usr/bin/env python3
"""Decode and prefill throughput at Qwen1.5-MoE-A2.7B sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096]
                    [--layers L] [--sizes a2.7b|57b-a14b] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second of the default run:
random weights at the A2.7B layer sizes, batch 8, context 4096, bfloat16, timed on
the device with CUDA events over exactly K decode steps after W warm-up steps.
``e2e`` is the same through ``Engine.step`` (host token ids in through pinned
memory, sampled ids back to the host every step).  ``prefill`` is one 2,048-token
prompt in one step; ``points`` holds decode at batch 1 and 64 and one step that
carries a 2,048-token prompt portion beside the decoding requests; ``roofline`` is the
bytes a decode step has to read (every weight it uses once, and the cache of the
live requests) over its time, against the measured copy bandwidth.

``--sizes 57b-a14b`` runs the same measurements at the Qwen2-57B-A14B layer sizes
(context 32768, the wide point at batch 32 and the longest context that fits).

A decode step's working set (gigabytes of weights and cache) is far larger than the
126 MB L2, so nothing stays resident between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 16,
    "num_key_value_heads": 16, "head_dim": 128, "num_experts": 60, "num_experts_per_tok": 4,
    "moe_intermediate_size": 1408, "shared_expert_intermediate_size": 5632,
    "intermediate_size": 5632, "decoder_sparse_step": 1, "mlp_only_layers": [],
    "norm_topk_prob": False, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "use_sliding_window": False, "tie_word_embeddings": False,
    "torch_dtype": "bfloat16",
}
FULL_LAYERS = 24
METRIC = "decode tok/s at batch 8, context 4096 (Qwen1.5-MoE-A2.7B sizes)"

# The larger configuration of the same architecture (about 115 GB of bf16 weights);
# `--sizes 57b-a14b` measures it: decode at context 32768, and a 2,048-token prompt
# portion beside the decoding requests in one step.
Q57B = dict(A27B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
            num_key_value_heads=4, num_experts=64, num_experts_per_tok=8,
            moe_intermediate_size=2560, shared_expert_intermediate_size=20480,
            intermediate_size=18944)
SIZES = {
    "a2.7b": {"cfg": A27B, "name": "Qwen1.5-MoE-A2.7B sizes", "context": 4096, "big_batch": 64},
    "57b-a14b": {"cfg": Q57B, "name": "Qwen2-57B-A14B sizes", "context": 32768, "big_batch": 32},
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            hbm = float(p.get("hbm_gbs") or 0)
            tf = float(p.get("bf16_tflops_sustained") or p.get("bf16_tflops") or 0)
            if hbm > 0 and tf > 0:
                return hbm, tf, "measured"
        except (OSError, ValueError):
            pass
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs.  It is
    started ahead of the region (the tool takes a moment to come up) and keeps the samples
    that arrive between ``begin()`` and ``stop()``."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None
        self.t_begin = None

    def begin(self):
        self.t_begin = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t_end = time.perf_counter()
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        t0 = self.t_begin if self.t_begin is not None else 0.0
        inside = [r for t, r in self.rows if t0 <= t <= t_end]
        for r in inside:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
def weight_bytes(cfg, esize=2):
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    dq = cfg["num_attention_heads"] * cfg["head_dim"]
    dkv = cfg["num_key_value_heads"] * cfg["head_dim"]
    attn = (dq + 2 * dkv) * H + H * dq
    shared = 3 * H * cfg["shared_expert_intermediate_size"]
    expert = 3 * H * cfg["moe_intermediate_size"]
    head = cfg["vocab_size"] * H
    small = 4 * ((dq + 2 * dkv) + 2 * H + cfg["num_experts"] * H + H)   # fp32 biases/gains/router
    return {"per_layer_fixed": (attn + shared) * esize + small, "per_expert": expert * esize,
            "head": head * esize, "layers": L}


def decode_step_bytes(cfg, batch, context, experts_touched_per_layer):
    wb = weight_bytes(cfg)
    kv_per_tok = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * cfg["num_hidden_layers"]
    fixed = wb["layers"] * wb["per_layer_fixed"] + wb["head"]
    experts = wb["per_expert"] * experts_touched_per_layer * wb["layers"]
    kv = batch * context * kv_per_tok
    embed = batch * cfg["hidden_size"] * 2
    return fixed + experts + kv + embed


def prefill_flops(cfg, T):
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    dq = cfg["num_attention_heads"] * cfg["head_dim"]
    dkv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_tok = 2 * ((dq + 2 * dkv) * H + H * dq + cfg["num_experts"] * H
                   + 3 * H * cfg["moe_intermediate_size"] * cfg["num_experts_per_tok"]
                   + 3 * H * cfg["shared_expert_intermediate_size"] + H)
    attn = 4 * cfg["num_attention_heads"] * cfg["head_dim"] * T * T / 2
    return L * (per_tok * T + attn) + 2 * cfg["vocab_size"] * H


def make_runtime(cfg, batch, context, extra_tokens, use_graphs=True, max_slots=None,
                 dtype="bfloat16"):
    import torch
    from inferx_b200.engine import Runtime, load_model
    from inferx_b200.weights.loader import RandomSource
    _, model = load_model(dtype=dtype, device="cuda", config_json=cfg,
                          source=RandomSource(0, device="cuda"))
    page = 16
    pages = batch * (-(-(context + extra_tokens) // page) + 1)
    rt = Runtime(model, page_size=page, num_pages=pages, max_slots=max_slots or max(batch, 1),
                 use_graphs=use_graphs)
    return rt


def fill_context(rt, batch, context):
    """Requests that already hold ``context - 1`` tokens: random keys and values stand
    in for a prompt (the timed region is decode only)."""
    import torch
    mgr = rt.manager
    for rid in list(mgr.live_requests()):
        mgr.close(rid)
    for per in rt.storage.paged.values():
        for t in per.values():
            t.normal_(0.0, 0.5)
    for i in range(batch):
        mgr.open(i)
        assert mgr.reserve(i, context - 1)
        mgr.advance(i, context - 1)


def time_decode(rt, batch, context, steps, warmup, seed=0, sampler_clock=None):
    import torch
    from inferx_b200.engine import StepEntry
    from inferx_b200.kernels import ops
    fill_context(rt, batch, context)
    mgr = rt.manager
    vocab = rt.vocab_size
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, vocab, (warmup + steps, batch), generator=g).tolist()

    def one(i):
        for r in range(batch):
            assert mgr.reserve(r, mgr.length(r) + 1)
        logits = rt.executor.step([StepEntry(r, [toks[i][r]], [0]) for r in range(batch)])
        ids = ops.sample(logits)
        for r in range(batch):
            mgr.advance(r, 1)
        return ids

    if sampler_clock:
        sampler_clock.start()
    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    l0, c0 = ops.LAUNCHES[0], ops.LIBRARY_CALLS[0]
    r0 = rt.executor.graph_replays
    if sampler_clock:
        sampler_clock.begin()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    clocks = sampler_clock.stop() if sampler_clock else None
    per_step_own = getattr(rt.executor, "graph_kernel_count", None)
    launches = ops.LAUNCHES[0] - l0
    replays = rt.executor.graph_replays - r0
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "library_calls": ops.LIBRARY_CALLS[0] - c0, "replays": replays, "clocks": clocks}


def count_step_kernels(rt, batch, context):
    """Own kernels and library products in one eager decode step, and the number of
    distinct experts each sparse layer touched."""
    import torch
    from inferx_b200.engine import StepEntry
    from inferx_b200.kernels import ops
    fill_context(rt, batch, context)
    mgr = rt.manager
    seen = []
    orig = ops.moe_dispatch

    def spy(topk_idx, num_experts):
        seen.append(int(torch.unique(topk_idx).numel()))
        return orig(topk_idx, num_experts)

    ops.moe_dispatch = spy
    graphs, rt.executor.use_graphs = rt.executor.use_graphs, False
    try:
        g = torch.Generator().manual_seed(1)
        toks = torch.randint(0, rt.vocab_size, (batch,), generator=g).tolist()
        for r in range(batch):
            assert mgr.reserve(r, mgr.length(r) + 1)
        l0, c0 = ops.LAUNCHES[0], ops.LIBRARY_CALLS[0]
        logits = rt.executor.step([StepEntry(r, [toks[r]], [0]) for r in range(batch)])
        ops.sample(logits)
        torch.cuda.synchronize()
        own, lib = ops.LAUNCHES[0] - l0, ops.LIBRARY_CALLS[0] - c0
    finally:
        ops.moe_dispatch = orig
        rt.executor.use_graphs = graphs
    touched = sum(seen) / max(1, len(seen))
    return own, lib, touched


def time_prefill(rt, tokens, reps, warmup):
    import torch
    from inferx_b200.engine import StepEntry
    mgr = rt.manager
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, rt.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for i in range(warmup + reps):
        for rid in list(mgr.live_requests()):
            mgr.close(rid)
        mgr.open("p")
        assert mgr.reserve("p", tokens)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        rt.executor.step([StepEntry("p", toks, [tokens - 1])])
        e.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(s.elapsed_time(e))
    mgr.close("p")
    times.sort()
    return times[len(times) // 2]


def time_prefill_sustained(rt, tokens, seconds):
    """Prompt steps back to back for ``seconds``: a prompt step draws enough power for the
    part to reach its power limit within a second or two, the clock sinks, and the step
    takes longer than the first few did.  Returns the median of the last third of the steps
    with the clock and the throttle reasons sampled during that third."""
    import torch
    from inferx_b200.engine import StepEntry
    mgr = rt.manager
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, rt.vocab_size, (tokens,), generator=g).tolist()
    clock = ClockSampler()
    clock.start()
    times, stamps = [], []
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end:
        for rid in list(mgr.live_requests()):
            mgr.close(rid)
        mgr.open("p")
        assert mgr.reserve("p", tokens)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        rt.executor.step([StepEntry("p", toks, [tokens - 1])])
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
        stamps.append(time.perf_counter())
    mgr.close("p")
    last = max(1, len(times) // 3)
    clock.t_begin = stamps[-last]
    seen = clock.stop()
    tail = sorted(times[-last:])
    return {"ms": tail[len(tail) // 2], "steps": len(times), "sm_mhz": seen["sm_mhz"],
            "reasons": "+".join(seen["reasons"]) or "none"}


def time_mixed(rt, batch, context, chunk, reps, warmup):
    """One step that carries a prompt portion of ``chunk`` tokens beside ``batch``
    decoding requests at ``context``: milliseconds a step (median)."""
    import torch
    from inferx_b200.engine import StepEntry
    fill_context(rt, batch, context)
    mgr = rt.manager
    g = torch.Generator().manual_seed(9)
    toks = torch.randint(0, rt.vocab_size, (chunk,), generator=g).tolist()
    times = []
    for i in range(warmup + reps):
        if mgr.has("p"):
            mgr.close("p")
        mgr.open("p")
        assert mgr.reserve("p", chunk)
        for r in range(batch):
            assert mgr.reserve(r, mgr.length(r) + 1)
        entries = [StepEntry(r, [7 + r], [0]) for r in range(batch)]
        entries.append(StepEntry("p", toks, [chunk - 1]))
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        rt.executor.step(entries)
        e.record()
        torch.cuda.synchronize()
        for r in range(batch):
            mgr.advance(r, 1)
        if i >= warmup:
            times.append(s.elapsed_time(e))
    mgr.close("p")
    times.sort()
    return times[len(times) // 2]


def time_e2e(cfg, batch, context, steps, warmup):
    """Decode through the public entry point: host ids in (pinned staging), sampled
    ids back to the host, every step.  Requests are given more tokens to generate than
    the run needs, so the batch stays whole; the first decode steps of a shape (one
    eager, one captured) count as warm-up."""
    import torch
    from inferx_b200 import Engine, EngineConfig, SamplingParams
    warm = warmup + 3
    slack = 64                      # prompts finish prefill at different steps
    prompt_len = context - (warm + steps + slack // 2)
    eng = Engine.create(EngineConfig(
        config_json=cfg, dtype="bfloat16", max_num_seqs=batch, max_model_len=context + slack + 8,
        max_num_batched_tokens=4096, block_size=16,
        num_gpu_blocks_override=batch * (-(-(context + slack + 8) // 16) + 1)))
    g = torch.Generator().manual_seed(11)
    for r in range(batch):
        eng.submit(torch.randint(0, cfg["vocab_size"], (prompt_len,), generator=g).tolist(),
                   SamplingParams(max_tokens=warm + steps + slack, ignore_eos=True))
    guard = 0
    while any(s.pending() != 1 for s in eng.scheduler.running) or eng.scheduler.waiting \
            or len(eng.scheduler.running) < batch:
        eng.step()
        guard += 1
        assert guard < 10000
    for _ in range(warm):
        eng.step()
    torch.cuda.synchronize()
    r0 = eng.runtime.executor.graph_replays
    t0 = time.perf_counter()
    n = 0
    for _ in range(steps):
        n += len(eng.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert n == batch * steps, "a request left the batch during the timed region"
    h2d = eng.runtime.executor.last_h2d_bytes
    replays = eng.runtime.executor.graph_replays - r0
    del eng
    torch.cuda.empty_cache()
    return {"value": round(n / dt, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4 * batch, "ms_per_step": round(dt / steps * 1e3, 4),
            "graph_replays": replays}


FP32_FMA_PER_SM_PER_CLOCK = 128      # fp32 lanes of one multiprocessor


def fp32_points(cfg, batch, context, hbm_peak):
    """The 32-bit path at the same sizes: weights, cache and every product in fp32 on the
    CUDA cores.  Decode against the bytes it has to read (twice the bfloat16 step's),
    a 2,048-token prompt against the fp32 multiply-add rate of the device at its
    maximum clock."""
    import torch
    rt = make_runtime(cfg, 1, batch * (context + 32) + 2048 + 64, 0, use_graphs=True,
                      max_slots=batch + 1, dtype="float32")
    own, lib, touched = count_step_kernels(rt, batch, context)
    dec = time_decode(rt, batch, context, steps=6, warmup=3)
    step_bytes = 2 * decode_step_bytes(cfg, batch, context, touched)
    pms = time_prefill(rt, 2048, reps=3, warmup=1)
    prop = torch.cuda.get_device_properties(0)
    mhz = float(getattr(prop, "clock_rate", 1965000)) / 1e3      # the maximum SM clock
    peak = prop.multi_processor_count * FP32_FMA_PER_SM_PER_CLOCK * 2 * mhz * 1e6
    fl = prefill_flops(cfg, 2048)
    out = {
        f"fp32_decode_b{batch}": round(dec["tok_s"], 1),
        f"fp32_decode_b{batch}_ms": round(dec["ms_per_step"], 3),
        f"fp32_decode_b{batch}_hbm_frac": round(step_bytes / (dec["ms_per_step"] / 1e3) / 1e9
                                                / hbm_peak, 4),
        "fp32_prefill_2048": round(2048 / (pms / 1e3), 1),
        "fp32_prefill_2048_ms": round(pms, 2),
        "fp32_prefill_2048_ffma_frac": round(fl / (pms / 1e3) / peak, 4),
        "fp32_ffma_peak_tflops": round(peak / 1e12, 1),
        "fp32_library_gemms": lib,
    }
    del rt
    torch.cuda.empty_cache()
    return out


def breakdown(rt, batch, context, steps, prefill_tokens=0):
    """Device time per kernel face over eager steps (CUDA events around every call of
    the kernel module), as a table sorted by share.  A diagnostic, not a bench value."""
    import torch
    from inferx_b200.engine import StepEntry
    from inferx_b200.kernels import ops
    names = ["embed", "add_rmsnorm", "silu_mul", "linear", "gate_up_swiglu", "qkv_rope_append", "paged_attention",
             "router_topk", "moe_dispatch", "grouped_gate_up_swiglu", "grouped_down",
             "moe_combine", "sample"]
    records, originals = [], {}

    def wrap(name, fn):
        def timed(*a, **k):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*a, **k)
            e.record()
            tag = name
            if name == "linear":
                tag = f"linear[{a[0].shape[0]}x{a[1].shape[0]}x{a[1].shape[1]}]"
            records.append((tag, s, e))
            return out
        return timed

    graphs, rt.executor.use_graphs = rt.executor.use_graphs, False
    mgr = rt.manager
    try:
        if prefill_tokens:
            for rid in list(mgr.live_requests()):
                mgr.close(rid)
        else:
            fill_context(rt, batch, context)
        g = torch.Generator().manual_seed(3)
        for i in range(steps + 1):
            if i == 1:
                for n in names:
                    originals[n] = getattr(ops, n)
                    setattr(ops, n, wrap(n, originals[n]))
            if prefill_tokens:
                if mgr.has("p"):
                    mgr.close("p")
                mgr.open("p")
                assert mgr.reserve("p", prefill_tokens)
                toks = torch.randint(0, rt.vocab_size, (prefill_tokens,), generator=g).tolist()
                logits = rt.executor.step([StepEntry("p", toks, [prefill_tokens - 1])])
            else:
                toks = torch.randint(0, rt.vocab_size, (batch,), generator=g).tolist()
                for r in range(batch):
                    assert mgr.reserve(r, mgr.length(r) + 1)
                logits = rt.executor.step([StepEntry(r, [toks[r]], [0]) for r in range(batch)])
                for r in range(batch):
                    mgr.advance(r, 1)
            ops.sample(logits)
        torch.cuda.synchronize()
    finally:
        for n, fn in originals.items():
            setattr(ops, n, fn)
        rt.executor.use_graphs = graphs
    totals = {}
    for tag, s, e in records:
        t = totals.setdefault(tag, [0.0, 0])
        t[0] += s.elapsed_time(e)
        t[1] += 1
    whole = sum(v[0] for v in totals.values())
    lines = [f"{'kernel face':44s} {'calls/step':>10s} {'ms/step':>9s} {'share':>7s}"]
    for tag, (ms, n) in sorted(totals.items(), key=lambda kv: -kv[1][0]):
        lines.append(f"{tag:44s} {n / steps:10.1f} {ms / steps:9.4f} {ms / whole:7.1%}")
    lines.append(f"{'sum of device time':44s} {'':10s} {whole / steps:9.4f}")
    return "\n".join(lines)


def marginal(rt, batch, context, steps, prefill_tokens=0, qkv_rows=0):
    """What each kernel face costs *inside* the recorded step: the decode step (or, with
    ``prefill_tokens``, a prompt step of that many tokens) is timed again with that
    face's launches left out (it hands back the result of its first call), and the
    difference is what the face adds to the step where it runs, with dependent launch, the
    side stream and its neighbours as they are.  A diagnostic, not a bench value: the
    steps it times compute nonsense."""
    import torch
    from inferx_b200.engine.executor import GraphCache
    from inferx_b200.kernels import ops

    # A prompt step draws enough power for the clock to sink while the list is measured
    # (11.5 ms on a cool part, 12.8 ms forty steps later), which is more than most faces
    # cost.  So the whole step is recorded once, every variant is recorded beside it, and
    # the two recordings are replayed in turns: what is reported is the median of the
    # differences between neighbours.
    whole = {}

    def record_prompt():
        rt.executor._graphs = GraphCache()
        time_prefill(rt, prefill_tokens, 1, 3)      # a prompt shape is recorded the third time
        return rt.executor._graphs

    def run():
        if prefill_tokens:
            if "graphs" not in whole:
                whole["graphs"] = record_prompt()
                rt.executor._graphs = whole["graphs"]
                return time_prefill(rt, prefill_tokens, 7, 0)
            variant = record_prompt()
            pairs = []
            for _ in range(9):
                rt.executor._graphs = whole["graphs"]
                a = time_prefill(rt, prefill_tokens, 1, 0)
                rt.executor._graphs = variant
                pairs.append((a, time_prefill(rt, prefill_tokens, 1, 0)))
            whole["base"] = sorted(a for a, _ in pairs)[len(pairs) // 2]
            return whole["base"] - sorted(a - b for a, b in pairs)[len(pairs) // 2]
        rt.executor._graphs = GraphCache()       # the same shape must be recorded anew
        return time_decode(rt, batch, context, steps, 4)["ms_per_step"]

    # with a face left out, the expert offsets are no longer two launches back
    settled = ops.grouped_down
    ops.grouped_down = lambda act, offsets, w, offsets_settled=False: settled(act, offsets, w)
    layers = rt.model.spec.schedule.__len__()
    base = run()
    what = (f"prompt step, {prefill_tokens} tokens" if prefill_tokens
            else f"decode step, batch {batch}, context {context}")
    lines = [f"{what}: {base:.4f} ms",
             f"{'left out':44s} {'ms/step':>9s} {'us/layer':>9s} {'us/step':>9s}"]

    def without(names, pred=None):
        cache, orig = {}, {n: getattr(ops, n) for n in names}

        def fake(n, fn):
            def call(*a, **k):
                if pred is not None and not pred(n, a):
                    return fn(*a, **k)
                key = (n,) + tuple(tuple(x.shape) for x in a if isinstance(x, torch.Tensor))
                if key not in cache:
                    cache[key] = fn(*a, **k)
                return cache[key]
            return call
        for n, fn in orig.items():
            setattr(ops, n, fake(n, fn))
        try:
            return run()
        finally:
            for n, fn in orig.items():
                setattr(ops, n, fn)

    hidden = rt.model.spec.hidden
    faces = [
        ("attention over the cache (+ merge)", ["paged_attention"], None),
        ("QKV product + rotation + cache write", ["qkv_project_rope_append"], None),
        ("QKV product (library)", ["linear"],
         lambda n, a: tuple(a[1].shape) == (qkv_rows, hidden) and qkv_rows != hidden),
        ("rotation + cache write", ["qkv_rope_append"], None),
        ("shared expert's SwiGLU", ["silu_mul"], None),
        ("gather of the routed rows", ["gather_rows"], None),
        ("output projection", ["linear"], lambda n, a: tuple(a[1].shape) == (hidden, hidden)),
        ("vocabulary projection", ["linear"], lambda n, a: a[1].shape[0] == rt.vocab_size),
        ("routed gate/up + SwiGLU", ["grouped_gate_up_swiglu"], None),
        ("routed down", ["grouped_down"], None),
        ("shared expert (side stream)", ["gate_up_swiglu", "linear"],
         lambda n, a: n == "gate_up_swiglu" or a[1].shape[0] == hidden and a[1].shape[1] != hidden),
        ("router logits + selection", ["router_topk"], None),
        ("dispatch tables", ["moe_dispatch"], None),
        ("both norms (+ combine)", ["add_rmsnorm"], None),
        ("sampling", ["sample"], None),
    ]
    try:
        for name, names, pred in faces:
            t = without(names, pred)
            base = whole.get("base", base)       # a prompt step: the whole step timed beside it
            lines.append(f"{name:44s} {t:9.4f} {(base - t) * 1e3 / layers:9.1f} "
                         f"{(base - t) * 1e3:9.0f}")
    finally:
        ops.grouped_down = settled
    return "\n".join(lines)


def serving_run(args):
    """Continuous batching under memory pressure, in the shape of BASELINE.json's fifth
    configuration: A2.7B layer sizes with every second layer dense, renormalised top-k
    and a sliding window on the last three layers; requests with prompts of uniform random
    length, a fixed number of decoded tokens each, prefill portions of 512 tokens beside
    decoding sequences, and a cache pool sized to a fraction of what the requests would
    need at once, so that sequences are preempted and recomputed.  Returns the record
    (tokens per second, steps, preemptions) that ``--serving`` prints."""
    import torch
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    layers = args.layers
    cfg = dict(A27B, num_hidden_layers=layers, decoder_sparse_step=2, norm_topk_prob=True,
               use_sliding_window=True, sliding_window=4096, max_window_layers=max(0, layers - 3))
    n_req, max_prompt, new_tokens = args.requests, args.max_prompt, args.new_tokens
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(16, max_prompt + 1, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    page = 16
    demand = sum(-(-(n + new_tokens) // page) for n in lens[:args.max_num_seqs])
    longest = -(-(max_prompt + new_tokens) // page) + 1
    pages = max(longest, int(args.pool_fraction * demand))
    eng = Engine.create(EngineConfig(
        config_json=cfg, dtype="bfloat16", max_num_seqs=args.max_num_seqs,
        max_model_len=max_prompt + new_tokens + 8, max_num_batched_tokens=2048,
        prefill_chunk=512, block_size=page, num_gpu_blocks_override=pages))
    reqs = [Request(p, SamplingParams(max_tokens=new_tokens, ignore_eos=True)) for p in prompts]
    # one short request first, untimed: it loads the kernels and the library's plans, as a
    # server that has been up for a while has; its steps are not counted below
    eng.generate([Request(prompts[0][:700], SamplingParams(max_tokens=4, ignore_eos=True))])
    before = eng.stats()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate(reqs)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.stats()
    for k, v in before.items():               # what the timed run added
        if isinstance(v, dict):
            st[k] = {kk: round(st[k][kk] - vv, 4) for kk, vv in v.items()}
        elif isinstance(v, (int, float)) and not isinstance(v, bool):
            st[k] = st[k] - v
    reasons = {}
    for c in outs:
        reasons[c.reason] = reasons.get(c.reason, 0) + 1
    del eng
    torch.cuda.empty_cache()
    return {
        "workload": "serving", "requests": n_req, "max_num_seqs": args.max_num_seqs,
        "warmup_requests": 1,
        "prompt_tokens": sum(lens), "generated_tokens": st["tokens_generated"],
        "seconds": round(dt, 3), "output_tok_s": round(st["tokens_generated"] / dt, 1),
        "total_tok_s": round((st["tokens_generated"] + st["tokens_prefilled"]) / dt, 1),
        "steps": st["steps"], "graph_replays": st["graph_replays"],
        "preemptions": st["preemptions"],
        "tokens_prefilled_incl_recompute": st["tokens_prefilled"],
        "host_seconds": st["host_seconds"], "graph_captures": st["graph_captures"],
        "capture_seconds": st["capture_seconds"], "eager_steps": st["eager_steps"],
        "host_share_not_waiting": round(1.0 - st["host_seconds"]["wait"] / dt, 3),
        "pool_pages": pages, "pool_fraction_of_demand": args.pool_fraction,
        "finish_reasons": reasons, "layers": layers, "layers_of_config": FULL_LAYERS}


def serving(args):
    print(json.dumps(serving_run(args)))
    return 0


def serving_check(args):
    """The correctness claim of the serving workload: preemption by recompute does not
    change what a request generates.  The same requests run greedily in 32-bit twice,
    with a roomy cache pool and with one sized to a fraction of the demand (so that
    sequences are preempted and recomputed), at the serving configuration's layer sizes
    with few layers and smaller counts.  Two runs batch tokens differently, which moves
    32-bit sums by rounding; so where a request's tokens differ, the logits at the first
    difference are computed once more for that request alone, and the two tokens chosen
    must be level there within the 32-bit bound (2e-5 of the largest logit)."""
    import torch
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    from inferx_b200.engine import StepEntry
    layers = args.layers
    cfg = dict(A27B, num_hidden_layers=layers, decoder_sparse_step=2, norm_topk_prob=True,
               use_sliding_window=True, sliding_window=4096, max_window_layers=max(0, layers - 1),
               torch_dtype="float32")
    n_req, max_prompt, new_tokens = args.requests, args.max_prompt, args.new_tokens
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(16, max_prompt + 1, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    page = 16
    demand = sum(-(-(n + new_tokens) // page) for n in sorted(lens)[-args.max_num_seqs:])
    longest = -(-(max_prompt + new_tokens) // page) + 1

    def run(pages):
        eng = Engine.create(EngineConfig(
            config_json=cfg, dtype="float32", max_num_seqs=args.max_num_seqs,
            max_model_len=max_prompt + new_tokens + 8, max_num_batched_tokens=2048,
            prefill_chunk=512, block_size=page, num_gpu_blocks_override=pages))
        outs = eng.generate([Request(p, SamplingParams(max_tokens=new_tokens, ignore_eos=True))
                             for p in prompts])
        return eng, [c.output_tokens for c in outs], eng.stats()["preemptions"]

    tight_pages = max(longest, int(args.pool_fraction * demand))
    eng, tight, pre_tight = run(tight_pages)
    del eng
    torch.cuda.empty_cache()
    eng, roomy, pre_roomy = run(demand + longest)
    identical = level = 0
    worst_gap = 0.0
    failures = []
    rt = eng.runtime
    for i, (a, b) in enumerate(zip(roomy, tight)):
        if a == b:
            identical += 1
            continue
        j = next(k for k in range(min(len(a), len(b))) if a[k] != b[k])
        seq = prompts[i] + a[:j]
        rt.manager.open(("check", i))
        assert rt.manager.reserve(("check", i), len(seq))
        row = rt.executor.step([StepEntry(("check", i), seq, [len(seq) - 1])])[0].float()
        gap = abs(float(row[a[j]] - row[b[j]])) / float(row.abs().max())
        top = float(row.max() - max(row[a[j]], row[b[j]])) / float(row.abs().max())
        rt.manager.close(("check", i))
        worst_gap = max(worst_gap, gap, top)
        if gap <= 2e-5 and top <= 2e-5:
            level += 1
        else:
            failures.append({"request": i, "position": j, "gap": gap, "below_top": top})
    ok = not failures and pre_tight >= 1 and pre_roomy == 0
    print(json.dumps({
        "workload": "serving --check", "dtype": "float32", "layers": layers,
        "requests": n_req, "max_num_seqs": args.max_num_seqs, "new_tokens": new_tokens,
        "preemptions_tight": pre_tight, "preemptions_roomy": pre_roomy,
        "pool_pages_tight": tight_pages, "identical_requests": identical,
        "level_at_first_difference": level, "worst_relative_gap": worst_gap,
        "failures": failures, "ok": ok}))
    return 0 if ok else 1


def reference_arm():
    why = ("divedb/InferX is a C++20/CMake project with no Python package (no setup.py or "
           "pyproject.toml) and needs abseil, CLI11, folly and FlashInfer sources that are absent "
           "offline; it also cannot load Qwen2-MoE checkpoints at all")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--sizes", default="a2.7b", choices=sorted(SIZES),
                    help="layer sizes: the headline configuration, or the 57B one")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the default decode run")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--serving", action="store_true",
                    help="continuous batching with preemption instead of the bench line")
    ap.add_argument("--check", action="store_true",
                    help="with --serving: preempted and unpreempted runs generate the same "
                         "(32-bit, greedy, few layers)")
    ap.add_argument("--requests", type=int, default=None, help="64; with --check 24")
    ap.add_argument("--max-num-seqs", type=int, default=None, help="64 (every request may run at once; the pool then decides); with --check 8")
    ap.add_argument("--max-prompt", type=int, default=None, help="6000; with --check 1500")
    ap.add_argument("--new-tokens", type=int, default=None, help="256; with --check 48")
    ap.add_argument("--pool-fraction", type=float, default=None, help="0.6; with --check 0.3")
    ap.add_argument("--breakdown", choices=["decode", "prefill"],
                    help="print device time per kernel face instead of the bench line")
    ap.add_argument("--marginal", action="store_true",
                    help="print what each kernel face adds to the recorded decode step")
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help="with --marginal: a prompt step of this many tokens instead")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from inferx_b200.kernels import ops
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    sizes = SIZES[args.sizes]
    full_layers = sizes["cfg"]["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    if args.context is None:
        args.context = sizes["context"]
    small = bool(args.check)
    for key, full, few in (("requests", 64, 24), ("max_num_seqs", 64, 8), ("max_prompt", 6000, 1500),
                           ("new_tokens", 256, 48), ("pool_fraction", 0.6, 0.3)):
        if getattr(args, key) is None:
            setattr(args, key, few if small else full)
    if args.serving and args.check:
        if "--layers" not in (argv or sys.argv):
            args.layers = 3
        return serving_check(args)
    if args.serving:
        return serving(args)
    hbm_peak, tf_peak, peak_src = peaks()
    cfg = dict(sizes["cfg"], num_hidden_layers=args.layers)
    B, C = args.batch, args.context
    big_b, big_c = sizes["big_batch"], C
    extra = args.steps + args.warmup + 8
    points_wanted = not (args.skip_points or args.breakdown or args.marginal)
    # what the device has to hold: weights, and the cache pool of the widest run (plus
    # the 2,048-token portion of the mixed step); the widest run's context is cut, in
    # steps of 4096, until it fits
    wb = weight_bytes(cfg)
    weights = wb["layers"] * (wb["per_layer_fixed"] + cfg["num_experts"] * wb["per_expert"]) \
        + 2 * wb["head"]
    kv_tok = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * args.layers
    room = 0.88 * torch.cuda.get_device_properties(0).total_memory - weights - (6 << 30)
    pool_tokens = B * (C + extra + 16) + 2048 + 64
    if points_wanted:
        while big_c > 4096 and big_b * (big_c + extra + 16) * kv_tok > room:
            big_c -= 4096
        pool_tokens = max(pool_tokens, big_b * (big_c + extra + 16))
    if pool_tokens * kv_tok > room:
        print(f"bench.py: {weights / 1e9:.1f} GB of weights and {pool_tokens * kv_tok / 1e9:.1f} GB "
              f"of cache do not fit this device; give fewer --layers or a shorter --context")
        return 2
    rt = make_runtime(cfg, 1, pool_tokens, 0, use_graphs=not args.no_graphs,
                      max_slots=max(B, big_b if points_wanted else B) + 1)

    if args.marginal:
        print(marginal(rt, B, C, min(args.steps, 24), prefill_tokens=args.prefill_tokens,
                       qkv_rows=(cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"])
                       * cfg["head_dim"]))
        return 0
    if args.breakdown:
        print(breakdown(rt, B, C, min(args.steps, 4),
                        prefill_tokens=2048 if args.breakdown == "prefill" else 0))
        return 0
    own, lib, touched = count_step_kernels(rt, B, C)
    clock = ClockSampler()
    dec = time_decode(rt, B, C, args.steps, args.warmup, sampler_clock=clock)
    step_bytes = decode_step_bytes(cfg, B, C, touched)
    achieved = step_bytes / (dec["ms_per_step"] / 1e3) / 1e9
    out = {
        "metric": METRIC if args.sizes == "a2.7b" else
        f"decode tok/s at batch {B}, context {C} ({sizes['name']})",
        "value": round(dec["tok_s"], 1), "unit": "tok/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dec["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids, random cache",
        "impl": "ours",
        "config": {
            "model": sizes["name"], "global_batch": B, "seq_len": C,
            "parallelism": "single GPU", "layers": args.layers, "layers_of_config": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "experts": cfg["num_experts"], "top_k": cfg["num_experts_per_tok"],
            "moe_intermediate": cfg["moe_intermediate_size"],
            "shared_intermediate": cfg["shared_expert_intermediate_size"],
            "vocab": cfg["vocab_size"], "page_size": 16,
            "cuda_graphs": not args.no_graphs,
            "l2": "inputs larger than L2 (GBs of weights and cache per step)",
        },
        "clocks": dec["clocks"],
        "gpu_launches": own * args.steps,
        "launches_per_step": {"own_kernels": own, "library_gemms": lib},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak,
                     "unit": "GB/s", "frac": round(achieved / hbm_peak, 4),
                     "peak_source": peak_src, "bytes_per_step": int(step_bytes),
                     "experts_touched_per_layer": round(touched, 2)},
    }
    points = {}
    if not args.skip_points:
        for b, c in ((1, C), (big_b, big_c)):
            d = time_decode(rt, b, c, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(d["tok_s"], 1)
            points[f"decode_b{b}_ms"] = round(d["ms_per_step"], 4)
            if c != C:
                points[f"decode_b{b}_context"] = c
        mms = time_mixed(rt, B, C, 2048, reps=5, warmup=3)
        points["mixed_2048_plus_decode_ms"] = round(mms, 3)
        points["mixed_2048_plus_decode_tok_s"] = round((2048 + B) / (mms / 1e3), 1)
        pms = time_prefill(rt, 2048, reps=5, warmup=3)
        fl = prefill_flops(cfg, 2048)
        out["prefill"] = {"value": round(2048 / (pms / 1e3), 1), "tokens": 2048,
                          "ms": round(pms, 3),
                          "frac": round(fl / (pms / 1e3) / (tf_peak * 1e12), 4),
                          "flops": int(fl), "peak_tflops": tf_peak, "peak_source": peak_src}
        # further contexts and prompt lengths (what the cache pool of the widest run holds)
        for c in (16384, 32768):
            if B * (c + extra + 16) <= pool_tokens:
                d = time_decode(rt, B, c, max(8, args.steps // 4), args.warmup)
                by = decode_step_bytes(cfg, B, c, touched)
                points[f"decode_b{B}_ctx{c}_ms"] = round(d["ms_per_step"], 4)
                points[f"decode_b{B}_ctx{c}_hbm_frac"] = round(
                    by / (d["ms_per_step"] / 1e3) / 1e9 / hbm_peak, 4)
        for t in (4096, 8192):
            if t + 64 <= pool_tokens:
                ms = time_prefill(rt, t, reps=3, warmup=2)
                points[f"prefill_{t}_tok_s"] = round(t / (ms / 1e3), 1)
                points[f"prefill_{t}_frac"] = round(
                    prefill_flops(cfg, t) / (ms / 1e3) / (tf_peak * 1e12), 4)
        # last, because it leaves the part hot: prompt steps back to back for 2.5 s
        sus = time_prefill_sustained(rt, 2048, 2.5)
        points["prefill_2048_sustained_ms"] = round(sus["ms"], 3)
        points["prefill_2048_sustained_frac"] = round(
            fl / (sus["ms"] / 1e3) / (tf_peak * 1e12), 4)
        points["prefill_2048_sustained_sm_mhz"] = sus["sm_mhz"]
        points["prefill_2048_sustained_reasons"] = sus["reasons"]
        out["points"] = points
    del rt
    torch.cuda.empty_cache()
    if not args.skip_points and args.sizes == "a2.7b":
        out["e2e"] = time_e2e(cfg, B, C, args.steps, args.warmup)
    elif not args.skip_points:
        out["e2e"] = {"unmeasured": "a second copy of the weights for the entry point's own "
                                    "engine is not made at these sizes"}
    if not args.skip_points and args.sizes == "a2.7b":
        out["points"].update(fp32_points(cfg, B, C, hbm_peak))
    if not args.skip_points and args.sizes == "a2.7b" and args.layers == full_layers:
        sv = serving_run(args)
        out["points"].update({"serving_total_tok_s": sv["total_tok_s"],
                              "serving_seconds": sv["seconds"],
                              "serving_requests": sv["requests"],
                              "serving_preemptions": sv["preemptions"]})
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
