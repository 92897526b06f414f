"""A plain, slow implementation of Qwen2-MoE: whole sequences, no cache, fp32.

It rests on the formulas of divedb/InferX's sources, not on running them: the
reference's model code exists only as CUDA behind abseil/cuBLASLt/FlashInfer,
which cannot be compiled or imported on the CPU here (its ``third_party/`` is
empty), so there is no golden output of the forward pass made by the reference itself
(its scheduler and its host sampler do compile on the CPU: tests/golden/ holds what they
decide, and tests/test_scheduler_golden.py compares this file's sampling statements and
the package's scheduler with that; its CUDA kernels compile too, tests/golden/ops_golden.bin
holds what they computed on a B200 for every part below, and tests/test_ops_golden.py
compares the functions of this file with that).  Each function below cites the reference
lines whose arithmetic it restates.  It shares no code
with ``inferx_b200``: it reads config.json as a plain dict and the tensors by
their checkpoint names from a plain dict of fp32 CPU tensors.

One function per part; ``forward`` returns logits for every position.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch


# ---------------------------------------------------------------------------
# reading a model folder (independent of the package's loader)
# ---------------------------------------------------------------------------
_ST_DTYPES = {"F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2)}


def read_model_folder(path):
    """(config dict, {name: fp32 tensor}) from config.json + model.safetensors."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode())
    data = blob[8 + hlen:]
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt, isz = _ST_DTYPES[meta["dtype"]]
        b, e = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=dt).reshape(meta["shape"])
        tensors[name] = t.to(torch.float32)
    return cfg, tensors


# ---------------------------------------------------------------------------
# config helpers: the per-layer rules
# ---------------------------------------------------------------------------
def head_dim_of(cfg):
    # src/model/config.cc:313-317: head_dim defaults to hidden/heads
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_is_sparse(cfg, i):
    """Sparse iff experts exist, i is not an MLP-only layer and (i+1) is a multiple
    of decoder_sparse_step (the reference has no rule for this architecture; its
    DeepSeek rule is include/inferx/model/config.h:121-126)."""
    return (cfg.get("num_experts", 0) > 0 and i not in cfg.get("mlp_only_layers", [])
            and (i + 1) % cfg.get("decoder_sparse_step", 1) == 0)


def layer_window(cfg, i):
    """Window W (keys max(0,p-W+1)..p) of layer i; 0 = all keys.  Nothing slides
    without use_sliding_window and a positive sliding_window
    (include/inferx/model/config.h:196-203: no window, no sliding layer).  With them,
    the entry of "layer_types" decides when config.json has that list
    (src/model/config.cc:438-456); a file without the list slides on the layers from
    max_window_layers on."""
    if not cfg.get("use_sliding_window", False) or cfg.get("sliding_window", 0) <= 0:
        return 0
    kinds = cfg.get("layer_types")
    if kinds:
        if kinds[i] not in ("full_attention", "sliding_attention"):
            raise ValueError(f"unknown layer_type {kinds[i]!r}")
        return cfg["sliding_window"] if kinds[i] == "sliding_attention" else 0
    if i >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return cfg["sliding_window"]
    return 0


# ---------------------------------------------------------------------------
# parts
#
# Every part takes ``rf``, a rounding function applied where an engine that stores
# activations in a narrower type rounds them (after a norm, a projection, the
# attention output, an activation, a combine).  The default is the identity: pure
# fp32.  With ``rf=round_bf16`` the same formulas give what bfloat16 storage alone
# costs, which is how the error budget of the bfloat16 tests is derived (the
# reference derives its tolerance the same way, scripts/gen_reference_logits.py:51-55).
# ---------------------------------------------------------------------------
def _identity(t):
    return t


def round_bf16(t):
    return t.to(torch.bfloat16).to(torch.float32)


def rmsnorm(x, gain, eps):
    """x * rsqrt(mean(x^2) + eps) * gain  (src/backends/cuda/ops/layers.cu:50-76)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(ms + eps)) * gain


def rope(x, positions, theta):
    """Half-split rotation of x [T, heads, hd] (layers.cu:80-115): for j < hd/2,
    inv_freq = theta^(-2j/hd), a = pos * inv_freq,
    (x[j], x[j+hd/2]) <- (x[j] cos a - x[j+hd/2] sin a, x[j+hd/2] cos a + x[j] sin a)."""
    hd = x.shape[-1]
    half = hd // 2
    j = torch.arange(half, dtype=torch.float64)
    inv_freq = (float(theta) ** (-2.0 * j / hd)).to(torch.float32)
    a = positions.to(torch.float32)[:, None] * inv_freq[None, :]     # [T, half] fp32
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def attention(q, k, v, scale, window):
    """Causal grouped-query attention over a whole sequence
    (layers.cu:256-318; window: layers.cu:346-354).  q [T, heads, hd], k, v
    [T, kv_heads, hd]; kv head of head h is h // (heads / kv_heads); query at
    position p sees keys max(0, p-W+1)..p; softmax with max subtraction."""
    T, heads, hd = q.shape
    kvh = k.shape[1]
    rep = heads // kvh
    out = torch.zeros_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible &= pos[None, :] >= (pos[:, None] - window + 1)
    for h in range(heads):
        kh = h // rep
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def attention_block(cfg, w, prefix, x, positions, window, rf=_identity):
    """QKV projection with bias on q, k, v only, rotation after the bias, no bias on
    the output projection (src/model/qwen2.cc:920-1027; layers.cu:485-510)."""
    heads, kvh, hd = cfg["num_attention_heads"], cfg.get("num_key_value_heads",
                                                         cfg["num_attention_heads"]), head_dim_of(cfg)
    T = x.shape[0]

    def proj(name):
        y = rf(x @ w[f"{prefix}.{name}.weight"].T)
        b = w.get(f"{prefix}.{name}.bias")
        return y + b if b is not None else y

    q = proj("q_proj").view(T, heads, hd)
    k = proj("k_proj").view(T, kvh, hd)
    v = rf(proj("v_proj").view(T, kvh, hd))
    theta = cfg.get("rope_theta", 10000.0)
    q, k = rf(rope(q, positions, theta)), rf(rope(k, positions, theta))
    o = rf(attention(q, k, v, 1.0 / math.sqrt(hd), window))      # scale: qwen2.cc:890
    return rf(o.reshape(T, heads * hd) @ w[f"{prefix}.o_proj.weight"].T)


def silu(g):
    """g / (1 + exp(-g))  (layers.cu:512-529)."""
    return g / (1.0 + torch.exp(-g))


def swiglu_mlp(w, prefix, x, rf=_identity):
    """down(silu(gate(x)) * up(x)), no biases (qwen2.cc:1042-1048)."""
    g = x @ w[f"{prefix}.gate_proj.weight"].T
    u = x @ w[f"{prefix}.up_proj.weight"].T
    return rf(rf(silu(g) * u) @ w[f"{prefix}.down_proj.weight"].T)


def route(logits, k, renorm, scale=1.0):
    """Softmax over all experts, k rounds of argmax with ties to the lower index,
    optional renormalisation guarded by total > 0, then the routed scale
    (src/backends/cuda/ops/moe.cu:36-127).  Returns (weights [T,k], experts [T,k])."""
    m = logits.max(dim=-1, keepdim=True).values
    p = torch.exp(logits - m)
    p = p / p.sum(dim=-1, keepdim=True)
    T, E = p.shape
    weights = torch.zeros(T, k)
    experts = torch.zeros(T, k, dtype=torch.long)
    for t in range(T):
        row = p[t].clone()
        for s in range(k):
            best, bi = -1.0, 0
            for e in range(E):
                if row[e].item() > best:        # strictly greater: ties keep the lower index
                    best, bi = row[e].item(), e
            weights[t, s] = best
            experts[t, s] = bi
            row[bi] = -2.0
        if renorm:
            total = weights[t].sum()
            if total > 0:
                weights[t] = weights[t] / total
    return weights * scale, experts


def moe_block(cfg, w, prefix, x, rf=_identity):
    """Routed experts combined in slot order plus the sigmoid-gated shared expert
    over every token (src/model/moe_ffn.cc:158-367; combine moe.cu:237-255; shared
    expert moe.cu:275-287).  Every expert is evaluated on its tokens only."""
    E, k = cfg["num_experts"], cfg["num_experts_per_tok"]
    logits = x @ w[f"{prefix}.gate.weight"].T
    # absent means renormalise (src/model/config.cc:361-362)
    weights, experts = route(logits, k, cfg.get("norm_topk_prob", True))
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        acc = torch.zeros(x.shape[1])
        for s in range(k):
            e = int(experts[t, s])
            y = swiglu_mlp(w, f"{prefix}.experts.{e}", x[t:t + 1], rf)[0]
            acc = acc + weights[t, s] * y
        out[t] = acc
    if cfg.get("shared_expert_intermediate_size", 0) > 0:
        shared = swiglu_mlp(w, f"{prefix}.shared_expert", x, rf)
        gate_w = w.get(f"{prefix}.shared_expert_gate.weight")
        if gate_w is not None:
            g = x @ gate_w.T                                     # [T, 1]
            shared = shared * (1.0 / (1.0 + torch.exp(-g)))
        out = out + shared
    return rf(out)


def decoder_layer(cfg, w, i, x, positions, rf=_identity):
    """r = x; x = attn(norm(x)) + r; r = x; x = ffn(norm(x)) + r (qwen2.cc:908-1051)."""
    p = f"model.layers.{i}"
    eps = cfg.get("rms_norm_eps", 1e-6)
    n = rf(rmsnorm(x, w[f"{p}.input_layernorm.weight"], eps))
    x = x + attention_block(cfg, w, f"{p}.self_attn", n, positions, layer_window(cfg, i), rf)
    n = rf(rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], eps))
    if layer_is_sparse(cfg, i):
        f = moe_block(cfg, w, f"{p}.mlp", n, rf)
    else:
        f = swiglu_mlp(w, f"{p}.mlp", n, rf)
    return x + f


def forward(cfg, w, tokens, rf=_identity):
    """Logits [T, vocab] of a whole sequence (embedding layers.cu:465-481; final norm
    and head qwen2.cc:1059-1066; tied head aliases the embedding qwen2.cc:1333-1341)."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["model.embed_tokens.weight"][ids]
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(cfg, w, i, x, positions, rf)
    n = rf(rmsnorm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6)))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return n @ head.T


# ---------------------------------------------------------------------------
# sampling (src/engine/host_sampling.cc:50-111; argmax ties to the lower index,
# src/backends/cuda/ops/layers.cu:413-452)
# ---------------------------------------------------------------------------
def greedy(logits_row):
    best, bi = None, 0
    for i, v in enumerate(logits_row.tolist()):
        if best is None or v > best:
            best, bi = v, i
    return bi


def uniform_from_seed(seed):
    """splitmix64(seed), top 24 bits as a float in [0, 1)."""
    mask = (1 << 64) - 1
    z = (seed + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def sample_temperature(logits_row, temperature, seed):
    """p ~ exp(logit/t - max); inverse CDF in index order with one uniform."""
    x = logits_row.to(torch.float64) / temperature
    p = torch.exp(x - x.max())
    target = uniform_from_seed(seed) * p.sum().item()
    c = torch.cumsum(p, 0)
    idx = int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64)).item())
    return min(idx, len(p) - 1), c, target


def penalised(logits_row, generated, presence, frequency, repetition, masked=()):
    """The logits a token is chosen from when its request has penalties
    (src/engine/host_sampling.cc:21-48): for every distinct token generated so far,
    x / repetition when positive else x * repetition, then minus presence, minus
    frequency times how often it was generated; masked tokens (stop tokens under
    ``min_tokens``, src/scheduler/scheduler.cc:647-657) end at -inf."""
    row = logits_row.clone().to(torch.float32)
    counts = {}
    for t in generated:
        counts[t] = counts.get(t, 0) + 1
    for t, n in counts.items():
        v = row[t]
        if repetition != 1.0:
            v = v / repetition if v > 0 else v * repetition
        row[t] = v - presence - frequency * n
    for t in masked:
        row[t] = float("-inf")
    return row


def logprobs(logits_row, chosen, k):
    """(log-probability of ``chosen``, [(token, log-probability)] of the k most probable,
    ties to the lower id) under softmax of the row at temperature 1
    (src/engine/host_sampling.cc:114-146)."""
    row = logits_row.to(torch.float64)
    log_z = float(torch.log(torch.exp(row - row.max()).sum()) + row.max())
    order = sorted(range(len(row)), key=lambda i: (-float(row[i]), i))[:k]
    return float(row[chosen]) - log_z, [(i, float(row[i]) - log_z) for i in order]
