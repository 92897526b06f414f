"""Plain fp32 statements of what each kernel computes, with torch on the CPU.

Two uses: (1) the ``-m gpu`` kernel tests compare each CUDA kernel with the
function of the same name here; (2) the CPU tests put this module where the engine
expects its kernel module, so that the cache manager, the step function and the
scheduler are exercised against the plain model without a GPU.  It is a test
double, not a product path: the package itself never imports it and refuses CPU
tensors.  Everything is computed in fp32 whatever the storage type.
"""
from __future__ import annotations

import torch


def _f(t):
    return t.to(torch.float32)


def embed(table, ids, out=None):
    r = _f(table)[ids.long()]
    if out is not None:
        out.copy_(r)
        return out
    return r


def add_rmsnorm(resid, delta, gain, eps, out_dtype, rows=None):
    if rows is None:
        if delta is not None:
            resid += _f(delta)
        v = resid
    else:
        v = resid[rows.long()]
        if delta is not None:
            v = v + _f(delta)[rows.long()]
    ms = (v * v).sum(-1, keepdim=True) / v.shape[-1]
    return (v * (1.0 / torch.sqrt(ms + eps)) * gain).to(out_dtype)


def silu_mul(gu):
    i = gu.shape[1] // 2
    g, u = _f(gu[:, :i]), _f(gu[:, i:])
    return (g / (1.0 + torch.exp(-g)) * u).to(gu.dtype)


def linear(x, w, out_dtype=None):
    return (_f(x) @ _f(w).T).to(out_dtype or x.dtype)


def gate_up_swiglu(x, w_gate_up):
    return silu_mul(linear(x, w_gate_up))


def _rotate(x, positions, inv_freq, rot):
    # x [T, heads, hd] fp32
    if not rot:
        return x
    half = rot // 2
    a = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:rot]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]], dim=-1)


def _scatter(cache, rows, slots):
    # cache [P, kvh, page, hd]; rows [T, kvh, hd]
    page = cache.shape[2]
    for t in range(rows.shape[0]):
        s = int(slots[t])
        if s >= 0:
            cache[s // page, :, s % page, :] = rows[t].to(cache.dtype)


def qkv_rope_append(qkv, bias, positions, inv_freq, rotary_dim, heads, kv_heads, head_dim,
                    k_cache, v_cache, slots, want_dense_kv=False):
    T = qkv.shape[0]
    x = _f(qkv)
    if bias is not None:
        x = x + bias
    dq, dkv = heads * head_dim, kv_heads * head_dim
    q = _rotate(x[:, :dq].reshape(T, heads, head_dim), positions, inv_freq, rotary_dim)
    k = _rotate(x[:, dq:dq + dkv].reshape(T, kv_heads, head_dim), positions, inv_freq, rotary_dim)
    v = x[:, dq + dkv:].reshape(T, kv_heads, head_dim)
    q, k, v = q.to(qkv.dtype), k.to(qkv.dtype), v.to(qkv.dtype)
    if k_cache is not None:
        _scatter(k_cache, k, slots)
        _scatter(v_cache, v, slots)
    return (q, k, v) if want_dense_kv else q


def append_kv(k, v, k_cache, v_cache, slots):
    _scatter(k_cache, k, slots)
    _scatter(v_cache, v, slots)


def paged_attention_generic(q, k_cache, v_cache, block_table, seq_of_token, positions, window,
                            scale):
    T, heads, hd = q.shape
    P, kvh, page, _ = k_cache.shape
    rep = heads // kvh
    out = torch.zeros(T, heads, hd, dtype=torch.float32)
    for t in range(T):
        s, pos = int(seq_of_token[t]), int(positions[t])
        start = max(0, pos - window + 1) if window > 0 else 0
        kp = torch.arange(start, pos + 1)
        pages = block_table[s][(kp // page).long()].long()
        assert (pages >= 0).all(), "attention reads a page that was given back"
        offs = (kp % page).long()
        for h in range(heads):
            kh = h // rep
            keys = _f(k_cache[pages, kh, offs, :])
            vals = _f(v_cache[pages, kh, offs, :])
            sc = (keys @ _f(q[t, h])) * scale
            p = torch.exp(sc - sc.max())
            out[t, h] = (p[:, None] * vals).sum(0) / p.sum()
    return out.to(q.dtype)


def paged_attention(q, k_cache, v_cache, block_table, step, window, scale):
    return paged_attention_generic(q, k_cache, v_cache, block_table, step.seq_of_token,
                                   step.positions, window, scale)


def router_topk(x, w, top_k, renormalize, scale, extra_w=None):
    logits = _f(x) @ w.T
    p = torch.softmax(logits, dim=-1)
    T, E = p.shape
    tw = torch.zeros(T, top_k)
    ti = torch.zeros(T, top_k, dtype=torch.int32)
    work = p.clone()
    for s in range(top_k):
        best = work.max(dim=-1).values
        # ties to the lower index: first position equal to the max
        idx = (work == best[:, None]).to(torch.int32).argmax(dim=-1)
        tw[:, s] = best
        ti[:, s] = idx.to(torch.int32)
        work[torch.arange(T), idx] = -2.0
    if renormalize:
        tot = tw.sum(-1, keepdim=True)
        tw = torch.where(tot > 0, tw / tot, tw)
    ex = (_f(x) @ extra_w) if extra_w is not None else None
    return tw * scale, ti, ex


def moe_dispatch(topk_idx, num_experts):
    T, k = topk_idx.shape
    flat = topk_idx.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    rows = (order // k).to(torch.int32)
    dest = torch.empty(T * k, dtype=torch.int32)
    dest[order] = torch.arange(T * k, dtype=torch.int32)
    return offsets, rows, dest


def grouped_gate_up_swiglu(x, rows, offsets, w_gate_up):
    E, two_i, H = w_gate_up.shape
    i = two_i // 2
    out = torch.zeros(rows.numel(), i, dtype=torch.float32)
    for e in range(E):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi > lo:
            xe = _f(x[rows[lo:hi].long()])
            g = xe @ _f(w_gate_up[e, :i]).T
            u = xe @ _f(w_gate_up[e, i:]).T
            out[lo:hi] = g / (1.0 + torch.exp(-g)) * u
    return out.to(x.dtype)


def grouped_down(act, offsets, w_down, offsets_settled=False):
    E, H, i = w_down.shape
    out = torch.zeros(act.shape[0], H, dtype=torch.float32)
    for e in range(E):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi > lo:
            out[lo:hi] = _f(act[lo:hi]) @ _f(w_down[e]).T
    return out.to(act.dtype)


def moe_combine(y, dest, topk_w, shared, shared_logit):
    T, k = topk_w.shape
    out = torch.zeros(T, y.shape[1], dtype=torch.float32)
    for s in range(k):
        out += topk_w[:, s:s + 1] * _f(y[dest.view(T, k)[:, s].long()])
    if shared is not None:
        sh = _f(shared)
        if shared_logit is not None:
            sh = sh * (1.0 / (1.0 + torch.exp(-shared_logit)))[:, None]
        out += sh
    return out.to(y.dtype)


def _uniform(seed):
    mask = (1 << 64) - 1
    z = (int(seed) + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def apply_penalties(logits, hist_ids, hist_counts, penalties, mask_ids):
    R, V = logits.shape
    for r in range(R):
        if hist_ids is not None:
            pres, freq, rep = (float(v) for v in penalties[r])
            if pres != 0.0 or freq != 0.0 or rep != 1.0:
                for j in range(hist_ids.shape[1]):
                    t = int(hist_ids[r, j])
                    if not 0 <= t < V:
                        continue
                    v = logits[r, t]
                    if rep != 1.0:
                        v = v / rep if v > 0 else v * rep
                    logits[r, t] = v - pres - freq * float(hist_counts[r, j])
        if mask_ids is not None:
            for j in range(mask_ids.shape[1]):
                t = int(mask_ids[r, j])
                if 0 <= t < V:
                    logits[r, t] = float("-inf")


def max_top_logprobs():
    return 20


def token_logprobs(logits, chosen, want_k=None, top=0):
    R, V = logits.shape
    chosen_lp = torch.zeros(R, dtype=torch.float32)
    top_ids = torch.full((R, top), -1, dtype=torch.int32) if top else None
    top_lps = torch.zeros((R, top), dtype=torch.float32) if top else None
    for r in range(R):
        k = int(want_k[r]) if want_k is not None else 0
        if k < 0:
            continue
        row = logits[r].to(torch.float64)
        log_z = torch.log(torch.exp(row - row.max()).sum()) + row.max()
        chosen_lp[r] = float(row[int(chosen[r])] - log_z)
        order = sorted(range(V), key=lambda i: (-float(row[i]), i))[:min(k, top)]
        for j, i in enumerate(order):
            top_ids[r, j] = i
            top_lps[r, j] = float(row[i] - log_z)
    return chosen_lp, top_ids, top_lps


def sample(logits, temperature=None, seeds=None, top_p=None, top_k=None, min_p=None, out=None):
    R, V = logits.shape
    ids = torch.zeros(R, dtype=torch.int32)
    for r in range(R):
        t = float(temperature[r]) if temperature is not None else 0.0
        row = logits[r].to(torch.float64)
        if not t > 0:
            ids[r] = int((row == row.max()).to(torch.int32).argmax())
            continue
        p = torch.exp(row / t - (row / t).max())
        keep = torch.ones(V, dtype=torch.bool)
        order = torch.sort(p, descending=True, stable=True).indices
        k = int(top_k[r]) if top_k is not None else 0
        if 0 < k < V:
            keep &= p >= p[order[k - 1]]
        mp = float(min_p[r]) if min_p is not None else 0.0
        if mp > 0:
            keep &= p >= mp * p.max()
        tp = float(top_p[r]) if top_p is not None else 1.0
        if tp < 1.0:
            ps = torch.where(keep, p, torch.zeros_like(p))[order]
            c = torch.cumsum(ps, 0) / p.sum()
            n = int((c < tp).sum().item()) + 1
            cut = ps[min(n, V) - 1]
            keep &= p >= cut
        pk = torch.where(keep, p, torch.zeros_like(p))
        c = torch.cumsum(pk, 0)
        target = _uniform(int(seeds[r]) if seeds is not None else 0) * c[-1].item()
        idx = int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64)).item())
        idx = min(idx, V - 1)
        while not keep[idx]:
            idx += 1
        ids[r] = idx
    if out is not None:
        out.copy_(ids)
        return out
    return ids
