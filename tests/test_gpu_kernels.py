"""Each CUDA kernel alone against its plain fp32 statement (tests/host_ops.py), at
sizes other than the engine's tiny configurations: head sizes in steps of 16, odd
numbers of heads and groups, widths and vocabularies that are no power of two."""
import math

import pytest
import torch

import host_ops

pytestmark = pytest.mark.gpu


def _ops():
    from inferx_b200.kernels import ops
    return ops


def _tol(dtype, ref=None):
    """bfloat16 keeps eight bits: a result rounded once lies within 2^-9 of its value,
    and a kernel that also rounds an intermediate (an activation between two products)
    or sums rounded terms within a few times that.  The bound is 2^-7, relative to the
    element or to the largest element of the reference, whichever is larger."""
    if dtype != torch.bfloat16:
        return dict(rtol=2e-5, atol=2e-5)
    scale = float(ref.abs().max()) if ref is not None else 1.0
    return dict(rtol=2.0 ** -7, atol=2.0 ** -7 * scale)


def _close(out, ref, dtype, **kw):
    ref = ref.float()
    torch.testing.assert_close(out.float(), ref, **_tol(dtype, ref), **kw)


def _rand(shape, dtype, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    ops = _ops()
    table = _rand((301, 72), dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = ops.embed(table.cuda(), ids.cuda())
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), host_ops.embed(table, ids), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [72, 1000, 2048])
def test_add_rmsnorm(dtype, H):
    ops = _ops()
    resid = _rand((7, H), torch.float32, seed=1)
    delta = _rand((7, H), dtype, seed=2)
    gain = 1 + _rand((H,), torch.float32, 0.1, seed=3)
    r_dev = resid.clone().cuda()
    out = ops.add_rmsnorm(r_dev, delta.cuda(), gain.cuda(), 1e-5, dtype)
    r_ref = resid.clone()
    ref = host_ops.add_rmsnorm(r_ref, delta, gain, 1e-5, dtype)
    torch.testing.assert_close(r_dev.cpu(), r_ref, rtol=1e-6, atol=1e-6)
    _close(out.cpu().float(), ref.float(), dtype)
    # gather form: picks rows, adds delta, leaves the residual alone
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    before = r_dev.clone()
    out2 = ops.add_rmsnorm(r_dev, delta.cuda(), gain.cuda(), 1e-5, dtype, rows=rows.cuda())
    ref2 = host_ops.add_rmsnorm(r_ref.clone(), delta, gain, 1e-5, dtype, rows=rows)
    assert torch.equal(before, r_dev)
    _close(out2.cpu().float(), ref2.float(), dtype)
    # no delta
    out3 = ops.add_rmsnorm(r_dev, None, gain.cuda(), 1e-5, dtype)
    ref3 = host_ops.add_rmsnorm(r_ref.clone(), None, gain, 1e-5, dtype)
    _close(out3.cpu().float(), ref3.float(), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    ops = _ops()
    gu = _rand((9, 2 * 88), dtype, 2.0)
    _close(ops.silu_mul(gu.cuda()).cpu().float(), host_ops.silu_mul(gu).float(), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 50, 70), (67, 130, 45), (128, 64, 256)])
def test_linear(dtype, M, N, K):
    ops = _ops()
    x, w = _rand((M, K), dtype, seed=4), _rand((N, K), dtype, 0.2, seed=5)
    out = ops.linear(x.cuda(), w.cuda())
    ref = host_ops.linear(x, w)
    _close(out.cpu().float(), ref.float(), dtype)
    out32 = ops.linear(x.cuda(), w.cuda(), out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    torch.testing.assert_close(out32.cpu(), host_ops.linear(x, w, torch.float32),
                               rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,rot", [(5, 5, 16, 16), (6, 2, 48, 48), (3, 1, 80, 32),
                                              (4, 2, 128, 0)])
def test_qkv_rope_append(dtype, heads, kvh, hd, rot):
    ops = _ops()
    T, page, P = 11, 4, 9
    qkv = _rand((T, (heads + 2 * kvh) * hd), dtype, seed=6)
    bias = _rand(((heads + 2 * kvh) * hd,), torch.float32, 0.5, seed=7)
    positions = torch.tensor([0, 1, 2, 3, 100, 101, 7, 8, 9, 31999, 32000], dtype=torch.int32)
    inv = (10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))).float()
    slots = torch.randperm(P * page)[:T].to(torch.int32)
    kc = torch.zeros(P, kvh, page, hd, dtype=dtype)
    vc = torch.zeros_like(kc)
    kc_d, vc_d = kc.clone().cuda(), vc.clone().cuda()
    q, k, v = ops.qkv_rope_append(qkv.cuda(), bias.cuda(), positions.cuda(),
                                  inv.cuda() if rot else None, rot, heads, kvh, hd, kc_d, vc_d,
                                  slots.cuda(), want_dense_kv=True)
    qr, kr, vr = host_ops.qkv_rope_append(qkv, bias, positions, inv if rot else None, rot, heads,
                                          kvh, hd, kc, vc, slots, want_dense_kv=True)
    _close(q.cpu(), qr, dtype)
    _close(k.cpu(), kr, dtype)
    _close(v.cpu(), vr, dtype)
    _close(kc_d.cpu(), kc, dtype)
    _close(vc_d.cpu(), vc, dtype)
    # append_kv writes the same cache
    kc2, vc2 = torch.zeros_like(kc_d), torch.zeros_like(vc_d)
    ops.append_kv(k, v, kc2, vc2, slots.cuda())
    assert torch.equal(kc2, kc_d) and torch.equal(vc2, vc_d)


@pytest.mark.parametrize("heads,kvh,hd,rot", [(5, 5, 16, 16), (6, 2, 48, 48), (3, 1, 80, 32),
                                              (4, 2, 128, 0), (16, 16, 128, 128)])
def test_qkv_rope_append_many_tokens_same_bits(heads, kvh, hd, rot):
    """The rows of a long step equal the same rows run in portions of 20, bit for bit, at
    positions up to 40,000, and agree with the plain statement.  One token has no slot: its
    keys and values go nowhere."""
    ops = _ops()
    dtype = torch.bfloat16
    T, page = 150, 8
    P = T // page + 2
    width = (heads + 2 * kvh) * hd
    qkv = _rand((T, width), dtype, seed=16)
    bias = _rand((width,), torch.float32, 0.5, seed=17)
    positions = (torch.arange(T, dtype=torch.int32) * 211) % 40000
    inv = (10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))).float()
    slots = torch.randperm(P * page)[:T].to(torch.int32)
    slots[77] = -1
    kc = torch.zeros(P, kvh, page, hd, dtype=dtype)
    vc = torch.zeros_like(kc)
    inv_d = inv.cuda() if rot else None
    kc_d, vc_d = kc.clone().cuda(), vc.clone().cuda()
    q, k, v = ops.qkv_rope_append(qkv.cuda(), bias.cuda(), positions.cuda(), inv_d, rot, heads,
                                  kvh, hd, kc_d, vc_d, slots.cuda(), want_dense_kv=True)
    kc_p, vc_p = kc.clone().cuda(), vc.clone().cuda()
    for lo in range(0, T, 20):
        hi = min(T, lo + 20)
        q2, k2, v2 = ops.qkv_rope_append(qkv[lo:hi].contiguous().cuda(), bias.cuda(),
                                         positions[lo:hi].contiguous().cuda(), inv_d, rot, heads,
                                         kvh, hd, kc_p, vc_p, slots[lo:hi].contiguous().cuda(),
                                         want_dense_kv=True)
        assert torch.equal(q[lo:hi], q2) and torch.equal(k[lo:hi], k2) and torch.equal(v[lo:hi], v2)
    assert torch.equal(kc_d, kc_p) and torch.equal(vc_d, vc_p)
    qr, kr, vr = host_ops.qkv_rope_append(qkv, bias, positions, inv if rot else None, rot, heads,
                                          kvh, hd, kc, vc, slots, want_dense_kv=True)
    _close(q.cpu(), qr, dtype)
    _close(k.cpu(), kr, dtype)
    _close(kc_d.cpu(), kc, dtype)
    _close(vc_d.cpu(), vc, dtype)


def _paged_case(dtype, heads, kvh, hd, page, window, seq_lens, q_lens, seed=0):
    """Random paged caches with shuffled pages; queries are the last q_len positions."""
    g = torch.Generator().manual_seed(seed)
    S = len(seq_lens)
    maxb = max(-(-n // page) for n in seq_lens)
    P = S * maxb + 3
    perm = torch.randperm(P, generator=g)
    bt = torch.full((S, maxb), -1, dtype=torch.int32)
    kc = torch.zeros(P, kvh, page, hd)
    vc = torch.zeros(P, kvh, page, hd)
    nxt = 0
    for s, n in enumerate(seq_lens):
        for b in range(-(-n // page)):
            bt[s, b] = perm[nxt]
            nxt += 1
        for p in range(n):
            kc[bt[s, p // page], :, p % page] = torch.randn(kvh, hd, generator=g)
            vc[bt[s, p // page], :, p % page] = torch.randn(kvh, hd, generator=g)
    seq_of, pos = [], []
    for s, (n, ql) in enumerate(zip(seq_lens, q_lens)):
        seq_of += [s] * ql
        pos += list(range(n - ql, n))
    T = len(pos)
    q = torch.randn(T, heads, hd, generator=g)
    return (q.to(dtype), kc.to(dtype), vc.to(dtype), bt, torch.tensor(seq_of, dtype=torch.int32),
            torch.tensor(pos, dtype=torch.int32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,page,window", [
    (4, 2, 16, 4, 0), (3, 1, 32, 8, 8), (6, 3, 48, 16, 5), (2, 2, 128, 16, 0), (5, 1, 80, 2, 33)])
def test_paged_attention_generic(dtype, heads, kvh, hd, page, window):
    ops = _ops()
    seq_lens, q_lens = [1, 37, 200, 64], [1, 5, 1, 64]
    q, kc, vc, bt, seq_of, pos = _paged_case(dtype, heads, kvh, hd, page, window, seq_lens, q_lens)
    scale = 1.0 / math.sqrt(hd)
    out = ops.paged_attention_generic(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), seq_of.cuda(),
                                      pos.cuda(), window, scale)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, window, scale)
    _close(out.cpu().float(), ref.float(), dtype)


def test_attention_finds_one_far_key():
    """One key far back among hundreds carries the whole weight: a kernel that skips
    a page, a tile edge or the first key would miss it."""
    ops = _ops()
    heads, kvh, hd, page = 2, 1, 32, 8
    n = 700
    for far in (0, 7, 8, 127, 128, 129, 511, 699):
        q, kc, vc, bt, seq_of, pos = _paged_case(torch.float32, heads, kvh, hd, page, 0, [n], [1],
                                                 seed=far)
        kc *= 0.01
        key = torch.randn(hd) * 3
        kc[bt[0, far // page], 0, far % page] = key
        q[0, :, :] = key * 2
        marker = torch.zeros(hd)
        marker[0] = 1000.0
        vc[bt[0, far // page], 0, far % page] = marker
        out = ops.paged_attention_generic(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), seq_of.cuda(),
                                          pos.cuda(), 0, 1.0)
        ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, 0, 1.0)
        assert ref[0, 0, 0] > 900
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-3)


def test_attention_window_edge():
    """The key just outside the window must not count; the one just inside must."""
    ops = _ops()
    heads, kvh, hd, page, W = 1, 1, 16, 4, 9
    n = 40
    for which, expect_hit in ((n - W, True), (n - W - 1, False)):
        q, kc, vc, bt, seq_of, pos = _paged_case(torch.float32, heads, kvh, hd, page, W, [n], [1])
        kc *= 0.01
        key = torch.ones(hd)
        kc[bt[0, which // page], 0, which % page] = key * 4
        q[0, 0] = key * 4
        vc[:] = 0
        vc[bt[0, which // page], 0, which % page, 0] = 1.0
        out = ops.paged_attention_generic(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), seq_of.cuda(),
                                          pos.cuda(), W, 1.0)
        assert (out[0, 0, 0].item() > 0.9) == expect_hit


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,E,k,renorm", [(1, 72, 5, 2, True), (33, 200, 60, 4, False),
                                            (300, 96, 8, 3, True), (1300, 64, 7, 7, False)])
def test_router_topk(dtype, T, H, E, k, renorm):
    ops = _ops()
    x = _rand((T, H), dtype, seed=8)
    w = _rand((E, H), torch.float32, 0.3, seed=9)
    extra = _rand((H,), torch.float32, 0.3, seed=10)
    tw, ti, ex = ops.router_topk(x.cuda(), w.cuda(), k, renorm, 1.5, extra_w=extra.cuda())
    rw, ri, rex = host_ops.router_topk(x, w, k, renorm, 1.5, extra_w=extra)
    assert torch.equal(ti.cpu(), ri)
    torch.testing.assert_close(tw.cpu(), rw, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(ex.cpu(), rex, rtol=1e-4, atol=1e-4)


def test_router_ties_go_to_lower_index():
    ops = _ops()
    x = torch.ones(3, 16)
    w = torch.zeros(6, 16)
    w[1] = w[4] = 0.5       # experts 1 and 4 tie for first, the rest tie below
    tw, ti, _ = ops.router_topk(x.cuda(), w.cuda(), 3, False, 1.0)
    assert ti.cpu().tolist() == [[1, 4, 0]] * 3


@pytest.mark.parametrize("T,E,k", [(1, 4, 2), (50, 60, 4), (700, 8, 3), (2048, 60, 4)])
def test_moe_dispatch(T, E, k):
    ops = _ops()
    g = torch.Generator().manual_seed(T)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    off, rows, dest = ops.moe_dispatch(idx.cuda(), E)
    roff, rrows, rdest = host_ops.moe_dispatch(idx, E)
    assert torch.equal(off.cpu(), roff)
    assert torch.equal(rows.cpu(), rrows)
    assert torch.equal(dest.cpu(), rdest)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,I,E,k", [(1, 64, 32, 4, 2), (70, 96, 48, 8, 3), (300, 72, 40, 5, 2)])
def test_grouped_experts_and_combine(dtype, T, H, I, E, k):
    ops = _ops()
    x = _rand((T, H), dtype, seed=11)
    wgu = _rand((E, 2 * I, H), dtype, 0.2, seed=12)
    wd = _rand((E, H, I), dtype, 0.2, seed=13)
    g = torch.Generator().manual_seed(14)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    tw = torch.rand(T, k, generator=g)
    off, rows, dest = host_ops.moe_dispatch(idx, E)
    act = ops.grouped_gate_up_swiglu(x.cuda(), rows.cuda(), off.cuda(), wgu.cuda())
    ract = host_ops.grouped_gate_up_swiglu(x, rows, off, wgu)
    _close(act.cpu().float(), ract.float(), dtype)
    y = ops.grouped_down(ract.cuda(), off.cuda(), wd.cuda())
    ry = host_ops.grouped_down(ract, off, wd)
    _close(y.cpu().float(), ry.float(), dtype)
    shared = _rand((T, H), dtype, seed=15)
    logit = _rand((T,), torch.float32, 2.0, seed=16)
    out = ops.moe_combine(ry.cuda(), dest.cuda(), tw.cuda(), shared.cuda(), logit.cuda())
    rout = host_ops.moe_combine(ry, dest, tw, shared, logit)
    _close(out.cpu().float(), rout.float(), dtype)
    out2 = ops.moe_combine(ry.cuda(), dest.cuda(), tw.cuda(), None, None)
    _close(out2.cpu().float(), host_ops.moe_combine(ry, dest, tw, None, None).float(), dtype)


def test_sample_greedy_and_temperature():
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    R, V = 6, 1003
    logits = torch.randn(R, V, generator=g) * 3
    logits[2, 10] = logits[2, 900] = 50.0          # tie: lower index wins
    ids = ops.sample(logits.cuda())
    assert ids.cpu().tolist() == host_ops.sample(logits).tolist()
    assert ids[2].item() == 10
    temp = torch.tensor([0.7, 1.0, 0.0, 1.3, 0.5, 2.0])
    seeds = torch.tensor([1, 2, 3, 4, 5, 2 ** 62 + 11], dtype=torch.int64)
    a = ops.sample(logits.cuda(), temp.cuda(), seeds.cuda())
    b = ops.sample(logits.cuda(), temp.cuda(), seeds.cuda())
    assert torch.equal(a, b)                       # same seed, same draw
    ref = host_ops.sample(logits, temp, seeds)
    assert a.cpu().tolist() == ref.tolist()
    # top_k = 1 and min_p = 1 are argmax whatever the temperature
    one = torch.ones(R, dtype=torch.int32)
    hot = torch.full((R,), 1.5)
    c = ops.sample(logits.cuda(), hot.cuda(), seeds.cuda(), top_k=one.cuda())
    d = ops.sample(logits.cuda(), hot.cuda(), seeds.cuda(), min_p=torch.ones(R).cuda())
    assert c.cpu().tolist() == ids.cpu().tolist() == d.cpu().tolist()


def test_sample_distribution_and_filters():
    ops = _ops()
    V, N = 50, 4000
    logits = torch.linspace(0, 4, V).repeat(N, 1)
    seeds = torch.arange(N, dtype=torch.int64) * 7919 + 13
    temp = torch.ones(N)
    ids = ops.sample(logits.cuda(), temp.cuda(), seeds.cuda()).cpu().long()
    freq = torch.bincount(ids, minlength=V).float() / N
    p = torch.softmax(logits[0], 0)
    assert (freq - p).abs().max() < 0.03
    # top-k 5: only the five most probable tokens ever appear
    ids = ops.sample(logits.cuda(), temp.cuda(), seeds.cuda(),
                     top_k=torch.full((N,), 5, dtype=torch.int32).cuda()).cpu()
    assert ids.min().item() >= V - 5
    # top-p 0.5: the smallest head whose mass reaches 0.5
    ids = ops.sample(logits.cuda(), temp.cuda(), seeds.cuda(),
                     top_p=torch.full((N,), 0.5).cuda()).cpu()
    c = torch.cumsum(p.flip(0), 0)
    n_keep = int((c < 0.5).sum().item()) + 1
    assert ids.min().item() >= V - n_keep
    assert ids.min().item() <= V - n_keep + 1


def test_cpu_tensor_is_refused():
    ops = _ops()
    with pytest.raises(ops.KernelError):
        ops.silu_mul(torch.zeros(2, 4))
    with pytest.raises(ops.KernelError):
        ops.linear(torch.zeros(2, 4).cuda(), torch.zeros(3, 4).cuda().to(torch.bfloat16))


def _decode_forms(dtype, hd, page):
    """The kernel forms that take this case: TMA-fed and cp.async-fed tensor-core
    kernels (bf16, head size 64/128) and the scalar one."""
    forms = ["scalar"]
    if dtype == torch.bfloat16 and hd in (64, 128):
        forms.append("mma")
        if page in (8, 16, 32, 64):
            forms.append("tma")
    return forms


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,page,window,splits", [
    (4, 4, 128, 16, 0, None), (8, 2, 64, 8, 0, 3), (6, 3, 128, 16, 50, None),
    (16, 2, 64, 4, 0, 1), (3, 1, 128, 16, 7, 5), (2, 2, 256, 16, 0, None),
    (40, 2, 64, 16, 0, 2), (5, 5, 128, 12, 0, None), (6, 2, 128, 32, 0, 4),
    (4, 1, 64, 64, 100, None), (7, 7, 128, 8, 130, 2), (34, 2, 128, 16, 0, 1)])
def test_paged_attention_decode(dtype, heads, kvh, hd, page, window, splits):
    ops = _ops()
    if dtype == torch.float32 and hd == 256:
        pytest.skip("fp32 decode kernel is built for head sizes 64 and 128")
    seq_lens = [1, 37, 1000, 64, 513, 2]
    q, kc, vc, bt, seq_of, pos = _paged_case(dtype, heads, kvh, hd, page, window, seq_lens,
                                             [1] * len(seq_lens), seed=hd)
    kv_len = torch.tensor(seq_lens, dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, window, scale)
    if window > 0:
        # pages that the window has wholly passed are given back: the table says -1 there
        # and the page may hold anything
        for s, n in enumerate(seq_lens):
            for b in range(max(0, n - window) // page):
                kc[bt[s, b]] = float("nan")
                vc[bt[s, b]] = float("nan")
                bt[s, b] = -1
    tol = _tol(dtype, ref) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
    for form in _decode_forms(dtype, hd, page):
        out = ops.paged_attention_decode(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), kv_len.cuda(),
                                         max(seq_lens), window, scale, splits=splits, kernel=form)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **tol, msg=lambda m: f"{form}: {m}")
    if hasattr(ops, "check_async_errors"):
        ops.check_async_errors()


def test_decode_attention_forms_refuse_what_they_do_not_take():
    ops = _ops()
    q, kc, vc, bt, _, _ = _paged_case(torch.bfloat16, 2, 2, 128, 12, 0, [20], [1])
    with pytest.raises(ops.KernelError):
        ops.paged_attention_decode(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                   torch.tensor([20], dtype=torch.int32).cuda(), 20, 0, 1.0,
                                   kernel="tma")
    with pytest.raises(ops.KernelError):
        ops.paged_attention_decode(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                   torch.tensor([20], dtype=torch.int32).cuda(), 20, 0, 1.0,
                                   kernel="other")


def test_decode_attention_finds_one_far_key():
    ops = _ops()
    heads, kvh, hd, page = 4, 2, 128, 16
    n = 3000
    for far in (0, 15, 16, 255, 256, 1023, 1024, 2999):
        q, kc, vc, bt, seq_of, pos = _paged_case(torch.bfloat16, heads, kvh, hd, page, 0, [n], [1],
                                                 seed=far)
        kc = kc * 0.01
        key = torch.randn(hd)
        kc[bt[0, far // page], :, far % page] = key.to(torch.bfloat16)
        q[0, :, :] = (key * 2).to(torch.bfloat16)
        vc[bt[0, far // page], :, far % page, 0] = 1000.0
        ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, 0, 1.0)
        assert ref[0, 0, 0] > 900
        for form in ("tma", "mma", "scalar"):
            out = ops.paged_attention_decode(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                             torch.tensor([n], dtype=torch.int32).cuda(), n, 0,
                                             1.0, kernel=form)
            torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=1.0)


def test_decode_attention_long_context_many_splits():
    """Twenty thousand keys of one sequence (dozens of key splits, more than a thousand
    pages of 8 in a shuffled table): one marked key near either end and in the middle."""
    ops = _ops()
    heads, kvh, hd, page = 8, 1, 64, 8
    n = 20011
    q, kc, vc, bt, seq_of, pos = _paged_case(torch.bfloat16, heads, kvh, hd, page, 0, [n], [1],
                                             seed=9)
    kc = kc * 0.01
    key = torch.randn(hd)
    q[0, :, :] = (key * 2).to(torch.bfloat16)
    for far in (3, 9999, 20010):
        kcf, vcf = kc.clone(), vc.clone()
        kcf[bt[0, far // page], :, far % page] = key.to(torch.bfloat16)
        vcf[bt[0, far // page], :, far % page, 0] = 1000.0
        ref = host_ops.paged_attention_generic(q, kcf, vcf, bt, seq_of, pos, 0, 1.0)
        assert ref[0, 0, 0] > 900
        for form in ("tma", "mma", "scalar"):
            out = ops.paged_attention_decode(q.cuda(), kcf.cuda(), vcf.cuda(), bt.cuda(),
                                             torch.tensor([n], dtype=torch.int32).cuda(), n, 0,
                                             1.0, kernel=form)
            torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=1.0,
                                       msg=lambda m: f"{form}, key {far}: {m}")
    ops.check_async_errors()


@pytest.mark.parametrize("T,H,I,E,k", [(1, 64, 32, 4, 2), (9, 200, 72, 8, 3), (40, 96, 48, 60, 4),
                                       (16, 2048, 1408, 6, 2), (8, 264, 328, 60, 4),
                                       (3, 1000, 256, 33, 2), (20, 512, 520, 5, 3)])
def test_small_m_grouped_experts(T, H, I, E, k):
    """The weight-streaming kernel (few rows per expert) against the plain statement,
    including an expert with more rows than one chunk holds."""
    ops = _ops()
    dtype = torch.bfloat16
    x = _rand((T, H), dtype, seed=21)
    wgu = _rand((E, 2 * I, H), dtype, 0.1, seed=22)
    wd = _rand((E, H, I), dtype, 0.1, seed=23)
    g = torch.Generator().manual_seed(24)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    if T >= 9:
        idx[:, 0] = 1          # one expert gets every token: more rows than a chunk
        idx[:, 1:] = torch.where(idx[:, 1:] == 1, torch.zeros_like(idx[:, 1:]), idx[:, 1:])
        for t in range(T):     # keep the k experts of a token distinct
            seen, row = set(), idx[t].tolist()
            for j, e in enumerate(row):
                while e in seen:
                    e = (e + 1) % E
                seen.add(e)
                row[j] = e
            idx[t] = torch.tensor(row, dtype=torch.int32)
    off, rows, dest = host_ops.moe_dispatch(idx, E)
    ract = host_ops.grouped_gate_up_swiglu(x, rows, off, wgu)
    ry = host_ops.grouped_down(ract, off, wd)
    forms = [ops.gemm_small_m]
    if H >= 256 and I >= 256:       # the persistent form splits K over eight warps
        forms.append(ops.gemm_stream_grouped)
    for form in forms:
        for per_pass in (8, 16):
            act = form(x.cuda(), wgu.cuda(), rows.cuda(), off.cuda(), True, rows.numel(),
                       rows_per_pass=per_pass)
            _close(act.cpu().float(), ract.float(), dtype)
            y = form(ract.cuda(), wd.cuda(), None, off.cuda(), False, ract.shape[0],
                     rows_per_pass=per_pass)
            _close(y.cpu().float(), ry.float(), dtype)


def test_stream_grouped_refuses_short_k():
    ops = _ops()
    with pytest.raises(ops.KernelError):
        ops.gemm_stream_grouped(torch.zeros(4, 128, dtype=torch.bfloat16).cuda(),
                                torch.zeros(2, 16, 128, dtype=torch.bfloat16).cuda(), None,
                                torch.tensor([0, 2, 4], dtype=torch.int32).cuda(), False, 4)


@pytest.mark.parametrize("M,N,K", [(1, 50, 72), (8, 130, 200), (13, 64, 256), (16, 1000, 2048),
                                   (3, 300, 5632), (29, 90, 1408), (32, 48, 40)])
def test_small_m_dense(M, N, K):
    ops = _ops()
    dtype = torch.bfloat16
    x, w = _rand((M, K), dtype, seed=31), _rand((N, K), dtype, 0.1, seed=32)
    out = ops.linear(x.cuda(), w.cuda())
    _close(out.cpu().float(), host_ops.linear(x, w).float(), dtype)
    out32 = ops.linear(x.cuda(), w.cuda(), out_dtype=torch.float32)
    torch.testing.assert_close(out32.cpu(), host_ops.linear(x, w, torch.float32),
                               rtol=1e-3, atol=1e-3)
    if K % 8 == 0:
        # the streaming kernel itself, whatever ``linear`` chose for this row count
        per_pass = 8 if M <= 8 else (16 if M <= 16 else 32)
        direct = ops.gemm_small_m(x.cuda(), w.cuda().unsqueeze(0), None, None, False, M,
                                  rows_per_pass=per_pass)
        _close(direct.cpu().float(), host_ops.linear(x, w).float(), dtype)
    if N % 2 == 0:
        act = ops.gate_up_swiglu(x.cuda(), w.cuda())
        _close(act.cpu().float(), host_ops.gate_up_swiglu(x, w).float(), dtype)


@pytest.mark.parametrize("T,H", [(600, 256), (1024, 256), (1412, 136), (2050, 136), (1800, 4096),
                                 (1180, 4096), (2048, 2048)])
def test_router_paths_agree_bitwise(T, H):
    """Few tokens take the two-kernel router, many the fused one with 4 to 16 tokens a block
    (1024 tokens: 8 a block; 1412: 10; 1800: 14, 1180: 8, and at a width of 4096 the tile of
    bfloat16 where the widened one does not fit; 2050: 14): same routing, same bits."""
    ops = _ops()
    x = _rand((T, H), torch.bfloat16, seed=41).cuda()
    w = _rand((60, H), torch.float32, 0.3, seed=42).cuda()
    extra = _rand((H,), torch.float32, 0.3, seed=43).cuda()
    tw, ti, ex = ops.router_topk(x, w, 4, False, 1.0, extra_w=extra)
    for lo in (0, T - 40):
        part = x[lo:lo + 40].contiguous()
        tw2, ti2, ex2 = ops.router_topk(part, w, 4, False, 1.0, extra_w=extra)
        assert torch.equal(ti[lo:lo + 40], ti2) and torch.equal(tw[lo:lo + 40], tw2)
        assert torch.equal(ex[lo:lo + 40], ex2)
    want_w, want_i = host_ops.router_topk(x.cpu(), w.cpu(), 4, False, 1.0)[:2]
    same = (ti.cpu() == want_i).all(dim=1)
    assert same.float().mean() > 0.995            # a near-tie may fall the other way
    torch.testing.assert_close(tw.cpu()[same], want_w[same], rtol=1e-4, atol=1e-6)


def _prefill_forms(page):
    """The mma.sync form takes any page size, the tcgen05 form powers of two from 8 to 64."""
    return ["mma", "tc"] if page in (8, 16, 32, 64) else ["mma"]


@pytest.mark.parametrize("heads,kvh,hd,page,window", [
    (4, 2, 128, 16, 0), (3, 1, 64, 8, 0), (2, 2, 128, 4, 40), (6, 3, 64, 16, 7),
    (2, 1, 128, 16, 100), (5, 5, 128, 32, 0), (2, 1, 64, 64, 260), (3, 3, 128, 8, 33)])
def test_paged_attention_prefill(heads, kvh, hd, page, window):
    """Ragged batch: whole prompts, a portion deep in a sequence, single tokens."""
    ops = _ops()
    dtype = torch.bfloat16
    seq_lens, q_lens = [150, 1, 333, 64, 65, 700, 520], [150, 1, 70, 64, 2, 1, 390]
    q, kc, vc, bt, seq_of, pos = _paged_case(dtype, heads, kvh, hd, page, window, seq_lens, q_lens,
                                             seed=hd + window)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    cu_q = torch.tensor(cu, dtype=torch.int32)
    q_pos0 = torch.tensor([n - ql for n, ql in zip(seq_lens, q_lens)], dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, window, scale)
    if window > 0:
        # pages that the window of the first query of the step has wholly passed are given
        # back: the table says -1 there and the page may hold anything
        for s, (n, ql) in enumerate(zip(seq_lens, q_lens)):
            for b in range(max(0, n - ql - window + 1) // page):
                kc[bt[s, b]] = float("nan")
                vc[bt[s, b]] = float("nan")
                bt[s, b] = -1
    for form in _prefill_forms(page):
        out = ops.paged_attention_prefill(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cu_q.cuda(),
                                          q_pos0.cuda(), window, scale, kernel=form)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(torch.bfloat16, ref),
                                   msg=lambda m: f"{form}: {m}")
    if "tc" in _prefill_forms(page):
        # the keys of every query tile cut into runs (some of them empty, some wholly
        # masked for the earlier queries of the tile) and merged
        for splits in (2, 3, 7):
            out = ops.paged_attention_prefill(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                              cu_q.cuda(), q_pos0.cuda(), window, scale,
                                              kernel="tc", splits=splits)
            torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(torch.bfloat16, ref),
                                       msg=lambda m: f"tc, {splits} runs: {m}")
    ops.check_async_errors()


def test_short_portion_over_a_long_context_is_cut_into_runs():
    """70 queries at the end of 5,000 keys: few (query tile, head) items, so the tcgen05
    form cuts the keys into runs by itself (two launches); one far key is marked so that
    a run that was dropped or merged with the wrong weight shows."""
    ops = _ops()
    heads, kvh, hd, page = 4, 2, 128, 16
    n, ql = 5000, 70
    q, kc, vc, bt, seq_of, pos = _paged_case(torch.bfloat16, heads, kvh, hd, page, 0, [n], [ql],
                                             seed=11)
    far = 1234
    kc[bt[0, far // page], :, far % page] *= 3.0
    cu_q = torch.tensor([0, ql], dtype=torch.int32)
    q_pos0 = torch.tensor([n - ql], dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, 0, scale)
    assert ops._lib().ix_attn_prefill_tc_splits(ql, 1, heads, n, 0) > 1
    before = ops.LAUNCHES[0]
    out = ops.paged_attention_prefill(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cu_q.cuda(),
                                      q_pos0.cuda(), 0, scale, kernel="tc")
    assert ops.LAUNCHES[0] - before == 2
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(torch.bfloat16, ref))
    one = ops.paged_attention_prefill(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cu_q.cuda(),
                                      q_pos0.cuda(), 0, scale, kernel="tc", splits=1)
    torch.testing.assert_close(one.cpu().float(), ref.float(), **_tol(torch.bfloat16, ref))
    ops.check_async_errors()


def test_mixed_batch_goes_to_both_attention_kernels():
    """ops.paged_attention on a batch whose first sequences bring one token each: those
    go to the split-KV kernel, the prompt portions to the tiled one, and the result is
    that of the general kernel on the whole batch."""
    import types
    ops = _ops()
    heads, kvh, hd, page, window = 6, 2, 128, 16, 90
    seq_lens, q_lens = [700, 33, 1, 150, 400, 65], [1, 1, 1, 150, 70, 2]
    q, kc, vc, bt, seq_of, pos = _paged_case(torch.bfloat16, heads, kvh, hd, page, window,
                                             seq_lens, q_lens, seed=77)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    nd = 3
    step = types.SimpleNamespace(
        num_seqs=len(seq_lens), num_tokens=cu[-1], all_decode=False, num_decode_seqs=nd,
        seq_of_token=seq_of.cuda(), positions=pos.cuda(),
        cu_q=torch.tensor(cu, dtype=torch.int32).cuda(),
        cu_q_prompt=torch.tensor([c - cu[nd] for c in cu[nd:]], dtype=torch.int32).cuda(),
        q_pos0=torch.tensor([n - ql for n, ql in zip(seq_lens, q_lens)], dtype=torch.int32).cuda(),
        kv_len=torch.tensor(seq_lens, dtype=torch.int32).cuda(),
        max_q_len=max(q_lens), max_kv_len=max(seq_lens))
    scale = 1.0 / math.sqrt(hd)
    before = ops.LAUNCHES[0]
    out = ops.paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), step, window, scale)
    assert ops.LAUNCHES[0] - before >= 2      # two kernels (and a merge when keys are split)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, window, scale)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(torch.bfloat16, ref))
    step.num_decode_seqs = 0          # the same through the tiled kernel alone
    out2 = ops.paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), step, window, scale)
    torch.testing.assert_close(out2.cpu().float(), ref.float(), **_tol(torch.bfloat16, ref))
    ops.check_async_errors()


def test_prefill_attention_rescales_when_the_max_grows():
    """Scores that climb by far more than the lazy-rescale step from tile to tile, then
    fall: the running max of the tcgen05 form has to follow them."""
    ops = _ops()
    heads, kvh, hd, page = 2, 1, 128, 16
    n = 600
    q, kc, vc, bt, seq_of, pos = _paged_case(torch.bfloat16, heads, kvh, hd, page, 0, [n], [n],
                                             seed=5)
    ramp = torch.cat([torch.linspace(0.05, 3.0, 400), torch.linspace(3.0, 0.2, 200)])
    for p in range(n):
        kc[bt[0, p // page], :, p % page] *= ramp[p]
    cu_q = torch.tensor([0, n], dtype=torch.int32)
    q_pos0 = torch.tensor([0], dtype=torch.int32)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, 0, 1.0)
    for form in ("mma", "tc"):
        out = ops.paged_attention_prefill(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cu_q.cuda(),
                                          q_pos0.cuda(), 0, 1.0, kernel=form)
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=3e-2, atol=3e-2,
                                   msg=lambda m: f"{form}: {m}")
    ops.check_async_errors()


def test_prefill_attention_window_edge_and_far_key():
    """A marked key just inside / just outside the window of one query in a long
    portion, and a far key without a window."""
    ops = _ops()
    heads, kvh, hd, page = 1, 1, 64, 16
    n, ql = 300, 130
    for window, which, qrow, expect in ((50, 299 - 49 - 20, 129 - 20, True),
                                        (50, 299 - 50 - 20, 129 - 20, False),
                                        (0, 3, 129, True), (0, 64, 0, True), (0, 171, 0, False)):
        q, kc, vc, bt, seq_of, pos = _paged_case(torch.bfloat16, heads, kvh, hd, page, window, [n],
                                                 [ql], seed=which)
        kc = kc * 0.01
        vc = vc * 0.0
        key = torch.ones(hd)
        kc[bt[0, which // page], 0, which % page] = (key * 4).to(torch.bfloat16)
        vc[bt[0, which // page], 0, which % page, 0] = 1.0
        q = q * 0.01
        q[qrow, 0] = (key * 4).to(torch.bfloat16)
        cu_q = torch.tensor([0, ql], dtype=torch.int32)
        q_pos0 = torch.tensor([n - ql], dtype=torch.int32)
        for form in ("mma", "tc"):
            out = ops.paged_attention_prefill(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                              cu_q.cuda(), q_pos0.cuda(), window, 1.0, kernel=form)
            assert (out[qrow, 0, 0].item() > 0.9) == expect, (form, window, which, qrow)


@pytest.mark.parametrize("T,K,heads,kvh,hd,rot,bias,page", [
    (1, 2048, 16, 16, 128, 128, True, 16), (8, 2048, 16, 16, 128, 128, True, 16),
    (16, 3584, 28, 4, 128, 128, True, 16), (5, 200, 3, 1, 64, 64, False, 8),
    (9, 96, 2, 2, 32, 0, True, 4), (13, 1032, 7, 7, 96, 96, True, 12)])
def test_qkv_projection_with_rotation_and_cache_write_in_one_launch(T, K, heads, kvh, hd, rot,
                                                                    bias, page):
    """The fused kernel of few-token steps against the two kernels it replaces (the same
    bits: the projection is rounded to bfloat16 where the tensor between them would be)
    and against the plain statement."""
    ops = _ops()
    g = torch.Generator().manual_seed(T + K)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    width = (heads + 2 * kvh) * hd
    w = (torch.randn(width, K, generator=g) * (1.0 / math.sqrt(K))).to(torch.bfloat16)
    b = torch.randn(width, generator=g) * 0.3 if bias else None
    positions = torch.randint(0, 5000, (T,), generator=g).to(torch.int32)
    inv = (10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))).float() \
        if rot else None
    pages = T + 3
    slots = (torch.randperm(pages * page, generator=g)[:T]).to(torch.int32)
    kc = torch.randn(pages, kvh, page, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(pages, kvh, page, hd, generator=g).to(torch.bfloat16)
    assert ops.qkv_project_applies(x.cuda(), w.cuda(), heads, kvh, hd, rot)
    kc1, vc1 = kc.cuda(), vc.cuda()
    launched = ops.LAUNCHES[0]
    q1 = ops.qkv_project_rope_append(x.cuda(), w.cuda(), None if b is None else b.cuda(),
                                     positions.cuda(), None if inv is None else inv.cuda(), rot,
                                     heads, kvh, hd, kc1, vc1, slots.cuda())
    assert ops.LAUNCHES[0] - launched == 1
    # the two kernels it replaces
    kc2, vc2 = kc.cuda(), vc.cuda()
    qkv = ops.linear(x.cuda(), w.cuda())
    q2 = ops.qkv_rope_append(qkv, None if b is None else b.cuda(), positions.cuda(),
                             None if inv is None else inv.cuda(), rot, heads, kvh, hd, kc2, vc2,
                             slots.cuda())
    # the plain statement, from the plain product
    kc3, vc3 = kc.clone(), vc.clone()
    q3, _, _ = host_ops.qkv_rope_append(host_ops.linear(x, w), b, positions, inv, rot, heads, kvh,
                                        hd, kc3, vc3, slots, want_dense_kv=True)
    _close(q1.cpu(), q3, torch.bfloat16)
    _close(kc1.cpu(), kc3, torch.bfloat16)
    _close(vc1.cpu(), vc3, torch.bfloat16)
    # rows of the cache that no slot names are untouched
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[slots.long()] = False
    flat = lambda c: c.permute(0, 2, 1, 3).reshape(pages * page, kvh * hd)
    assert torch.equal(flat(kc1.cpu())[untouched], flat(kc)[untouched])
    assert torch.equal(flat(vc1.cpu())[untouched], flat(vc)[untouched])
    # against the separate kernels: the same sums in the same order when both split K the
    # same way; otherwise equal within one rounding of the projection
    same = (q1 == q2).float().mean().item()
    assert same > 0.98, same
    _close(q1.cpu(), q2.cpu(), torch.bfloat16)
    _close(kc1.cpu(), kc2.cpu(), torch.bfloat16)


def _close_sum(out, ref, dtype):
    """For sums of many terms: in 32-bit two orders of summation differ by rounding that
    grows with the size of the sums, so the bound is 2e-5 of the largest element of the
    reference (the bound the model tests use for logits); bfloat16 as everywhere."""
    if dtype == torch.bfloat16:
        return _close(out, ref, dtype)
    bound = 2e-5 * float(ref.abs().max())
    err = float((out.float() - ref.float()).abs().max())
    assert err <= bound, f"max error {err:.3e} exceeds {bound:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 37, 50), (9, 130, 64), (16, 256, 2048), (17, 100, 96),
                                   (70, 64, 33), (300, 193, 260), (129, 129, 1000)])
def test_cuda_core_product_single_matrix(dtype, M, N, K):
    """The product of the 32-bit mode for one matrix, plain and with the SwiGLU folded
    in: the weight-streaming kernel (up to 16 rows) and the tiled kernel, at sizes that
    are no multiple of a tile, of four (no vector loads) or of anything."""
    ops = _ops()
    x, w = _rand((M, K), dtype, seed=M + N), _rand((N, K), dtype, 0.2, seed=K)
    out = ops.gemm_generic(x.cuda(), w.cuda().unsqueeze(0), None, None, dual=False)
    _close_sum(out.cpu(), host_ops.linear(x, w).float(), dtype)
    if N % 2 == 0:
        act = ops.gemm_generic(x.cuda(), w.cuda().unsqueeze(0), None, None, dual=True)
        _close_sum(act.cpu(), host_ops.gate_up_swiglu(x, w).float(), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,I,E,k", [(3, 64, 40, 6, 2), (40, 100, 36, 5, 3), (700, 96, 50, 4, 2)])
def test_cuda_core_product_grouped(dtype, T, H, I, E, k):
    """The same for experts: a few rows an expert (weights streamed once), dozens (64-row
    tiles) and hundreds (128-row tiles); empty experts; rows gathered through a list."""
    ops = _ops()
    g = torch.Generator().manual_seed(T)
    idx = torch.stack([torch.randperm(E - 1, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    off, rows, dest = host_ops.moe_dispatch(idx, E)          # the last expert gets no rows
    x = _rand((T, H), dtype, seed=1)
    wgu, wd = _rand((E, 2 * I, H), dtype, 0.2, seed=2), _rand((E, H, I), dtype, 0.2, seed=3)
    act = ops.gemm_generic(x.cuda(), wgu.cuda(), rows.cuda(), off.cuda(), dual=True,
                           num_out_rows=T * k)
    ract = host_ops.grouped_gate_up_swiglu(x, rows, off, wgu)
    _close_sum(act.cpu(), ract.float(), dtype)
    y = ops.gemm_generic(ract.cuda(), wd.cuda(), None, off.cuda(), dual=False, num_out_rows=T * k)
    _close_sum(y.cpu(), host_ops.grouped_down(ract, off, wd).float(), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,page,window", [
    (4, 2, 16, 4, 0), (3, 1, 32, 8, 8), (6, 3, 48, 16, 5), (2, 2, 128, 16, 0), (5, 1, 80, 2, 33),
    (2, 1, 256, 16, 100), (7, 7, 96, 12, 0), (4, 2, 112, 64, 70)])
def test_paged_attention_tiled(dtype, heads, kvh, hd, page, window):
    """The tiled CUDA-core kernel on a ragged batch: whole prompts, a portion that starts
    deep in its sequence, a two-token portion, a single token; query tiles that end inside
    a key tile; pages behind the window given back (block table -1, contents poisoned)."""
    ops = _ops()
    seq_lens, q_lens = [150, 1, 333, 64, 65, 700, 97], [150, 1, 70, 64, 2, 1, 33]
    q, kc, vc, bt, seq_of, pos = _paged_case(dtype, heads, kvh, hd, page, window, seq_lens, q_lens,
                                             seed=hd + window)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    q_pos0 = torch.tensor([n - ql for n, ql in zip(seq_lens, q_lens)], dtype=torch.int32)
    scale = 1.0 / math.sqrt(hd)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, seq_of, pos, window, scale)
    if window > 0:
        kc, vc, bt = kc.clone(), vc.clone(), bt.clone()
        for s, (n, ql) in enumerate(zip(seq_lens, q_lens)):
            # pages no query of this step can see: wholly before the first query's window
            for b in range(max(0, n - ql - window + 1) // page):
                kc[bt[s, b]] = float("nan")
                vc[bt[s, b]] = float("nan")
                bt[s, b] = -1
    out = ops.paged_attention_tiled(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                    torch.tensor(cu, dtype=torch.int32).cuda(), q_pos0.cuda(),
                                    window, scale)
    assert torch.isfinite(out).all()
    if dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-5)
    else:
        _close(out.cpu(), ref, dtype)


@pytest.mark.parametrize("R,V,H,M", [(1, 97, 5, 2), (4, 1000, 256, 16), (3, 151936, 40, 3)])
def test_apply_penalties(R, V, H, M):
    """Penalties over a row's distinct generated tokens and the mask under min_tokens,
    against the plain statement; rows whose penalties are neutral, padding ids, ids past
    the vocabulary and a token that is both penalised and masked."""
    ops = _ops()
    g = torch.Generator().manual_seed(R * V)
    logits = torch.randn(R, V, generator=g) * 4
    ids = torch.full((R, H), -1, dtype=torch.int32)
    counts = torch.zeros((R, H), dtype=torch.int32)
    pen = torch.tensor([[0.0, 0.0, 1.0]] * R)
    mask = torch.full((R, M), -1, dtype=torch.int32)
    for r in range(R):
        n = int(torch.randint(1, H + 1, (1,), generator=g))
        ids[r, :n] = torch.randperm(V, generator=g)[:n].to(torch.int32)
        counts[r, :n] = torch.randint(1, 9, (n,), generator=g).to(torch.int32)
        if r != 1:                              # row 1 keeps neutral penalties
            pen[r] = torch.tensor([0.7, 0.3, 1.6]) if r % 2 == 0 else torch.tensor([-0.5, 0.0, 0.8])
        if r % 2 == 0:
            mask[r, 0] = ids[r, 0]              # penalised and masked: masked wins
            if M > 1:
                mask[r, 1] = V - 1
    if H > 3:
        ids[0, 2] = V + 5                       # past the vocabulary: ignored
    ref = logits.clone()
    host_ops.apply_penalties(ref, ids, counts, pen, mask)
    out = logits.clone().cuda()
    ops.apply_penalties(out, ids.cuda(), counts.cuda(), pen.cuda(), mask.cuda())
    # to rounding: the device contracts the frequency term into one multiply-add
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-6, atol=1e-6)
    untouched = ref == logits
    assert torch.equal(out.cpu()[untouched], logits[untouched])
    assert torch.isinf(ref[0, int(mask[0, 0])]) and (ref != logits).any()
    only_mask = logits.clone().cuda()
    ops.apply_penalties(only_mask, None, None, None, mask.cuda())
    ref2 = logits.clone()
    host_ops.apply_penalties(ref2, None, None, None, mask)
    assert torch.equal(only_mask.cpu(), ref2)


@pytest.mark.parametrize("R,V,top", [(2, 97, 5), (5, 1000, 20), (3, 151936, 7), (2, 33, 0)])
def test_token_logprobs(R, V, top):
    """log softmax of the chosen token and the most probable alternatives (ties to the
    lower id) against the plain statement; rows that ask for fewer or for none, tied
    logits, masked (-inf) entries."""
    import plain_qwen2_moe as plain
    ops = _ops()
    g = torch.Generator().manual_seed(V + top)
    logits = torch.randn(R, V, generator=g) * 3
    logits[0, 5] = logits[0, 3] = logits[0].max() + 1.0      # a tie at the top: 3 before 5
    logits[-1, 7] = float("-inf")
    chosen = torch.randint(0, V, (R,), generator=g).to(torch.int32)
    chosen[0] = 5
    want = torch.tensor([top, -1, max(top - 2, 0), 0, top][:R], dtype=torch.int32)
    lp, ids, lps = ops.token_logprobs(logits.cuda(), chosen.cuda(), want.cuda(), top)
    lp = lp.cpu()
    for r in range(R):
        k = int(want[r])
        if k < 0:
            continue
        ref_lp, ref_top = plain.logprobs(logits[r], int(chosen[r]), k)
        assert abs(float(lp[r]) - ref_lp) <= 2e-5 * max(1.0, abs(ref_lp))
        if top:
            got_ids, got_lps = ids[r].cpu().tolist(), lps[r].cpu().tolist()
            assert got_ids[:k] == [t for t, _ in ref_top]
            assert all(t == -1 for t in got_ids[k:])
            for a, (_, b) in zip(got_lps[:k], ref_top):
                assert abs(a - b) <= 2e-5 * max(1.0, abs(b))
    if top >= 2:
        assert ids[0, :2].cpu().tolist() == [3, 5]
    # chosen token only, every row
    lp_all, none_ids, _ = ops.token_logprobs(logits.cuda(), chosen.cuda())
    assert none_ids is None
    for r in range(R):
        ref_lp, _ = plain.logprobs(logits[r], int(chosen[r]), 0)
        assert abs(float(lp_all[r]) - ref_lp) <= 2e-5 * max(1.0, abs(ref_lp))
