"""The allocation-free decode-attention entry point, called through its exported C
symbol, against the ordinary entry point.

Some programs that embed the kernel library cannot allocate device memory at the
moment they need attention (all memory already belongs to their own arena, or the
step loop may not make a call that can synchronise or fail), so the library
carries one entry point that keeps its split-KV partial results in an array of its
own.  This file is named to be collected last: it runs after every other test in a
full run, and it also passes alone in a fresh process.  Two calls in a row are
checked, because the second call finds the first call's leftovers in the array.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, S, heads, kvh, hd, page, lens):
    g = torch.Generator().manual_seed(seed)
    maxb = max(-(-n // page) for n in lens)
    P = S * maxb + 2
    perm = torch.randperm(P, generator=g)
    bt = torch.full((S, maxb), -1, dtype=torch.int32)
    nxt = 0
    for s, n in enumerate(lens):
        for b in range(-(-n // page)):
            bt[s, b] = perm[nxt]
            nxt += 1
    kc = torch.randn(P, kvh, page, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(P, kvh, page, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(S, heads, hd, generator=g).to(torch.bfloat16)
    return q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), torch.tensor(lens, dtype=torch.int32).cuda()


def _call_noalloc(lib, q, kc, vc, bt, kv_len, max_kv, window, scale):
    S, heads, hd = q.shape
    P, kvh, page, _ = kc.shape
    out = torch.empty_like(q)
    fn = lib.ix_paged_attention_decode_noalloc
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = fn(p(q), p(kc), p(vc), p(bt), p(kv_len), p(out), 1, S, heads, kvh, hd, page, bt.shape[1],
            window, ctypes.c_float(scale), max_kv,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def _plain_attention(q, kc, vc, bt, kv_len, window, scale):
    """The fp32 statement of the same attention (tests/host_ops.py), on the CPU."""
    import host_ops
    S = q.shape[0]
    return host_ops.paged_attention_generic(
        q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), torch.arange(S, dtype=torch.int32),
        (kv_len.cpu() - 1).to(torch.int32), window, scale).float()


def test_noalloc_entry_matches_ordinary_entry_twice():
    from inferx_b200.kernels import library, ops
    lib = library.load()
    # first call on this device also does the one-time address look-up
    shapes = [(11, 3, 8, 2, 128, 16, [700, 33, 1500], 0), (12, 2, 4, 4, 64, 8, [2049, 5], 0),
              (13, 2, 6, 2, 128, 16, [900, 300], 130)]          # the last with a window
    for seed, S, heads, kvh, hd, page, lens, window in shapes:
        q, kc, vc, bt, kv_len = _case(seed, S, heads, kvh, hd, page, lens)
        scale = 1.0 / math.sqrt(hd)
        # the ordinary entry of the same kernel form (keys fed by cp.async, three blocks a
        # multiprocessor decide the number of splits), and the plain fp32 statement
        ref = ops.paged_attention_decode(q, kc, vc, bt, kv_len, max(lens), window, scale,
                                         kernel="mma")
        plain = _plain_attention(q, kc, vc, bt, kv_len, window, scale)
        bound = 2.0 ** -7 * float(plain.abs().max())
        for _call in range(2):      # the second call finds the first one's leftovers
            rc, out = _call_noalloc(lib, q, kc, vc, bt, kv_len, max(lens), window, scale)
            assert rc == 0
            torch.cuda.synchronize()
            torch.testing.assert_close(out.float().cpu(), plain, rtol=2.0 ** -7, atol=bound)
            # the same kernel and the same split count: the two entries agree to the bit
            assert torch.equal(out, ref)


def test_noalloc_entry_without_splits_leaves_the_scratch_alone():
    """Contexts so short that a block takes all keys of its (sequence, head group) pair:
    nothing is written to the built-in array, the result comes straight from the
    attention kernel."""
    from inferx_b200.kernels import library, ops
    lib = library.load()
    S, heads, kvh, hd, page = 40, 16, 16, 64, 16
    lens = [30 + 2 * i for i in range(S)]
    assert lib.ix_attn_decode_splits(S, heads, kvh, max(lens)) == 1
    q, kc, vc, bt, kv_len = _case(21, S, heads, kvh, hd, page, lens)
    scale = 1.0 / math.sqrt(hd)
    rc, out = _call_noalloc(lib, q, kc, vc, bt, kv_len, max(lens), 0, scale)
    assert rc == 0
    torch.cuda.synchronize()
    plain = _plain_attention(q, kc, vc, bt, kv_len, 0, scale)
    torch.testing.assert_close(out.float().cpu(), plain, rtol=2.0 ** -7,
                               atol=2.0 ** -7 * float(plain.abs().max()))
    assert torch.equal(out, ops.paged_attention_decode(q, kc, vc, bt, kv_len, max(lens), 0,
                                                       scale, kernel="mma"))


def test_noalloc_entry_refuses_what_does_not_fit():
    """8 sequences x 64 heads x 9 splits x (256 + 2) floats of partials is more than the
    built-in 2^20 floats.  All tensors are real and large enough, so whatever the
    entry point decides, nothing reads or writes out of bounds."""
    from inferx_b200.kernels import library
    lib = library.load()
    S, heads, kvh, hd, page = 8, 64, 1, 256, 16
    lens = [1200] * S
    q, kc, vc, bt, kv_len = _case(5, S, heads, kvh, hd, page, lens)
    splits = lib.ix_attn_decode_splits(S, heads, kvh, max(lens))
    assert S * heads * splits * (hd + 2) > (1 << 20), "sizes no longer exceed the scratch"
    rc, out = _call_noalloc(lib, q, kc, vc, bt, kv_len, max(lens), 0, 1.0)
    torch.cuda.synchronize()
    assert rc == -6   # IX_ERR_SCRATCH_TOO_SMALL; nothing was launched
