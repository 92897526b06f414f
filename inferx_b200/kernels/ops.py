"""Python faces of the CUDA kernels: argument checks, output allocation, launch.

Every function takes CUDA tensors and launches on torch's current stream, so a
step can be captured into a CUDA graph.  A CPU tensor, a non-contiguous tensor,
a wrong element type or a size the kernel does not take raises; nothing here
falls back to a library implementation.

Matrix products without a fused epilogue go to cuBLAS through ``torch`` in the
bfloat16 mode, where the reference engine also calls a library
(src/backends/cuda/ops/gemm_cublaslt.cc:391-396); the 32-bit mode runs the
library's own fp32 FFMA kernel so that no reduced-precision matrix mode can
enter.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import library

# The library GEMM behind ``torch.mm`` may add its split-K partial sums in bf16; sums are
# to be fp32 here (a small result of large terms otherwise carries the rounding of the
# terms).  A process-wide torch setting: this package turns it off where it is imported.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

F32, BF16 = 0, 1

_ERRORS = {
    -1: "element type not supported by this kernel",
    -2: "a size this kernel does not take",
    -3: "pointer or stride not aligned as the kernel requires",
    -4: "shared memory need exceeds the device limit for these sizes",
    -5: "this combination of options is not built",
}


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {t.dtype} is not float32 or bfloat16")


def _chk(name: str, t: Optional[torch.Tensor], dtype=None, optional: bool = False):
    if t is None:
        if optional:
            return
        raise KernelError(f"{name}: tensor required")
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise KernelError(
            f"{name}: tensor is on {t.device}; the kernels run on a CUDA device only "
            "(there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous, strides {t.stride()}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current CUDA stream's handle.  ``torch.cuda.current_stream()`` costs several
    microseconds of Python per call (device lookups, a Stream object); with a few hundred
    launches in an eager step that adds up, so the raw getter is used where torch has it."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str):
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _lib():
    return library.load()


LAUNCHES = [0]        # launches of this library's own kernels issued through this module
LIBRARY_CALLS = [0]   # matrix products handed to cuBLAS


def _count(n: int = 1):
    LAUNCHES[0] += n


# Steps of at most this many tokens launch their kernels with programmatic stream
# serialisation, and their dense projections stream the weights with this library's own
# kernel (SMALL_M_DENSE_ROWS below is the same number on purpose).  Beyond it the dense
# projections go to the library GEMM and dependent launch is off: a step that mixes
# dependent launches with the library's plain launches measured far slower than either
# (batch 32: 11.7 ms mixed, 9.8 ms own kernels + dependent launch, 9.2 ms library GEMMs
# without it; batch 16: 7.3 / 5.9 / 6.0 ms).
DEPENDENT_LAUNCH_MAX_TOKENS = 16


def set_dependent_launch(on: bool) -> None:
    """Let the kernels of the coming launches start while their predecessor drains
    (programmatic dependent launch).  Worth it for steps of a few tokens."""
    _lib().ix_dependent_launch_flag(1 if on else 0)


# ---------------------------------------------------------------------------
# Sizes the kernels refuse.  Parts call these when a model is built, so that a model the
# kernels cannot run is refused with the offending size named, before weights are read;
# the kernels' own checks remain (they return "a size this kernel does not take").
def check_attention_limits(heads: int, kv_heads: int, head_dim: int, dtype, where: str = ""):
    lib = _lib()
    most = lib.ix_attention_max_head_dim()
    if head_dim > most:
        raise KernelError(f"{where}: head size {head_dim} exceeds the largest the attention "
                          f"kernels take ({most})")
    if head_dim % 2:
        raise KernelError(f"{where}: head size {head_dim} is odd")
    if heads > 65535 or heads % max(1, kv_heads):
        raise KernelError(f"{where}: {heads} heads over {kv_heads} key/value heads is not a "
                          "grouping the attention kernels take (a multiple, at most 65535)")


def check_router_limits(hidden: int, num_experts: int, top_k: int, where: str = ""):
    lib = _lib()
    if top_k > lib.ix_router_max_topk():
        raise KernelError(f"{where}: {top_k} experts per token exceed the router kernel's "
                          f"limit of {lib.ix_router_max_topk()}")
    if num_experts > lib.ix_router_max_experts():
        raise KernelError(f"{where}: {num_experts} experts exceed the dispatch kernels' limit "
                          f"of {lib.ix_router_max_experts()}")
    if top_k > num_experts:
        raise KernelError(f"{where}: {top_k} experts per token of {num_experts}")


def embed(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None):
    """out[t] = table[ids[t]] widened to fp32 (the residual stream)."""
    _chk("table", table)
    _chk("ids", ids, torch.int32)
    V, H = table.shape
    T = ids.numel()
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _chk("out", out, torch.float32)
    _check(_lib().ix_embed(_ptr(table), _dtype_code(table), _ptr(ids), T, H, V, _ptr(out),
                           _stream()), "embed")
    _count()
    return out


class CombinePending:
    """The output of a mixture-of-experts block that has not been written yet: the
    expert rows, where each token's rows are, their weights and the shared expert's
    part.  ``add_rmsnorm`` consumes it in the same pass that adds it to the residual;
    ``materialize`` writes it out like ``moe_combine``."""

    def __init__(self, y, dest, topk_w, shared, shared_logit):
        self.y, self.dest, self.topk_w = y, dest, topk_w
        self.shared, self.shared_logit = shared, shared_logit
        self.shape = (topk_w.shape[0], y.shape[1])
        self.dtype = y.dtype

    def materialize(self):
        return moe_combine(self.y, self.dest, self.topk_w, self.shared, self.shared_logit)


def moe_combine_pending(y, dest, topk_w, shared, shared_logit):
    """``moe_combine`` deferred into the next residual add + norm where that kernel
    exists (bfloat16, width a multiple of 8); the combined tensor otherwise."""
    if y.dtype == torch.bfloat16 and y.shape[1] % 8 == 0 and y.shape[1] <= 8192:
        return CombinePending(y, dest, topk_w, shared, shared_logit)
    return moe_combine(y, dest, topk_w, shared, shared_logit)


def add_rmsnorm(resid: torch.Tensor, delta, gain: torch.Tensor,
                eps: float, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
    """resid += delta (kept when ``rows`` is None); returns RMSNorm(resid) * gain.

    With ``rows`` the listed rows are gathered, normalised and returned without
    writing the residual back.  ``delta`` may be a ``CombinePending``."""
    if isinstance(delta, CombinePending):
        if rows is None and out_dtype == torch.bfloat16 and delta.shape == tuple(resid.shape):
            _chk("resid", resid, torch.float32)
            _chk("gain", gain, torch.float32)
            T, H = resid.shape
            out = torch.empty((T, H), dtype=out_dtype, device=resid.device)
            code = _lib().ix_combine_add_rmsnorm(
                _ptr(resid), _ptr(delta.y), _ptr(delta.dest), _ptr(delta.topk_w),
                _ptr(delta.shared), _ptr(delta.shared_logit), _ptr(gain), _ptr(out), T, H,
                delta.topk_w.shape[1], ctypes.c_float(eps), _stream())
            _check(code, "combine_add_rmsnorm")
            _count()
            return out
        delta = delta.materialize()
    _chk("resid", resid, torch.float32)
    _chk("gain", gain, torch.float32)
    _chk("delta", delta, optional=True)
    _chk("rows", rows, torch.int32, optional=True)
    T, H = resid.shape
    if gain.numel() != H:
        raise KernelError(f"add_rmsnorm: gain has {gain.numel()} entries, rows have {H}")
    if delta is not None and (delta.shape != resid.shape or delta.dtype != out_dtype):
        raise KernelError("add_rmsnorm: delta must match the residual's shape and the "
                          f"activation type ({tuple(delta.shape)}, {delta.dtype})")
    R = T if rows is None else rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=resid.device)
    _check(_lib().ix_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(gain), _ptr(rows), _ptr(out),
                                 _dtype_code(out), R, H, ctypes.c_float(eps),
                                 1 if rows is None else 0, _stream()), "add_rmsnorm")
    _count()
    return out


def silu_mul(gu: torch.Tensor):
    _chk("gu", gu)
    T, two_i = gu.shape
    if two_i % 2:
        raise KernelError("silu_mul: width must be even (gate | up)")
    out = torch.empty((T, two_i // 2), dtype=gu.dtype, device=gu.device)
    _check(_lib().ix_silu_mul(_ptr(gu), _ptr(out), _dtype_code(gu), T, two_i // 2, _stream()),
           "silu_mul")
    _count()
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None):
    """x[M,K] . w[N,K]^T.  bfloat16: cuBLAS, fp32 accumulation.  float32: own FFMA kernel."""
    _chk("x", x)
    _chk("w", w)
    if x.dtype != w.dtype:
        raise KernelError(f"linear: activations are {x.dtype} but weights are {w.dtype}")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"linear: inner sizes differ ({K} vs {K2})")
    out_dtype = out_dtype or x.dtype
    if M <= SMALL_M_DENSE_ROWS and _streams_weights(x, w):
        return gemm_small_m(x, w.unsqueeze(0), None, None, False, M, out_dtype=out_dtype,
                            rows_per_pass=M)
    if x.dtype == torch.bfloat16:
        LIBRARY_CALLS[0] += 1
        if out_dtype == torch.bfloat16:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    return gemm_generic(x, w.unsqueeze(0), None, None, dual=False, out_dtype=out_dtype)


def gemm_generic(x: torch.Tensor, w: torch.Tensor, rows: Optional[torch.Tensor],
                 offsets: Optional[torch.Tensor], dual: bool,
                 out_dtype: Optional[torch.dtype] = None, num_out_rows: Optional[int] = None):
    """CUDA-core product, single (offsets None) or grouped by expert."""
    _chk("x", x)
    _chk("w", w)
    _chk("rows", rows, torch.int32, optional=True)
    _chk("offsets", offsets, torch.int32, optional=True)
    E, w_rows, K = w.shape
    N = w_rows // 2 if dual else w_rows
    if x.shape[1] != K:
        raise KernelError(f"gemm: inner sizes differ ({x.shape[1]} vs {K})")
    out_dtype = out_dtype or x.dtype
    if offsets is None:
        M = x.shape[0]
        A = M
    else:
        M = 0
        A = num_out_rows if num_out_rows is not None else (
            rows.numel() if rows is not None else x.shape[0])
    out = torch.empty((A, N), dtype=out_dtype, device=x.device)
    code = _lib().ix_gemm_generic(
        _ptr(x), _ptr(rows), _ptr(offsets), _ptr(w), _ptr(out), _dtype_code(x),
        F32 if out_dtype == torch.float32 else BF16, 1 if dual else 0, M, N, K, E, A, _stream())
    _check(code, "gemm_generic")
    _count()
    return out


def qkv_rope_append(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                    inv_freq: Optional[torch.Tensor], rotary_dim: int, heads: int, kv_heads: int,
                    head_dim: int, k_cache: Optional[torch.Tensor],
                    v_cache: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                    want_dense_kv: bool = False):
    """Split + bias + rotate; returns q [T,heads,hd] (and dense k, v when asked);
    writes k, v into the paged cache at ``slots`` when a cache is given."""
    _chk("qkv", qkv)
    _chk("bias", bias, torch.float32, optional=True)
    _chk("positions", positions, torch.int32)
    _chk("inv_freq", inv_freq, torch.float32, optional=True)
    _chk("slots", slots, torch.int32, optional=True)
    T, width = qkv.shape
    if width != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qkv_rope_append: row width {width} is not (heads+2*kv_heads)*head_dim")
    if bias is not None and bias.numel() != width:
        raise KernelError("qkv_rope_append: bias length does not match the fused row")
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("qkv_rope_append: inv_freq must have rotary_dim/2 entries")
    page_size = 1
    if k_cache is not None:
        _chk("k_cache", k_cache, qkv.dtype)
        _chk("v_cache", v_cache, qkv.dtype)
        if slots is None:
            raise KernelError("qkv_rope_append: a cache needs slots")
        P, ckv, page_size, chd = k_cache.shape
        if ckv != kv_heads or chd != head_dim or v_cache.shape != k_cache.shape:
            raise KernelError("qkv_rope_append: cache geometry does not match the heads")
    q = torch.empty((T, heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    k = v = None
    if want_dense_kv:
        k = torch.empty((T, kv_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
        v = torch.empty_like(k)
    code = _lib().ix_qkv_rope_append(
        _ptr(qkv), _ptr(bias), _ptr(positions), _ptr(inv_freq), rotary_dim, _ptr(slots), _ptr(q),
        _ptr(k_cache), _ptr(v_cache), page_size, _ptr(k), _ptr(v), _dtype_code(qkv), T, heads,
        kv_heads, head_dim, _stream())
    _check(code, "qkv_rope_append")
    _count()
    return (q, k, v) if want_dense_kv else q


USE_FUSED_QKV = True


def qkv_project_applies(x: torch.Tensor, w: torch.Tensor, heads: int, kv_heads: int,
                        head_dim: int, rotary_dim: int) -> bool:
    """Whether ``qkv_project_rope_append`` takes this step: bfloat16, a few tokens, a full
    rotation or none."""
    return bool(USE_FUSED_QKV and x.is_cuda and x.dtype == torch.bfloat16
                and w.dtype == torch.bfloat16 and x.is_contiguous()
                and _lib().ix_qkv_project_rope_applies(x.shape[0], x.shape[1], heads, kv_heads,
                                                       head_dim, rotary_dim))


def qkv_project_rope_append(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                            positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                            rotary_dim: int, heads: int, kv_heads: int, head_dim: int,
                            k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor):
    """For a step of a few tokens: q = rotate(x . Wq^T + bq) returned as [T, heads, hd],
    rotate(x . Wk^T + bk) and x . Wv^T + bv written into the cache pages at ``slots``, in one
    launch (``linear`` followed by ``qkv_rope_append`` otherwise)."""
    _chk("x", x, torch.bfloat16)
    _chk("w", w, torch.bfloat16)
    _chk("bias", bias, torch.float32, optional=True)
    _chk("positions", positions, torch.int32)
    _chk("inv_freq", inv_freq, torch.float32, optional=True)
    _chk("slots", slots, torch.int32)
    _chk("k_cache", k_cache, torch.bfloat16)
    _chk("v_cache", v_cache, torch.bfloat16)
    T, K = x.shape
    width = (heads + 2 * kv_heads) * head_dim
    if w.shape != (width, K) or (bias is not None and bias.numel() != width):
        raise KernelError("qkv_project_rope_append: weight or bias does not match the heads")
    P, ckv, page_size, chd = k_cache.shape
    if ckv != kv_heads or chd != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("qkv_project_rope_append: cache geometry does not match the heads")
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("qkv_project_rope_append: inv_freq must have rotary_dim/2 entries")
    if positions.numel() != T or slots.numel() != T:
        raise KernelError("qkv_project_rope_append: one position and one slot per token")
    q = torch.empty((T, heads, head_dim), dtype=torch.bfloat16, device=x.device)
    code = _lib().ix_qkv_project_rope_append(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(positions), _ptr(inv_freq), rotary_dim, _ptr(slots),
        _ptr(q), _ptr(k_cache), _ptr(v_cache), page_size, T, K, heads, kv_heads, head_dim,
        _stream())
    _check(code, "qkv_project_rope_append")
    _count()
    return q


def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            block_table: torch.Tensor, seq_of_token: torch.Tensor,
                            positions: torch.Tensor, window: int, scale: float):
    _chk("q", q)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("seq_of_token", seq_of_token, torch.int32)
    _chk("positions", positions, torch.int32)
    T, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    if chd != hd:
        raise KernelError("paged_attention: cache head size differs from the query's")
    out = torch.empty_like(q)
    code = _lib().ix_paged_attention_generic(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(seq_of_token),
        _ptr(positions), _ptr(out), _dtype_code(q), T, heads, kvh, hd, page,
        block_table.shape[1], window, ctypes.c_float(scale), _stream())
    _check(code, "paged_attention_generic")
    _count()
    return out


def paged_attention_tiled(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          block_table: torch.Tensor, cu_q: torch.Tensor, q_pos0: torch.Tensor,
                          window: int, scale: float):
    """CUDA-core attention for a ragged batch, tiled (32 queries of a sequence against 64
    keys at a time in shared memory, fp32 math): sequence s brings the queries
    q[cu_q[s]:cu_q[s+1]] at positions q_pos0[s], q_pos0[s]+1, ...  Any element type, head
    sizes that are a multiple of 4 up to 256."""
    _chk("q", q)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("cu_q", cu_q, torch.int32)
    _chk("q_pos0", q_pos0, torch.int32)
    T, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    S = q_pos0.numel()
    if chd != hd or v_cache.shape != k_cache.shape:
        raise KernelError("paged_attention_tiled: cache geometry differs from the query's")
    if cu_q.numel() != S + 1 or block_table.shape[0] != S:
        raise KernelError("paged_attention_tiled: cu_q, q_pos0 and block_table disagree")
    out = torch.empty_like(q)
    code = _lib().ix_paged_attention_tiled(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(cu_q), _ptr(q_pos0),
        _ptr(out), _dtype_code(q), T, S, heads, kvh, hd, page, block_table.shape[1], window,
        ctypes.c_float(scale), _stream())
    _check(code, "paged_attention_tiled")
    _count()
    return out


# A batch with at least this many queries a sequence on average goes to the tiled
# CUDA-core kernel where the tensor-core kernels do not apply; fewer (single decoded
# tokens, mostly) to the kernel that gives every (token, head) a block of its own.
TILED_ATTENTION_MIN_QUERIES = 4


# below this many tokens the router runs as two kernels (logits by one warp per (token,
# expert), then selection); from it on as one fused kernel (equal at 128 tokens, 13 us
# against 19-21 us at 200-256)
ROUTER_FEW_TOKENS = 128


def router_topk(x: torch.Tensor, w: torch.Tensor, top_k: int, renormalize: bool, scale: float,
                extra_w: Optional[torch.Tensor] = None
                ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """fp32 router logits, softmax over all experts, top-k (ties to the lower index).

    Returns (weights [T,k] fp32, experts [T,k] int32, x.extra_w [T] fp32 or None).
    Few tokens: one warp per (token, expert) computes the logits and one warp per
    token selects; many tokens: one fused kernel over 4 to 16 tokens per block.  Both form
    a dot product in the same order, so a token's routing is the same in either."""
    _chk("x", x)
    _chk("w", w, torch.float32)
    _chk("extra_w", extra_w, torch.float32, optional=True)
    T, H = x.shape
    E = w.shape[0]
    if w.shape[1] != H or (extra_w is not None and extra_w.numel() != H):
        raise KernelError("router_topk: weight width differs from the activations'")
    tw = torch.empty((T, top_k), dtype=torch.float32, device=x.device)
    ti = torch.empty((T, top_k), dtype=torch.int32, device=x.device)
    ex = torch.empty((T,), dtype=torch.float32, device=x.device) if extra_w is not None else None
    few = T < ROUTER_FEW_TOKENS   # few tokens: logits by many blocks, then a selection kernel
    scratch = torch.empty((T, E), dtype=torch.float32, device=x.device) if few else None
    code = _lib().ix_router_topk(_ptr(x), _ptr(w), _ptr(extra_w), _dtype_code(x), T, H, E, top_k,
                                 1 if renormalize else 0, ctypes.c_float(scale), _ptr(tw),
                                 _ptr(ti), _ptr(ex), _ptr(scratch), _stream())
    _check(code, "router_topk")
    _count(2 if few else 1)
    return tw, ti, ex


def moe_dispatch(topk_idx: torch.Tensor, num_experts: int):
    """offsets[E+1], rows[A] (token of each grouped row), dest[A] (grouped row of t*k+slot)."""
    _chk("topk_idx", topk_idx, torch.int32)
    T, k = topk_idx.shape
    dev = topk_idx.device
    offsets = torch.empty((num_experts + 1,), dtype=torch.int32, device=dev)
    rows = torch.empty((T * k,), dtype=torch.int32, device=dev)
    dest = torch.empty((T * k,), dtype=torch.int32, device=dev)
    n_scratch = _lib().ix_moe_dispatch_scratch_ints(T, num_experts, k)
    scratch = torch.empty((n_scratch,), dtype=torch.int32, device=dev) if n_scratch else None
    _check(_lib().ix_moe_dispatch(_ptr(topk_idx), T, num_experts, k, _ptr(offsets), _ptr(rows),
                                  _ptr(dest), _ptr(scratch), _stream()), "moe_dispatch")
    _count(3 if n_scratch else 1)
    return offsets, rows, dest


def moe_combine(y: torch.Tensor, dest: torch.Tensor, topk_w: torch.Tensor,
                shared: Optional[torch.Tensor], shared_logit: Optional[torch.Tensor]):
    _chk("y", y)
    _chk("dest", dest, torch.int32)
    _chk("topk_w", topk_w, torch.float32)
    _chk("shared", shared, y.dtype, optional=True)
    _chk("shared_logit", shared_logit, torch.float32, optional=True)
    T, k = topk_w.shape
    H = y.shape[1]
    out = torch.empty((T, H), dtype=y.dtype, device=y.device)
    _check(_lib().ix_moe_combine(_ptr(y), _ptr(dest), _ptr(topk_w), _ptr(shared),
                                 _ptr(shared_logit), _ptr(out), _dtype_code(y), T, H, k,
                                 _stream()), "moe_combine")
    _count()
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seeds: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           top_k: Optional[torch.Tensor] = None, min_p: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None):
    """Token ids [R] int32 from fp32 logits [R,V]; greedy where temperature <= 0 or absent."""
    _chk("logits", logits, torch.float32)
    _chk("temperature", temperature, torch.float32, optional=True)
    _chk("seeds", seeds, torch.int64, optional=True)
    _chk("top_p", top_p, torch.float32, optional=True)
    _chk("top_k", top_k, torch.int32, optional=True)
    _chk("min_p", min_p, torch.float32, optional=True)
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _chk("out", out, torch.int32)
    _check(_lib().ix_sample(_ptr(logits), R, V, _ptr(temperature), _ptr(top_p), _ptr(top_k),
                            _ptr(min_p), _ptr(seeds), _ptr(out), _stream()), "sample")
    _count()
    return out


def apply_penalties(logits: torch.Tensor, hist_ids: Optional[torch.Tensor],
                    hist_counts: Optional[torch.Tensor], penalties: Optional[torch.Tensor],
                    mask_ids: Optional[torch.Tensor]) -> None:
    """Penalties and masks on fp32 logits [R,V], in place, before a token is chosen:
    ``hist_ids`` / ``hist_counts`` [R,H] int32 (distinct generated ids and how often, -1
    padded) with ``penalties`` [R,3] (presence, frequency, repetition), and ``mask_ids``
    [R,M] int32 (tokens set to -inf, -1 padded); either group may be absent."""
    _chk("logits", logits, torch.float32)
    _chk("hist_ids", hist_ids, torch.int32, optional=True)
    _chk("hist_counts", hist_counts, torch.int32, optional=True)
    _chk("penalties", penalties, torch.float32, optional=True)
    _chk("mask_ids", mask_ids, torch.int32, optional=True)
    R, V = logits.shape
    if (hist_ids is None) != (hist_counts is None) or (hist_ids is None) != (penalties is None):
        raise KernelError("apply_penalties: history ids, counts and penalties come together")
    if hist_ids is not None and (hist_ids.shape != hist_counts.shape or hist_ids.shape[0] != R
                                 or tuple(penalties.shape) != (R, 3)):
        raise KernelError("apply_penalties: history or penalties do not match the rows")
    if mask_ids is not None and mask_ids.shape[0] != R:
        raise KernelError("apply_penalties: mask does not match the rows")
    if hist_ids is None and mask_ids is None:
        return
    _check(_lib().ix_apply_penalties(
        _ptr(logits), R, V, _ptr(hist_ids), _ptr(hist_counts),
        0 if hist_ids is None else hist_ids.shape[1], _ptr(penalties), _ptr(mask_ids),
        0 if mask_ids is None else mask_ids.shape[1], _stream()), "apply_penalties")
    _count()


def max_top_logprobs() -> int:
    return int(_lib().ix_logprobs_max_top())


def token_logprobs(logits: torch.Tensor, chosen: torch.Tensor,
                   want_k: Optional[torch.Tensor] = None, top: int = 0):
    """Log-probabilities under softmax(logits) of the chosen tokens [R] and of each row's
    ``want_k[r]`` most probable tokens (ties to the lower id; a negative entry skips the
    row): (chosen_lp [R] fp32, top_ids [R,top] int32 with -1 where unused, top_lps)."""
    _chk("logits", logits, torch.float32)
    _chk("chosen", chosen, torch.int32)
    _chk("want_k", want_k, torch.int32, optional=True)
    R, V = logits.shape
    if chosen.numel() != R or (want_k is not None and want_k.numel() != R):
        raise KernelError("token_logprobs: one chosen token and one count per row")
    if not 0 <= top <= max_top_logprobs():
        raise KernelError(f"token_logprobs: at most {max_top_logprobs()} alternatives")
    dev = logits.device
    chosen_lp = torch.empty((R,), dtype=torch.float32, device=dev)
    top_ids = torch.empty((R, top), dtype=torch.int32, device=dev) if top else None
    top_lps = torch.empty((R, top), dtype=torch.float32, device=dev) if top else None
    _check(_lib().ix_token_logprobs(_ptr(logits), R, V, _ptr(chosen), _ptr(want_k), top,
                                    _ptr(chosen_lp), _ptr(top_ids), _ptr(top_lps), _stream()),
           "token_logprobs")
    _count()
    return chosen_lp, top_ids, top_lps


def append_kv(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              slots: torch.Tensor):
    """Write dense k, v rows [T,kv_heads,hd] into the paged cache at ``slots``."""
    _chk("k", k)
    _chk("v", v, k.dtype)
    _chk("k_cache", k_cache, k.dtype)
    _chk("v_cache", v_cache, k.dtype)
    _chk("slots", slots, torch.int32)
    T, kvh, hd = k.shape
    P, ckv, page, chd = k_cache.shape
    if (ckv, chd) != (kvh, hd) or v.shape != k.shape or v_cache.shape != k_cache.shape:
        raise KernelError("append_kv: cache geometry does not match the rows")
    _check(_lib().ix_append_kv(_ptr(k), _ptr(v), _ptr(slots), _ptr(k_cache), _ptr(v_cache), page,
                               _dtype_code(k), T, kvh, hd, _stream()), "append_kv")
    _count()


_DECODE_HEAD_SIZES = {torch.bfloat16: (64, 128, 256), torch.float32: (64, 128)}


# Decode attention forms: "tma" (keys and values brought in by TMA), "mma" (the same
# arithmetic fed by cp.async), "scalar" (CUDA cores; fp32 and sizes the others refuse).
USE_TMA_DECODE = True


def _tma_decode_applies(q, page: int) -> bool:
    return (q.dtype == torch.bfloat16 and q.shape[2] in (64, 128)
            and page in (8, 16, 32, 64))


def paged_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           block_table: torch.Tensor, kv_len: torch.Tensor, max_kv_len: int,
                           window: int, scale: float, splits: Optional[int] = None,
                           kernel: Optional[str] = None, out: Optional[torch.Tensor] = None):
    """Split-KV attention for a batch in which sequence s brings the one query q[s]
    at position kv_len[s] - 1.  ``kernel`` picks a form ("tma", "mma", "scalar");
    None takes the fastest that applies."""
    _chk("q", q)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("kv_len", kv_len, torch.int32)
    S, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    if chd != hd or v_cache.shape != k_cache.shape:
        raise KernelError("paged_attention_decode: cache geometry differs from the query's")
    if hd not in _DECODE_HEAD_SIZES.get(q.dtype, ()):
        raise KernelError(f"paged_attention_decode: head size {hd} with {q.dtype} is not built; "
                          "use the general kernel")
    if kv_len.numel() != S or block_table.shape[0] != S:
        raise KernelError("paged_attention_decode: one query per sequence is required")
    if kernel is None:
        if USE_TMA_DECODE and _tma_decode_applies(q, page):
            kernel = "tma"
        else:
            kernel = "mma"
    if kernel not in ("tma", "mma", "scalar"):
        raise KernelError(f"paged_attention_decode: no kernel form {kernel!r}")
    if kernel == "tma" and not _tma_decode_applies(q, page):
        raise KernelError(f"paged_attention_decode: the TMA form takes bf16, head size 64 or 128 "
                          f"and a page of 8, 16, 32 or 64 keys (got {q.dtype}, {hd}, {page})")
    lib = _lib()
    if splits is None:
        pick = lib.ix_attn_decode_tma_splits if kernel == "tma" else lib.ix_attn_decode_splits
        splits = pick(S, heads, kvh, int(max_kv_len))
    if out is None:
        out = torch.empty_like(q)
    else:
        _chk("out", out, q.dtype)
        if out.shape != q.shape:
            raise KernelError("paged_attention_decode: out must have the query's shape")
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((S, heads, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((S, heads, splits, 2), dtype=torch.float32, device=q.device)
    if kernel == "tma":
        code = lib.ix_paged_attention_decode_tma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), P, _ptr(block_table), _ptr(kv_len),
            _ptr(part_o), _ptr(part_ml), _ptr(out), S, heads, kvh, hd, page,
            block_table.shape[1], window, ctypes.c_float(scale), splits,
            _ptr(_tc_status(q.device)), _stream())
    else:
        entry = (lib.ix_paged_attention_decode_scalar if kernel == "scalar"
                 else lib.ix_paged_attention_decode)
        code = entry(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(kv_len), _ptr(part_o),
            _ptr(part_ml), _ptr(out), _dtype_code(q), S, heads, kvh, hd, page,
            block_table.shape[1], window, ctypes.c_float(scale), splits, _stream())
    _check(code, "paged_attention_decode")
    _count(2 if splits > 1 else 1)
    return out


_PREFILL_HEAD_SIZES = {torch.bfloat16: (64, 128)}


# Prompt attention forms: "tc" (tcgen05, S and O in tensor memory, K/V by TMA) and
# "mma" (mma.sync tiles fed by cp.async; any page size).
USE_TCGEN05_ATTENTION = True


def _tc_prefill_applies(q, page: int) -> bool:
    return (q.dtype == torch.bfloat16 and q.shape[2] in (64, 128)
            and page in (8, 16, 32, 64))


def paged_attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            block_table: torch.Tensor, cu_q: torch.Tensor, q_pos0: torch.Tensor,
                            window: int, scale: float, kernel: Optional[str] = None,
                            out: Optional[torch.Tensor] = None, splits: Optional[int] = None,
                            max_kv_len: Optional[int] = None):
    """Tensor-core attention for a ragged batch: sequence s brings the queries
    q[cu_q[s]:cu_q[s+1]] at positions q_pos0[s], q_pos0[s]+1, ...  ``kernel`` picks a
    form ("tc", "mma"); None takes the fastest that applies.  ``splits`` (tcgen05 form):
    runs the keys of a query tile are cut into, merged afterwards; None lets the kernel
    module choose (more than one only for few queries over a long context, which it
    judges from ``max_kv_len``, the longest context of the step, or else from the width
    of the block table)."""
    _chk("q", q, torch.bfloat16)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("cu_q", cu_q, torch.int32)
    _chk("q_pos0", q_pos0, torch.int32)
    T, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    S = q_pos0.numel()
    if chd != hd or v_cache.shape != k_cache.shape:
        raise KernelError("paged_attention_prefill: cache geometry differs from the query's")
    if hd not in _PREFILL_HEAD_SIZES.get(q.dtype, ()):
        raise KernelError(f"paged_attention_prefill: head size {hd} is not built; use the "
                          "general kernel")
    if cu_q.numel() != S + 1 or block_table.shape[0] != S:
        raise KernelError("paged_attention_prefill: cu_q, q_pos0 and block_table disagree")
    if kernel is None:
        kernel = "tc" if USE_TCGEN05_ATTENTION and _tc_prefill_applies(q, page) else "mma"
    if kernel not in ("tc", "mma"):
        raise KernelError(f"paged_attention_prefill: no kernel form {kernel!r}")
    if kernel == "tc" and not _tc_prefill_applies(q, page):
        raise KernelError(f"paged_attention_prefill: the tcgen05 form takes bf16, head size 64 "
                          f"or 128 and a page of 8, 16, 32 or 64 keys (got {q.dtype}, {hd}, "
                          f"{page})")
    if out is None:
        out = torch.empty_like(q)
    else:
        _chk("out", out, q.dtype)
        if out.shape != q.shape:
            raise KernelError("paged_attention_prefill: out must have the query's shape")
    launches = 1
    if kernel == "tc":
        if splits is None:
            keys = int(max_kv_len) if max_kv_len else block_table.shape[1] * page
            splits = _lib().ix_attn_prefill_tc_splits(T, S, heads, keys, window)
        if not 1 <= splits <= 64:
            raise KernelError(f"paged_attention_prefill: splits must be 1..64, got {splits}")
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((T, heads, splits, hd), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((T, heads, splits, 2), dtype=torch.float32, device=q.device)
            launches = 2
        code = _lib().ix_paged_attention_prefill_tc(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), P, _ptr(block_table), _ptr(cu_q),
            _ptr(q_pos0), _ptr(out), T, S, heads, kvh, hd, page, block_table.shape[1], window,
            ctypes.c_float(scale), splits, _ptr(part_o), _ptr(part_ml),
            _ptr(_tc_status(q.device)), _stream())
    else:
        code = _lib().ix_paged_attention_prefill(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(cu_q), _ptr(q_pos0),
            _ptr(out), _dtype_code(q), T, S, heads, kvh, hd, page, block_table.shape[1], window,
            ctypes.c_float(scale), _stream())
    _check(code, "paged_attention_prefill")
    _count(launches)
    return out


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, step, window: int, scale: float):
    """Causal attention of this step's queries over the paged cache.

    ``step`` carries the batch description (``seq_of_token``, ``positions``, ``cu_q``,
    ``q_pos0``, ``kv_len``, ``max_q_len``, ``max_kv_len``, ``all_decode``).  Steps of
    single tokens go to the split-KV kernel; everything else, and head sizes the
    tuned kernels do not take, to the general kernel."""
    hd = q.shape[2]
    if step.all_decode and hd in _DECODE_HEAD_SIZES.get(q.dtype, ()):
        return paged_attention_decode(q, k_cache, v_cache, block_table, step.kv_len,
                                      step.max_kv_len, window, scale)
    if hd in _PREFILL_HEAD_SIZES.get(q.dtype, ()):
        nd = getattr(step, "num_decode_seqs", 0)
        if 0 < nd < step.num_seqs and getattr(step, "cu_q_prompt", None) is not None:
            # a mixed batch: its single tokens (they come first) go to the split-KV kernel,
            # which streams their keys at full rate, the prompt portions to the tiled one
            out = torch.empty_like(q)
            paged_attention_decode(q[:nd], k_cache, v_cache, block_table[:nd], step.kv_len[:nd],
                                   step.max_kv_len, window, scale, out=out[:nd])
            paged_attention_prefill(q[nd:], k_cache, v_cache, block_table[nd:],
                                    step.cu_q_prompt, step.q_pos0[nd:], window, scale,
                                    out=out[nd:], max_kv_len=step.max_kv_len)
            return out
        return paged_attention_prefill(q, k_cache, v_cache, block_table, step.cu_q, step.q_pos0,
                                       window, scale, max_kv_len=step.max_kv_len)
    if (step.num_tokens >= TILED_ATTENTION_MIN_QUERIES * step.num_seqs
            and _lib().ix_paged_attention_tiled_applies(hd)
            and getattr(step, "cu_q", None) is not None):
        return paged_attention_tiled(q, k_cache, v_cache, block_table, step.cu_q, step.q_pos0,
                                     window, scale)
    return paged_attention_generic(q, k_cache, v_cache, block_table, step.seq_of_token,
                                   step.positions, window, scale)


USE_TCGEN05 = True           # prompt-sized grouped products go to the tcgen05 kernel
TCGEN05_MAX_EXPERTS = 1024   # its per-expert tile prefix lives in shared memory
# grouped: up to this many rows per expert on average stream the weights with the
# mma.sync kernel; beyond, the persistent tcgen05 kernel is faster (measured crossover at
# 60 experts: between 24 and 32 tokens of top-4 routing)
SMALL_M_ROWS_PER_GROUP = 2
SMALL_M_DENSE_ROWS = 16      # dense: up to this many rows stream the weights once


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, rows: Optional[torch.Tensor],
                 offsets: Optional[torch.Tensor], dual: bool, num_out_rows: int,
                 out_dtype: Optional[torch.dtype] = None, rows_per_pass: int = 8,
                 active_groups: int = 0, offsets_settled: bool = False):
    """Weight-streaming product for few rows per weight matrix (bf16 inputs).
    ``offsets_settled``: the kernel that wrote ``offsets`` is at least two launches back
    in this stream (so the launch may read it, and start on its weights, before waiting
    for its predecessor)."""
    _chk("x", x, torch.bfloat16)
    _chk("w", w, torch.bfloat16)
    _chk("rows", rows, torch.int32, optional=True)
    _chk("offsets", offsets, torch.int32, optional=True)
    E, w_rows, K = w.shape
    N = w_rows // 2 if dual else w_rows
    if x.shape[1] != K:
        raise KernelError(f"gemm_small_m: inner sizes differ ({x.shape[1]} vs {K})")
    out_dtype = out_dtype or x.dtype
    out = torch.empty((num_out_rows, N), dtype=out_dtype, device=x.device)
    code = _lib().ix_gemm_small_m(
        _ptr(x), _ptr(rows), _ptr(offsets), _ptr(w), _ptr(out),
        F32 if out_dtype == torch.float32 else BF16, 1 if dual else 0,
        0 if offsets is not None else x.shape[0], N, K, E, rows_per_pass,
        active_groups or min(E, num_out_rows), 1 if offsets_settled else 0, _stream())
    _check(code, "gemm_small_m")
    _count()
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor):
    """out[i] = x[rows[i]] with 16-byte copies (row size must be a multiple of 16 bytes)."""
    _chk("x", x)
    _chk("rows", rows, torch.int32)
    n = rows.numel()
    out = torch.empty((n, x.shape[1]), dtype=x.dtype, device=x.device)
    _check(_lib().ix_gather_rows(_ptr(x), _ptr(rows), _ptr(out), n,
                                 x.shape[1] * x.element_size(), _stream()), "gather_rows")
    _count()
    return out


_TC_STATUS = {}


def _tc_status(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


_STATUS_ROLES = {
    1: "grouped_gemm_tc: the TMA producer", 2: "grouped_gemm_tc: the MMA issuer",
    3: "grouped_gemm_tc: the epilogue",
    11: "paged_attention_decode (TMA form): the copying warp",
    12: "paged_attention_decode (TMA form): a computing warp",
    21: "paged_attention_prefill (tcgen05 form): the copying warp",
    22: "paged_attention_prefill (tcgen05 form): the MMA issuer",
    23: "paged_attention_prefill (tcgen05 form): a softmax warp",
    24: "paged_attention_prefill (tcgen05 form): shared memory not on a 1024-byte mark;",
}


def check_async_errors():
    """Raise if a kernel gave up on one of its bounded mbarrier waits.  Reads a status
    word from the device, so it synchronises; call it where the host waits for
    results anyway."""
    for key, st in _TC_STATUS.items():
        code = int(st.item())
        if code:
            st.zero_()
            role = _STATUS_ROLES.get(code, "a kernel")
            raise KernelError(f"cuda:{key}: {role} waited past its limit (status {code}); "
                              "the output of that call is not valid")


def grouped_gemm_tc(a: torch.Tensor, offsets: torch.Tensor, w: torch.Tensor, dual: bool):
    """Grouped product on tcgen05 tensor cores: ``a`` [rows, K] already grouped by
    expert, ``w`` [E, N or 2N, K]; returns [rows, N] bf16."""
    _chk("a", a, torch.bfloat16)
    _chk("w", w, torch.bfloat16)
    _chk("offsets", offsets, torch.int32)
    E, w_rows, K = w.shape
    N = w_rows // 2 if dual else w_rows
    if a.shape[1] != K:
        raise KernelError(f"grouped_gemm_tc: inner sizes differ ({a.shape[1]} vs {K})")
    out = torch.empty((a.shape[0], N), dtype=torch.bfloat16, device=a.device)
    code = _lib().ix_grouped_gemm_tc(_ptr(a), _ptr(offsets), _ptr(w), _ptr(out),
                                     1 if dual else 0, a.shape[0], N, K, E,
                                     _ptr(_tc_status(a.device)), _stream())
    _check(code, "grouped_gemm_tc")
    _count()
    return out


# The persistent streaming kernel measured faster than the one-block-per-tile kernel only
# while a handful of experts have rows (one sequence decoding: 15 + 8 us against 17 + 12 us a
# layer at 60 experts of 1408 x 2048), equal at 8 assignments and slower beyond.
USE_STREAM_GROUPED = True
STREAM_GROUPED_MAX_ROWS = 4


def gemm_stream_grouped(x: torch.Tensor, w: torch.Tensor, rows: Optional[torch.Tensor],
                        offsets: torch.Tensor, dual: bool, num_out_rows: int,
                        rows_per_pass: int = 8):
    """Grouped weight-streaming product, persistent form (few rows per expert, bf16)."""
    _chk("x", x, torch.bfloat16)
    _chk("w", w, torch.bfloat16)
    _chk("rows", rows, torch.int32, optional=True)
    _chk("offsets", offsets, torch.int32)
    E, w_rows, K = w.shape
    N = w_rows // 2 if dual else w_rows
    if x.shape[1] != K:
        raise KernelError(f"gemm_stream_grouped: inner sizes differ ({x.shape[1]} vs {K})")
    if offsets.numel() != E + 1:
        raise KernelError("gemm_stream_grouped: offsets must have one entry per expert plus one")
    out = torch.empty((num_out_rows, N), dtype=torch.bfloat16, device=x.device)
    code = _lib().ix_gemm_stream_grouped(_ptr(x), _ptr(rows), _ptr(offsets), _ptr(w), _ptr(out),
                                         1 if dual else 0, N, K, E, rows_per_pass, _stream())
    _check(code, "gemm_stream_grouped")
    _count()
    return out


def _stream_grouped_applies(x: torch.Tensor, w: torch.Tensor, num_rows: int) -> bool:
    return (USE_STREAM_GROUPED and num_rows <= STREAM_GROUPED_MAX_ROWS
            and _streams_weights(x, w) and w.shape[-1] >= 256 and w.shape[0] <= 1024)


def _streams_weights(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes these operands: bf16, K in 16-byte chunks."""
    return x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[-1] % 8 == 0


def grouped_gate_up_swiglu(x: torch.Tensor, rows: torch.Tensor, offsets: torch.Tensor,
                           w_gate_up: torch.Tensor):
    """act[r] = silu(x[rows[r]] . Wg[e]^T) * (x[rows[r]] . Wu[e]^T), e from offsets.

    ``w_gate_up``: [E, 2I, H], per expert the gate rows then the up rows."""
    A = rows.numel()
    per = A / w_gate_up.shape[0]
    if _stream_grouped_applies(x, w_gate_up, A):
        return gemm_stream_grouped(x, w_gate_up, rows, offsets, True, A,
                                   rows_per_pass=8 if per <= 2 else 16)
    if per <= SMALL_M_ROWS_PER_GROUP and _streams_weights(x, w_gate_up):
        return gemm_small_m(x, w_gate_up, rows, offsets, True, A,
                            rows_per_pass=8 if per <= 2 else 16)
    if USE_TCGEN05 and _streams_weights(x, w_gate_up) and w_gate_up.shape[0] <= TCGEN05_MAX_EXPERTS:
        return grouped_gemm_tc(gather_rows(x, rows), offsets, w_gate_up, True)
    return gemm_generic(x, w_gate_up, rows, offsets, dual=True, num_out_rows=A)


def grouped_down(act: torch.Tensor, offsets: torch.Tensor, w_down: torch.Tensor,
                 offsets_settled: bool = False):
    """y[r] = act[r] . Wd[e]^T with ``w_down`` [E, H, I].  ``offsets_settled``: see
    ``gemm_small_m`` (true when this follows ``grouped_gate_up_swiglu`` on the same
    offsets, as in a mixture layer)."""
    A = act.shape[0]
    per = A / w_down.shape[0]
    if _stream_grouped_applies(act, w_down, A):
        return gemm_stream_grouped(act, w_down, None, offsets, False, A,
                                   rows_per_pass=8 if per <= 2 else 16)
    if per <= SMALL_M_ROWS_PER_GROUP and _streams_weights(act, w_down):
        return gemm_small_m(act, w_down, None, offsets, False, A,
                            rows_per_pass=8 if per <= 2 else 16, offsets_settled=offsets_settled)
    if USE_TCGEN05 and _streams_weights(act, w_down) and w_down.shape[0] <= TCGEN05_MAX_EXPERTS:
        return grouped_gemm_tc(act, offsets, w_down, False)
    return gemm_generic(act, w_down, None, offsets, dual=False, num_out_rows=A)


def gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor):
    """Dense SwiGLU front half: silu(x . Wg^T) * (x . Wu^T) with ``w_gate_up`` [2I, H]."""
    _chk("x", x)
    _chk("w_gate_up", w_gate_up, x.dtype)
    M = x.shape[0]
    if M <= SMALL_M_DENSE_ROWS and _streams_weights(x, w_gate_up):
        return gemm_small_m(x, w_gate_up.unsqueeze(0), None, None, True, M, rows_per_pass=M)
    return silu_mul(linear(x, w_gate_up))
