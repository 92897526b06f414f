// MoE routing: router logits, softmax over all experts, top-k, and the stable
// group-by-expert dispatch tables.
//
// Reference behaviour: a library GEMM for the logits followed by RouteTopKKernel
// (src/backends/cuda/ops/moe.cu:36-127): fp32 softmax with max subtraction over
// all E, k rounds of masked argmax with a strictly-greater compare (ties go to
// the lower index), optional renormalisation of the k weights (guarded by
// total > 0), then the routed scale; slots are in descending-probability order.
// Here the logits are computed in the same kernel in fp32 (the router weight is
// kept in fp32), and one extra weight row (the shared expert's gate) can ride
// along since it reads the same activations.
//
// Dispatch: CountPerExpert / ScanOffsets / ScatterByExpert (moe.cu:130-221):
// offsets[E+1], rows[A] (source token of each grouped row) and dest[A] (grouped
// row of assignment t*k+slot); inside an expert rows ascend by assignment index.
#include "common.cuh"
#include "elementwise_vec.cuh"

#define ROUTER_THREADS 256
#define ROUTER_MAX_TOK 8
#define ROUTER_MAX_TOPK 32
#define ROUTER_MAX_EXPERTS 8192   // the dispatch kernels' histogram

// Softmax over p[0..E) (logits, overwritten), then k rounds of masked argmax by one
// warp; ties go to the lower index.  Writes k weights and k expert ids.
__device__ __forceinline__ void select_topk(float* p, int E, int k, int renorm, float scale,
                                            float* __restrict__ out_w, int* __restrict__ out_i,
                                            int lane) {
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, p[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = expf(p[e] - mx);
    p[e] = v;
    sum += v;
  }
  sum = warp_sum(sum);
  __syncwarp();
  float total = 0.f;
  float my_w = 0.f;  // lane s keeps slot s
  int my_i = 0;
  for (int s = 0; s < k; ++s) {
    float best = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = p[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    const float prob = best / sum;
    if (lane == s) { my_w = prob; my_i = bi; }
    total += prob;
    if (lane == 0) p[bi] = -2.f;  // masked: below every probability
    __syncwarp();
  }
  if (lane < k) {
    float wv = my_w;
    if (renorm && total > 0.f) wv = wv / total;
    wv *= scale;
    out_w[lane] = wv;
    out_i[lane] = my_i;
  }
}

template <typename TA, int TOK>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_topk_kernel(const TA* __restrict__ x, const float* __restrict__ w,
                   const float* __restrict__ extra_w, int T, int H, int E, int k, int renorm,
                   float scale, float* __restrict__ topk_w, int* __restrict__ topk_idx,
                   float* __restrict__ extra_out) {
  extern __shared__ float smem[];
  float* xs = smem;                         // [TOK][H]
  float* lg = smem + (size_t)TOK * H;       // [TOK][E]
  const int t0 = blockIdx.x * TOK;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = ROUTER_THREADS / 32;
  for (int idx = threadIdx.x; idx < TOK * H; idx += ROUTER_THREADS) {
    const int tk = idx / H, i = idx - tk * H;
    const int t = t0 + tk;
    xs[idx] = t < T ? to_f32(x[(size_t)t * H + i]) : 0.f;
  }
  __syncthreads();
  const int rows_total = E + (extra_w ? 1 : 0);
  for (int e = warp; e < rows_total; e += nwarps) {
    const float* wr = e < E ? w + (size_t)e * H : extra_w;
    float acc[TOK];
#pragma unroll
    for (int tk = 0; tk < TOK; ++tk) acc[tk] = 0.f;
    for (int i = lane; i < H; i += 32) {
      const float wv = wr[i];
#pragma unroll
      for (int tk = 0; tk < TOK; ++tk) acc[tk] += xs[tk * H + i] * wv;
    }
#pragma unroll
    for (int tk = 0; tk < TOK; ++tk) {
      const float v = warp_sum(acc[tk]);
      if (lane == 0) {
        if (e < E) lg[tk * E + e] = v;
        else if (t0 + tk < T) extra_out[t0 + tk] = v;
      }
    }
  }
  __syncthreads();
  // softmax + top-k: one warp per token
  for (int tk = warp; tk < TOK; tk += nwarps) {
    const int t = t0 + tk;
    if (t >= T) continue;
    select_topk(lg + tk * E, E, k, renorm, scale, topk_w + (size_t)t * k, topk_idx + (size_t)t * k,
                lane);
  }
}

template <typename TA, int TOK>
static int launch_router(const void* x, const float* w, const float* extra_w, int T, int H, int E,
                         int k, int renorm, float scale, float* topk_w, int* topk_idx,
                         float* extra_out, cudaStream_t stream) {
  const size_t smem = ((size_t)TOK * H + (size_t)TOK * E) * sizeof(float);
  if (smem > 200 * 1024) return IX_ERR_SMEM;
  auto kern = router_topk_kernel<TA, TOK>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int blocks = (T + TOK - 1) / TOK;
  kern<<<blocks, ROUTER_THREADS, smem, stream>>>((const TA*)x, w, extra_w, T, H, E, k, renorm,
                                                 scale, topk_w, topk_idx, extra_out);
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// bf16 activations, H a multiple of 8.  The dot product of a (token, expert) pair is
// formed the same way in both kernels below, so routing does not depend on how many
// tokens a step has: lane l takes the 8-element chunks l, l+32, ... in order, adds the
// eight products of a chunk in order, and the lanes are summed by the shuffle tree.
// ---------------------------------------------------------------------------

__device__ __forceinline__ void dot8(float& acc, const float* xf, const float4& wa,
                                     const float4& wb) {
  acc = fmaf(xf[0], wa.x, acc); acc = fmaf(xf[1], wa.y, acc);
  acc = fmaf(xf[2], wa.z, acc); acc = fmaf(xf[3], wa.w, acc);
  acc = fmaf(xf[4], wb.x, acc); acc = fmaf(xf[5], wb.y, acc);
  acc = fmaf(xf[6], wb.z, acc); acc = fmaf(xf[7], wb.w, acc);
}

#define ROUTER_VTHREADS 512
#define ROUTER_VROWS 4
#define ROUTER_MANY_TOKENS 1024
#define ROUTER_SMS 148   // B200; another count only shifts the choice, never the result

// WIDE: the block's activations are widened to 32-bit once, when they are staged, and kept
// as two planes of float4 (the first and the second half of every 8-element chunk, so that a
// warp's 16-byte reads are contiguous); otherwise they stay bfloat16 in shared memory and are
// widened at every use.  Widening is exact, so both give the same bits; the wide form issues
// a fifth fewer instructions and is taken when its tile fits.
template <int ROUTER_VTOK, bool WIDE>
__global__ void __launch_bounds__(ROUTER_VTHREADS)
router_topk_bf16_vec_kernel(const bf16* __restrict__ x, const float* __restrict__ w,
                            const float* __restrict__ extra_w, int T, int H, int E, int k,
                            int renorm, float scale, float* __restrict__ topk_w,
                            int* __restrict__ topk_idx, float* __restrict__ extra_out) {
  extern __shared__ __align__(16) unsigned char rsm[];
  const int chunks = H >> 3;
  uint4* xs = reinterpret_cast<uint4*>(rsm);                               // [VTOK][chunks]
  float4* xlo = reinterpret_cast<float4*>(rsm);                            // [VTOK][chunks]
  float4* xhi = xlo + (size_t)ROUTER_VTOK * chunks;                        // [VTOK][chunks]
  float* lg = reinterpret_cast<float*>(
      rsm + (size_t)ROUTER_VTOK * chunks * (WIDE ? 32 : 16));              // [VTOK][E]
  const int t0 = blockIdx.x * ROUTER_VTOK;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = ROUTER_VTHREADS / 32;
  for (int idx = threadIdx.x; idx < ROUTER_VTOK * chunks; idx += ROUTER_VTHREADS) {
    const int tk = idx / chunks, c = idx - tk * chunks;
    const int t = t0 + tk;
    const uint4 raw =
        t < T ? reinterpret_cast<const uint4*>(x + (size_t)t * H)[c] : make_uint4(0, 0, 0, 0);
    if (WIDE) {
      float xf[8];
      bf8_to_f32(raw, xf);
      xlo[idx] = make_float4(xf[0], xf[1], xf[2], xf[3]);
      xhi[idx] = make_float4(xf[4], xf[5], xf[6], xf[7]);
    } else {
      xs[idx] = raw;
    }
  }
  __syncthreads();
  const int rows_total = E + (extra_w ? 1 : 0);
  // A warp takes ROUTER_VROWS weight rows at a time, so that a chunk of activations
  // read from shared memory feeds that many dot products (one row at a time the loop is
  // bound by shared-memory reads, not by the multiply-adds).
  for (int e0 = warp * ROUTER_VROWS; e0 < rows_total; e0 += nwarps * ROUTER_VROWS) {
    const float4* wr[ROUTER_VROWS];
#pragma unroll
    for (int r = 0; r < ROUTER_VROWS; ++r) {
      const int e = min(e0 + r, rows_total - 1);       // a row past the end repeats the last
      wr[r] = reinterpret_cast<const float4*>(e < E ? w + (size_t)e * H : extra_w);
    }
    float acc[ROUTER_VTOK][ROUTER_VROWS];
#pragma unroll
    for (int tk = 0; tk < ROUTER_VTOK; ++tk)
#pragma unroll
      for (int r = 0; r < ROUTER_VROWS; ++r) acc[tk][r] = 0.f;
    for (int c = lane; c < chunks; c += 32) {
      float4 wa[ROUTER_VROWS], wb[ROUTER_VROWS];
#pragma unroll
      for (int r = 0; r < ROUTER_VROWS; ++r) {
        wa[r] = wr[r][2 * c];
        wb[r] = wr[r][2 * c + 1];
      }
#pragma unroll
      for (int tk = 0; tk < ROUTER_VTOK; ++tk) {
        float xf[8];
        if (WIDE) {
          const float4 lo = xlo[tk * chunks + c], hi = xhi[tk * chunks + c];
          xf[0] = lo.x; xf[1] = lo.y; xf[2] = lo.z; xf[3] = lo.w;
          xf[4] = hi.x; xf[5] = hi.y; xf[6] = hi.z; xf[7] = hi.w;
        } else {
          bf8_to_f32(xs[tk * chunks + c], xf);
        }
#pragma unroll
        for (int r = 0; r < ROUTER_VROWS; ++r) dot8(acc[tk][r], xf, wa[r], wb[r]);
      }
    }
#pragma unroll
    for (int tk = 0; tk < ROUTER_VTOK; ++tk)
#pragma unroll
      for (int r = 0; r < ROUTER_VROWS; ++r) {
        const float v = warp_sum(acc[tk][r]);
        const int e = e0 + r;
        if (lane == 0 && e < rows_total) {
          if (e < E) lg[tk * E + e] = v;
          else if (t0 + tk < T) extra_out[t0 + tk] = v;
        }
      }
  }
  __syncthreads();
  for (int tk = warp; tk < ROUTER_VTOK; tk += nwarps) {
    const int t = t0 + tk;
    if (t >= T) continue;
    select_topk(lg + tk * E, E, k, renorm, scale, topk_w + (size_t)t * k, topk_idx + (size_t)t * k,
                lane);
  }
}

template <int VTOK, bool WIDE>
static int launch_router_vec(const void* x, const float* w, const float* extra_w, int T, int H,
                             int E, int k, int renorm, float scale, float* topk_w, int* topk_idx,
                             float* extra_out, cudaStream_t stream) {
  const size_t smem = (size_t)VTOK * (H / 8) * (WIDE ? 32 : 16) + (size_t)VTOK * E * sizeof(float);
  auto kern = router_topk_bf16_vec_kernel<VTOK, WIDE>;
  if (smem > 48 * 1024) {
    cudaError_t e2 =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e2 != cudaSuccess) return (int)e2;
  }
  kern<<<(T + VTOK - 1) / VTOK, ROUTER_VTHREADS, smem, stream>>>(
      (const bf16*)x, w, extra_w, T, H, E, k, renorm, scale, topk_w, topk_idx, extra_out);
  return ix_launch_status();
}

__global__ void __launch_bounds__(ROUTER_THREADS)
router_logits_bf16_vec_kernel(const bf16* __restrict__ x, const float* __restrict__ w,
                              const float* __restrict__ extra_w, int T, int H, int E,
                              float* __restrict__ logits, float* __restrict__ extra_out) {
  IX_PDL_WAIT();
  const int lane = threadIdx.x & 31;
  const int pair = blockIdx.x * (ROUTER_THREADS / 32) + (threadIdx.x >> 5);
  const int rows_total = E + (extra_w ? 1 : 0);
  if (pair >= T * rows_total) return;
  const int t = pair / rows_total, e = pair - t * rows_total;
  const float4* wr = reinterpret_cast<const float4*>(e < E ? w + (size_t)e * H : extra_w);
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)t * H);
  const int chunks = H >> 3;
  float acc = 0.f;
  for (int c = lane; c < chunks; c += 32) {
    float xf[8];
    bf8_to_f32(xr[c], xf);
    dot8(acc, xf, wr[2 * c], wr[2 * c + 1]);
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    if (e < E) logits[(size_t)t * E + e] = acc;
    else extra_out[t] = acc;
  }
}

// Few tokens: one warp per (token, expert) for the logits, so that the router
// weights are streamed by many blocks at once, then one warp per token selects.
// The dot product uses the same lane striding and shuffle tree as the fused
// kernel, so a token's routing does not depend on which path ran.
template <typename TA>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_logits_kernel(const TA* __restrict__ x, const float* __restrict__ w,
                     const float* __restrict__ extra_w, int T, int H, int E,
                     float* __restrict__ logits, float* __restrict__ extra_out) {
  IX_PDL_WAIT();
  const int lane = threadIdx.x & 31;
  const int pair = blockIdx.x * (ROUTER_THREADS / 32) + (threadIdx.x >> 5);
  const int rows_total = E + (extra_w ? 1 : 0);
  if (pair >= T * rows_total) return;
  const int t = pair / rows_total, e = pair - t * rows_total;
  const float* wr = e < E ? w + (size_t)e * H : extra_w;
  const TA* xr = x + (size_t)t * H;
  float acc = 0.f;
  for (int i = lane; i < H; i += 32) acc += to_f32(xr[i]) * wr[i];
  acc = warp_sum(acc);
  if (lane == 0) {
    if (e < E) logits[(size_t)t * E + e] = acc;
    else extra_out[t] = acc;
  }
}

__global__ void __launch_bounds__(32)
router_select_kernel(const float* __restrict__ logits, int E, int k, int renorm, float scale,
                     float* __restrict__ topk_w, int* __restrict__ topk_idx) {
  extern __shared__ float prob[];
  IX_PDL_WAIT();
  const int t = blockIdx.x, lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) prob[e] = logits[(size_t)t * E + e];
  __syncwarp();
  select_topk(prob, E, k, renorm, scale, topk_w + (size_t)t * k, topk_idx + (size_t)t * k, lane);
}

// Sizes beyond which the router and dispatch kernels refuse a call; a model is checked
// against them when it is built.
IX_API int ix_router_max_topk() { return ROUTER_MAX_TOPK; }
IX_API int ix_router_max_experts() { return ROUTER_MAX_EXPERTS; }

IX_API int ix_router_topk(const void* x, const float* w, const float* extra_w, int act_dtype,
                          int T, int H, int E, int k, int renorm, float scale, float* topk_w,
                          int* topk_idx, float* extra_out, float* logits_scratch,
                          cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || E <= 0 || k <= 0 || k > E || k > ROUTER_MAX_TOPK) return IX_ERR_SIZE;
  if (extra_w && !extra_out) return IX_ERR_SIZE;
  const bool vec = act_dtype == IX_BF16 && H % 8 == 0 &&
                   (((uintptr_t)x | (uintptr_t)w | (uintptr_t)extra_w) & 15) == 0;
  if (logits_scratch && (size_t)E * sizeof(float) <= 48 * 1024) {   // the caller's choice
    // logits_scratch: [T, E] fp32
    const long long pairs = (long long)T * (E + (extra_w ? 1 : 0));
    const int blocks = (int)((pairs + ROUTER_THREADS / 32 - 1) / (ROUTER_THREADS / 32));
    if (vec) {
      ix_launch(router_logits_bf16_vec_kernel, dim3(blocks), dim3(ROUTER_THREADS), 0, stream,
                (const bf16*)x, w, extra_w, T, H, E, logits_scratch, extra_out);
      int rc = ix_launch_status();
      if (rc != 0) return rc;
      ix_launch(router_select_kernel, dim3(T), dim3(32), (size_t)E * sizeof(float), stream,
                (const float*)logits_scratch, E, k, renorm, scale, topk_w, topk_idx);
      return ix_launch_status();
    }
    IX_DISPATCH_DTYPE(act_dtype, TA,
                      (ix_launch(router_logits_kernel<TA>, dim3(blocks), dim3(ROUTER_THREADS), 0,
                                 stream, (const TA*)x, w, extra_w, T, H, E, logits_scratch,
                                 extra_out)));
    int rc = ix_launch_status();
    if (rc != 0) return rc;
    ix_launch(router_select_kernel, dim3(T), dim3(32), (size_t)E * sizeof(float), stream,
              (const float*)logits_scratch, E, k, renorm, scale, topk_w, topk_idx);
    return ix_launch_status();
  }
  if (vec) {
    // Tokens of a block share one pass over the router weights.  A block takes 4 tokens
    // while there are few.  From ROUTER_MANY_TOKENS on it takes 8 to 16: a block of v tokens
    // costs about 6.5 + 1.4 v microseconds at 60 experts of 2048 however many blocks run
    // beside it, one block fits an SM, and so the count is chosen for which the rounds of
    // blocks an SM sees cost least (2048 tokens: 14 a block is 147 blocks, one round on 147
    // SMs, 26.8 us; 16 a block leaves 20 SMs idle, 29.5 us; 4096 tokens: 51.5 against 56.7).
    int vtok = 4;
    if (T >= ROUTER_MANY_TOKENS) {
      float best = -1.f;
      for (int v = 16; v >= 8; v -= 2) {
        const long long blocks = (T + v - 1) / v;
        const float cost = (float)((blocks + ROUTER_SMS - 1) / ROUTER_SMS) * (6.5f + 1.4f * v);
        if (best < 0.f || cost < best) { best = cost; vtok = v; }
      }
    }
    const size_t lg_bytes = (size_t)vtok * E * sizeof(float);
    // widened staging pays from 10 tokens a block on (a few tenths of a microsecond)
    const bool wide = vtok >= 10 && (size_t)vtok * H * 4 + lg_bytes <= 200 * 1024;
    if ((size_t)vtok * H * 2 + lg_bytes <= 200 * 1024) {
#define IX_ROUTER_CASE(V)                                                                       \
  case V:                                                                                       \
    return wide ? launch_router_vec<V, true>(x, w, extra_w, T, H, E, k, renorm, scale, topk_w,  \
                                             topk_idx, extra_out, stream)                       \
                : launch_router_vec<V, false>(x, w, extra_w, T, H, E, k, renorm, scale, topk_w, \
                                              topk_idx, extra_out, stream);
      switch (vtok) {
        IX_ROUTER_CASE(4)
        IX_ROUTER_CASE(8)
        IX_ROUTER_CASE(10)
        IX_ROUTER_CASE(12)
        IX_ROUTER_CASE(14)
        IX_ROUTER_CASE(16)
      }
#undef IX_ROUTER_CASE
    }
  }
  // many tokens share one pass over the router weights; few tokens spread out
  const size_t per_tok = ((size_t)H + E) * sizeof(float);
  int tok = T >= 8 * 148 ? 8 : (T >= 2 * 148 ? 2 : 1);
  while (tok > 1 && tok * per_tok > 96 * 1024) tok >>= 1;
  IX_DISPATCH_DTYPE(act_dtype, TA, {
    if (tok == 8)
      return launch_router<TA, 8>(x, w, extra_w, T, H, E, k, renorm, scale, topk_w, topk_idx,
                                  extra_out, stream);
    if (tok == 4)
      return launch_router<TA, 4>(x, w, extra_w, T, H, E, k, renorm, scale, topk_w, topk_idx,
                                  extra_out, stream);
    if (tok == 2)
      return launch_router<TA, 2>(x, w, extra_w, T, H, E, k, renorm, scale, topk_w, topk_idx,
                                  extra_out, stream);
    return launch_router<TA, 1>(x, w, extra_w, T, H, E, k, renorm, scale, topk_w, topk_idx,
                                extra_out, stream);
  });
  return IX_OK;
}

// ---------------------------------------------------------------------------
// Dispatch tables.  One block; each warp owns experts warp, warp+32, ... and
// walks the assignment list with ballots, so the order inside an expert is the
// assignment order and no atomics are involved.
// ---------------------------------------------------------------------------
// `topk_idx` may be in shared or global memory; `counts` is [E + 1] ints of shared memory.
__device__ __forceinline__ void dispatch_in_block(const int* topk_idx, int A, int E, int k,
                                                  int* __restrict__ offsets,
                                                  int* __restrict__ rows, int* __restrict__ dest,
                                                  int* counts) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    int c = 0;
    for (int a0 = 0; a0 < A; a0 += 32) {
      const int a = a0 + lane;
      const bool hit = a < A && topk_idx[a] == e;
      c += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) counts[e] = c;
  }
  __syncthreads();
  if (warp == 0) {   // exclusive prefix sum over the experts, 32 at a time
    int run = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < E ? counts[e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (e < E) {
        counts[e] = run + incl - c;
        offsets[e] = run + incl - c;
      }
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      counts[E] = run;
      offsets[E] = run;
    }
  }
  __syncthreads();
  for (int e = warp; e < E; e += nwarps) {
    int base = counts[e];
    for (int a0 = 0; a0 < A; a0 += 32) {
      const int a = a0 + lane;
      const bool hit = a < A && topk_idx[a] == e;
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int r = base + __popc(mask & ((1u << lane) - 1u));
        rows[r] = a / k;
        dest[a] = r;
      }
      base += __popc(mask);
    }
  }
}

__global__ void __launch_bounds__(1024)
moe_dispatch_kernel(const int* __restrict__ topk_idx, int A, int E, int k,
                    int* __restrict__ offsets, int* __restrict__ rows, int* __restrict__ dest) {
  extern __shared__ int counts[];  // [E + 1]
  IX_PDL_WAIT();
  dispatch_in_block(topk_idx, A, E, k, offsets, rows, dest, counts);
}

// ---------------------------------------------------------------------------
// Dispatch for many assignments: blocks of 1024 assignments count their experts,
// one block turns the counts into bases (per block and expert) and offsets, and the
// blocks place their assignments: position = offsets[e] + (rows of e in earlier
// blocks) + (rows of e in earlier warps of this block) + (rank inside the warp).
// Stable, and free of atomics on global memory.  scratch: [blocks + 1][E] ints.
// ---------------------------------------------------------------------------
#define DISPATCH_CHUNK 1024
#define DISPATCH_MAX_E 512

__global__ void __launch_bounds__(DISPATCH_CHUNK)
dispatch_count_kernel(const int* __restrict__ topk_idx, int A, int E, int* __restrict__ counts) {
  __shared__ int hist[DISPATCH_MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int a = blockIdx.x * DISPATCH_CHUNK + threadIdx.x;
  if (a < A) atomicAdd(&hist[topk_idx[a]], 1);   // counts do not depend on the order
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[(size_t)blockIdx.x * E + e] = hist[e];
}

__global__ void __launch_bounds__(DISPATCH_MAX_E)
dispatch_scan_kernel(int* __restrict__ counts, int blocks, int E, int* __restrict__ offsets) {
  __shared__ int total[DISPATCH_MAX_E];
  const int e = threadIdx.x;
  if (e < E) {
    int run = 0;
    for (int b = 0; b < blocks; ++b) {
      const int c = counts[(size_t)b * E + e];
      counts[(size_t)b * E + e] = run;   // rows of e in earlier blocks
      run += c;
    }
    total[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < E; ++i) {
      offsets[i] = run;
      run += total[i];
    }
    offsets[E] = run;
  }
}

__global__ void __launch_bounds__(DISPATCH_CHUNK)
dispatch_place_kernel(const int* __restrict__ topk_idx, int A, int E, int k,
                      const int* __restrict__ bases, const int* __restrict__ offsets,
                      int* __restrict__ rows, int* __restrict__ dest) {
  extern __shared__ int warp_count[];   // [32][E]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) warp_count[i] = 0;
  __syncthreads();
  const int a = blockIdx.x * DISPATCH_CHUNK + threadIdx.x;
  const int e = a < A ? topk_idx[a] : -1 - lane;   // idle lanes match nobody
  const unsigned same = __match_any_sync(0xffffffffu, e);
  const int rank = __popc(same & ((1u << lane) - 1u));
  if (a < A && rank == 0) warp_count[warp * E + e] = __popc(same);
  __syncthreads();
  if (a < A) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_count[w * E + e];
    const int r = offsets[e] + bases[(size_t)blockIdx.x * E + e] + before + rank;
    rows[r] = a / k;
    dest[a] = r;
  }
}

// scratch: ints for ix_moe_dispatch_scratch_ints(T, E, k) entries, or null to force the
// single-block kernel.
IX_API int ix_moe_dispatch_scratch_ints(int T, int E, int k) {
  const long long A = (long long)T * k;
  if (A <= 512 || E > DISPATCH_MAX_E) return 0;
  return (int)(((A + DISPATCH_CHUNK - 1) / DISPATCH_CHUNK) * E);
}

IX_API int ix_moe_dispatch(const int* topk_idx, int T, int E, int k, int* offsets, int* rows,
                           int* dest, int* scratch, cudaStream_t stream) {
  if (E <= 0 || k <= 0 || E > ROUTER_MAX_EXPERTS) return IX_ERR_SIZE;
  if (T < 0) return IX_ERR_SIZE;
  const int A = T * k;
  if (scratch && A > 512 && E <= DISPATCH_MAX_E) {
    const int blocks = (A + DISPATCH_CHUNK - 1) / DISPATCH_CHUNK;
    dispatch_count_kernel<<<blocks, DISPATCH_CHUNK, 0, stream>>>(topk_idx, A, E, scratch);
    dispatch_scan_kernel<<<1, DISPATCH_MAX_E, 0, stream>>>(scratch, blocks, E, offsets);
    dispatch_place_kernel<<<blocks, DISPATCH_CHUNK, 32 * E * sizeof(int), stream>>>(
        topk_idx, A, E, k, scratch, offsets, rows, dest);
    return ix_launch_status();
  }
  const int threads = E >= 32 ? 1024 : 32 * E;
  ix_launch(moe_dispatch_kernel, dim3(1), dim3(threads), (E + 1) * sizeof(int), stream, topk_idx,
            A, E, k, offsets, rows, dest);
  return ix_launch_status();
}
