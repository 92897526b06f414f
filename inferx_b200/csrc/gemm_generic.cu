// General matrix product y = x . w^T on the CUDA cores, fp32 accumulation, for
// one weight matrix or for a ragged group of them (one per expert).
//
//   out[r, j] = sum_k x[src(r), k] * w[e(r), j, k]
//
// e(r) is the expert whose [offsets[e], offsets[e+1]) range holds grouped row r,
// src(r) = rows[r] when a gather list is given (the gather of the reference's
// GatherRowsKernel folded into the load), else r.  With DUAL the kernel computes
// the gate and the up projection of a SwiGLU together and writes
// silu(gate) * up, which is the reference's GroupedGemmBf16 + SiluMulFused
// (src/backends/cuda/ops/moe.cu:324-392, src/backends/cuda/ops/layers.cu:512-529).
//
// This is the whole matrix path of the 32-bit mode (true fp32 FFMA, no reduced
// precision mode) and the fallback of the bfloat16 mode for shapes the tensor
// core kernels refuse.  Two kernels:
//
// * tiles (many rows): a block computes BM x BN outputs (128 x 128, or 64 x 128 where
//   a weight matrix meets few rows; half as many columns for the SwiGLU form, which
//   keeps two accumulators), a thread 8 x 8 (or 4 x 8) of them from shared memory,
//   the next k-tile travelling from global memory into registers meanwhile.  Every
//   output element is one accumulator that takes its products in ascending k.
// * rows (at most 16 rows a weight matrix: decode steps): the product is bound by
//   reading the weights once, so a warp streams four weight rows with 16-byte loads,
//   lane l taking the k-chunks l, l + 32, ..., against all the activation rows (which
//   come through L1), and the lanes' sums are added by the shuffle tree.
//
// In either kernel a token's result is formed from that token's data alone in an
// order that does not depend on what else is in the batch; which kernel runs depends
// on the number of rows, so a step of a few tokens and a prompt differ by rounding.
#include "common.cuh"

#define GT_THREADS 256
#define GT_K 16

template <typename TA> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) {
    return *reinterpret_cast<const float4*>(p);
  }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    return make_float4(a.x, a.y, b.x, b.y);
  }
};

// four consecutive k of one row, zero where the row or k is out of range; `vec`:
// K is a multiple of 4 and the base is aligned for a vector load
template <typename TA>
__device__ __forceinline__ float4 load_k4(const TA* row, int k, int K, bool row_ok, bool vec) {
  if (!row_ok || k >= K) return make_float4(0.f, 0.f, 0.f, 0.f);
  if (vec) return Vec4<TA>::load(row + k);
  float4 v;
  v.x = to_f32(row[k]);
  v.y = k + 1 < K ? to_f32(row[k + 1]) : 0.f;
  v.z = k + 2 < K ? to_f32(row[k + 2]) : 0.f;
  v.w = k + 3 < K ? to_f32(row[k + 3]) : 0.f;
  return v;
}

// ---------------------------------------------------------------------------
// tiles
// ---------------------------------------------------------------------------
// BM rows x BN columns a block; a thread (ty, tx) of 16 x 16 owns rows ty*4 + {0..3}
// (+ BM/2 when BM is 128) and columns tx*4 + {0..3} and BN/2 + tx*4 + {0..3}.
template <typename TA, typename TO, bool DUAL, int BM>
__global__ void __launch_bounds__(GT_THREADS)
gemm_tiles_kernel(const TA* __restrict__ x, const int* __restrict__ rows,
                  const int* __restrict__ offsets, const TA* __restrict__ w,
                  TO* __restrict__ out, int M_single, int N, int K, int E,
                  long long w_expert_stride, int up_row_offset, int vec) {
  constexpr int BN = DUAL ? 64 : 128;
  constexpr int RM = BM / 16;            // rows a thread owns: 4 or 8
  constexpr int RN = BN / 16;            // columns a thread owns: 4 or 8
  constexpr int A_LD = BM * GT_K / 4 / GT_THREADS;   // float4 loads of a thread per A tile
  constexpr int B_LD = BN * GT_K / 4 / GT_THREADS;
  __shared__ __align__(16) float As[2][GT_K][BM + 4];
  __shared__ __align__(16) float Bs[2][GT_K][BN + 4];
  __shared__ __align__(16) float Bs2[DUAL ? 2 : 1][DUAL ? GT_K : 1][BN + 4];
  // locate this block's expert and row range
  int e = 0, m0 = 0, m_end = 0;
  {
    int tile = blockIdx.y;
    if (offsets) {
      bool found = false;
      for (int ee = 0; ee < E; ++ee) {
        const int lo = offsets[ee], hi = offsets[ee + 1];
        const int tiles = (hi - lo + BM - 1) / BM;
        if (tile < tiles) {
          e = ee; m0 = lo + tile * BM; m_end = hi; found = true;
          break;
        }
        tile -= tiles;
      }
      if (!found) return;
    } else {
      m0 = tile * BM;
      m_end = M_single;
      if (m0 >= m_end) return;
    }
  }
  const int n0 = blockIdx.x * BN;
  const TA* wb = w + (size_t)e * w_expert_stride;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const bool v = vec != 0;

  // loader mapping: a float4 covers 4 k of one row; 4 threads a row, 64 rows a pass
  const int lr = threadIdx.x / 4;
  const int lk = (threadIdx.x % 4) * 4;
  const TA* arow[A_LD];
  bool arow_ok[A_LD];
#pragma unroll
  for (int i = 0; i < A_LD; ++i) {
    const int r = m0 + lr + 64 * i;
    arow_ok[i] = r < m_end;
    const size_t src = arow_ok[i] ? (rows ? (size_t)rows[r] : (size_t)r) : 0;
    arow[i] = x + src * K;
  }
  const TA* brow[B_LD];
  bool brow_ok[B_LD];
#pragma unroll
  for (int i = 0; i < B_LD; ++i) {
    const int c = n0 + lr + 64 * i;
    brow_ok[i] = c < N;
    brow[i] = wb + (size_t)(brow_ok[i] ? c : 0) * K;
  }
  float4 ra[A_LD], rb[B_LD], rb2[DUAL ? B_LD : 1];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < A_LD; ++i) ra[i] = load_k4(arow[i], k0 + lk, K, arow_ok[i], v);
#pragma unroll
    for (int i = 0; i < B_LD; ++i) {
      rb[i] = load_k4(brow[i], k0 + lk, K, brow_ok[i], v);
      if (DUAL)
        rb2[i] = load_k4(brow[i] + (size_t)up_row_offset * K, k0 + lk, K, brow_ok[i], v);
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int i = 0; i < A_LD; ++i) {
      As[buf][lk + 0][lr + 64 * i] = ra[i].x;
      As[buf][lk + 1][lr + 64 * i] = ra[i].y;
      As[buf][lk + 2][lr + 64 * i] = ra[i].z;
      As[buf][lk + 3][lr + 64 * i] = ra[i].w;
    }
#pragma unroll
    for (int i = 0; i < B_LD; ++i) {
      Bs[buf][lk + 0][lr + 64 * i] = rb[i].x;
      Bs[buf][lk + 1][lr + 64 * i] = rb[i].y;
      Bs[buf][lk + 2][lr + 64 * i] = rb[i].z;
      Bs[buf][lk + 3][lr + 64 * i] = rb[i].w;
      if (DUAL) {
        Bs2[buf][lk + 0][lr + 64 * i] = rb2[i].x;
        Bs2[buf][lk + 1][lr + 64 * i] = rb2[i].y;
        Bs2[buf][lk + 2][lr + 64 * i] = rb2[i].z;
        Bs2[buf][lk + 3][lr + 64 * i] = rb2[i].w;
      }
    }
  };

  float acc[RM][RN], acc2[DUAL ? RM : 1][RN];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < RN; ++j) {
      acc[i][j] = 0.f;
      if (DUAL) acc2[i][j] = 0.f;
    }
  fetch(0);
  stage(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += GT_K) {
    const bool more = k0 + GT_K < K;
    if (more) fetch(k0 + GT_K);            // in flight while this tile is multiplied
#pragma unroll
    for (int kk = 0; kk < GT_K; ++kk) {
      float a[RM], b[RN], b2[DUAL ? RN : 1];
#pragma unroll
      for (int h = 0; h < RM / 4; ++h) {
        const float4 t4 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4 + h * (BM / 2)]);
        a[4 * h] = t4.x; a[4 * h + 1] = t4.y; a[4 * h + 2] = t4.z; a[4 * h + 3] = t4.w;
      }
#pragma unroll
      for (int h = 0; h < RN / 4; ++h) {
        const float4 t4 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4 + h * (BN / 2)]);
        b[4 * h] = t4.x; b[4 * h + 1] = t4.y; b[4 * h + 2] = t4.z; b[4 * h + 3] = t4.w;
        if (DUAL) {
          const float4 u4 =
              *reinterpret_cast<const float4*>(&Bs2[buf][kk][tx * 4 + h * (BN / 2)]);
          b2[4 * h] = u4.x; b2[4 * h + 1] = u4.y; b2[4 * h + 2] = u4.z; b2[4 * h + 3] = u4.w;
        }
      }
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < RN; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (DUAL) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    if (more) {
      stage(buf ^ 1);                      // the other buffer was read a tile ago
      __syncthreads();
      buf ^= 1;
    }
  }
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int r = m0 + ty * 4 + (i & 3) + (i >> 2) * (BM / 2);
    if (r >= m_end) continue;
#pragma unroll
    for (int j = 0; j < RN; ++j) {
      const int c = n0 + tx * 4 + (j & 3) + (j >> 2) * (BN / 2);
      if (c >= N) continue;
      float val = acc[i][j];
      if (DUAL) {
        const float g = val;
        val = g / (1.0f + expf(-g)) * acc2[i][j];
      }
      out[(size_t)r * N + c] = from_f32<TO>(val);
    }
  }
}

// ---------------------------------------------------------------------------
// rows: at most GR_ROWS activation rows a pass against GR_COLS weight rows a warp
// ---------------------------------------------------------------------------
#define GR_ROWS 8
#define GR_WARPS 8

template <typename TA, typename TO, bool DUAL>
__global__ void __launch_bounds__(GR_WARPS * 32)
gemm_rows_kernel(const TA* __restrict__ x, const int* __restrict__ rows,
                 const int* __restrict__ offsets, const TA* __restrict__ w,
                 TO* __restrict__ out, int M_single, int N, int K, long long w_expert_stride,
                 int up_row_offset, int vec) {
  constexpr int COLS = DUAL ? 2 : 4;     // output columns a warp owns
  constexpr int WR = DUAL ? 4 : 4;       // weight rows it streams (gate and up when DUAL)
  const int e = blockIdx.y;
  int lo = 0, hi = M_single;
  if (offsets) {
    lo = offsets[e];
    hi = offsets[e + 1];
  }
  if (lo >= hi) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * GR_WARPS + warp) * COLS;
  if (c0 >= N) return;
  const TA* wb = w + (size_t)e * w_expert_stride;
  const TA* wrow[WR];
  bool wok[WR];
#pragma unroll
  for (int j = 0; j < WR; ++j) {
    const int c = DUAL ? c0 + (j & 1) : c0 + j;
    wok[j] = c < N;
    wrow[j] = wb + ((size_t)(wok[j] ? c : 0) + (DUAL && j >= 2 ? (size_t)up_row_offset : 0)) * K;
  }
  const bool v = vec != 0;
  for (int r0 = lo; r0 < hi; r0 += GR_ROWS) {
    const TA* xrow[GR_ROWS];
    bool xok[GR_ROWS];
#pragma unroll
    for (int i = 0; i < GR_ROWS; ++i) {
      const int r = r0 + i;
      xok[i] = r < hi;
      const size_t src = xok[i] ? (rows ? (size_t)rows[r] : (size_t)r) : 0;
      xrow[i] = x + src * K;
    }
    float acc[GR_ROWS][WR];
#pragma unroll
    for (int i = 0; i < GR_ROWS; ++i)
#pragma unroll
      for (int j = 0; j < WR; ++j) acc[i][j] = 0.f;
    for (int k = lane * 4; k < K; k += 128) {
      float4 wv[WR];
#pragma unroll
      for (int j = 0; j < WR; ++j) wv[j] = load_k4(wrow[j], k, K, wok[j], v);
#pragma unroll
      for (int i = 0; i < GR_ROWS; ++i) {
        if (!xok[i]) continue;             // the same for every lane of the warp
        const float4 xv = load_k4(xrow[i], k, K, true, v);
#pragma unroll
        for (int j = 0; j < WR; ++j) {
          acc[i][j] = fmaf(xv.x, wv[j].x, acc[i][j]);
          acc[i][j] = fmaf(xv.y, wv[j].y, acc[i][j]);
          acc[i][j] = fmaf(xv.z, wv[j].z, acc[i][j]);
          acc[i][j] = fmaf(xv.w, wv[j].w, acc[i][j]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < GR_ROWS; ++i) {
      if (!xok[i]) continue;
#pragma unroll
      for (int j = 0; j < WR; ++j) acc[i][j] = warp_sum(acc[i][j]);
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < COLS; ++j) {
          const int c = c0 + j;
          if (c >= N) continue;
          float val = acc[i][j];
          if (DUAL) {
            const float g = val;
            val = g / (1.0f + expf(-g)) * acc[i][j + 2];
          }
          out[(size_t)(r0 + i) * N + c] = from_f32<TO>(val);
        }
      }
    }
  }
}

// x: [*, K]; w: [E, w_rows, K] with w_rows = N (or 2N when dual: gate rows then up
// rows); out: [A, N].  offsets == null means a single matrix with M rows.
template <typename TA, typename TO, bool DUAL>
static int launch_generic(const void* x, const int* rows, const int* offsets, const void* w,
                          void* out, int M, int N, int K, int E, int max_rows,
                          cudaStream_t stream) {
  const long long w_rows = DUAL ? 2LL * N : N;
  const long long stride = w_rows * K;
  const int esize = (int)sizeof(TA);
  const int vec = (K % 4 == 0 && (((uintptr_t)x | (uintptr_t)w) % (4 * esize)) == 0) ? 1 : 0;
  const int Ms = offsets ? 0 : M;
  // few rows a weight matrix: stream the weights once
  const double per_group = offsets ? (double)max_rows / (double)E : (double)M;
  if (per_group <= (offsets ? 2.0 : 16.0) && E <= 65535) {
    constexpr int COLS = DUAL ? 2 : 4;
    dim3 grid((N + GR_WARPS * COLS - 1) / (GR_WARPS * COLS), E);
    gemm_rows_kernel<TA, TO, DUAL><<<grid, GR_WARPS * 32, 0, stream>>>(
        (const TA*)x, rows, offsets, (const TA*)w, (TO*)out, Ms, N, K, stride, N, vec);
    return ix_launch_status();
  }
  constexpr int BN = DUAL ? 64 : 128;
  const bool small_m = offsets ? per_group <= 96.0 : M <= 64;
  const int bm = small_m ? 64 : 128;
  // grouped: every expert can add one partial tile
  const long long m_tiles = offsets ? (max_rows + bm - 1) / bm + E : (M + bm - 1) / bm;
  if (m_tiles > 65535) return IX_ERR_SIZE;
  dim3 grid((N + BN - 1) / BN, (unsigned)m_tiles);
  if (small_m)
    gemm_tiles_kernel<TA, TO, DUAL, 64><<<grid, GT_THREADS, 0, stream>>>(
        (const TA*)x, rows, offsets, (const TA*)w, (TO*)out, Ms, N, K, E, stride, N, vec);
  else
    gemm_tiles_kernel<TA, TO, DUAL, 128><<<grid, GT_THREADS, 0, stream>>>(
        (const TA*)x, rows, offsets, (const TA*)w, (TO*)out, Ms, N, K, E, stride, N, vec);
  return ix_launch_status();
}

IX_API int ix_gemm_generic(const void* x, const int* rows, const int* offsets, const void* w,
                           void* out, int in_dtype, int out_dtype, int dual, int M, int N, int K,
                           int E, int max_rows, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || E <= 0) return IX_ERR_SIZE;
  if (max_rows <= 0) return IX_OK;
#define IX_GG(TA, TO)                                                                        \
  return dual ? launch_generic<TA, TO, true>(x, rows, offsets, w, out, M, N, K, E, max_rows,  \
                                             stream)                                          \
              : launch_generic<TA, TO, false>(x, rows, offsets, w, out, M, N, K, E, max_rows, \
                                              stream)
  if (in_dtype == IX_F32 && out_dtype == IX_F32) IX_GG(float, float);
  if (in_dtype == IX_BF16 && out_dtype == IX_BF16) IX_GG(bf16, bf16);
  if (in_dtype == IX_BF16 && out_dtype == IX_F32) IX_GG(bf16, float);
#undef IX_GG
  return IX_ERR_DTYPE;
}
