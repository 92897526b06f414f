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
// core kernels refuse.  Every output element accumulates over k in ascending
// order in steps fixed by the tile depth, whatever the number of rows, so a
// token's result does not depend on what else is in the batch.
#include "common.cuh"

#define GT_M 64
#define GT_N 64
#define GT_K 16
#define GT_THREADS 256

template <typename TA, typename TO, bool DUAL>
__global__ void __launch_bounds__(GT_THREADS)
gemm_generic_kernel(const TA* __restrict__ x, const int* __restrict__ rows,
                    const int* __restrict__ offsets, const TA* __restrict__ w,
                    TO* __restrict__ out, int M_single, int N, int K, int E,
                    long long w_expert_stride, int up_row_offset) {
  __shared__ float As[GT_K][GT_M + 4];
  __shared__ float Bs[GT_K][GT_N + 4];
  __shared__ float Bs2[DUAL ? GT_K : 1][GT_N + 4];
  // locate this block's expert and row range
  int e = 0, m0 = 0, m_end = 0;
  {
    int tile = blockIdx.y;
    if (offsets) {
      bool found = false;
      for (int ee = 0; ee < E; ++ee) {
        const int lo = offsets[ee], hi = offsets[ee + 1];
        const int tiles = (hi - lo + GT_M - 1) / GT_M;
        if (tile < tiles) {
          e = ee; m0 = lo + tile * GT_M; m_end = hi; found = true;
          break;
        }
        tile -= tiles;
      }
      if (!found) return;
    } else {
      m0 = tile * GT_M;
      m_end = M_single;
      if (m0 >= m_end) return;
    }
  }
  const int n0 = blockIdx.x * GT_N;
  const TA* wb = w + (size_t)e * w_expert_stride;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4x4 each
  float acc[4][4], acc2[DUAL ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = 0.f;
      if (DUAL) acc2[i][j] = 0.f;
    }
  // loader mapping: 256 threads load 64 rows x 16 k: thread -> (row = tid/4, 4 k's)
  const int lr = threadIdx.x / 4;
  const int lk = (threadIdx.x % 4) * 4;
  const int arow = m0 + lr;
  const bool arow_ok = arow < m_end;
  const size_t asrc = arow_ok ? (rows ? (size_t)rows[arow] : (size_t)arow) : 0;
  const int brow = n0 + lr;
  const bool brow_ok = brow < N;
  for (int k0 = 0; k0 < K; k0 += GT_K) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kk = k0 + lk + i;
      const bool kok = kk < K;
      As[lk + i][lr] = (arow_ok && kok) ? to_f32(x[asrc * K + kk]) : 0.f;
      Bs[lk + i][lr] = (brow_ok && kok) ? to_f32(wb[(size_t)brow * K + kk]) : 0.f;
      if (DUAL)
        Bs2[lk + i][lr] =
            (brow_ok && kok) ? to_f32(wb[(size_t)(brow + up_row_offset) * K + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GT_K; ++kk) {
      float a[4], b[4], b2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b[j] = Bs[kk][tx * 4 + j];
        if (DUAL) b2[j] = Bs2[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (DUAL) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c >= N) continue;
      float v = acc[i][j];
      if (DUAL) {
        const float g = v;
        v = g / (1.0f + expf(-g)) * acc2[i][j];
      }
      out[(size_t)r * N + c] = from_f32<TO>(v);
    }
  }
}

// x: [*, K]; w: [E, w_rows, K] with w_rows = N (or 2N when dual: gate rows then up
// rows); out: [A, N].  offsets == null means a single matrix with M rows.
IX_API int ix_gemm_generic(const void* x, const int* rows, const int* offsets, const void* w,
                           void* out, int in_dtype, int out_dtype, int dual, int M, int N, int K,
                           int E, int max_rows, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || E <= 0) return IX_ERR_SIZE;
  if (max_rows <= 0) return IX_OK;
  const long long w_rows = dual ? 2LL * N : N;
  const long long stride = w_rows * K;
  // grouped: every expert can add one partial tile
  const int m_tiles = offsets ? (max_rows + GT_M - 1) / GT_M + E : (M + GT_M - 1) / GT_M;
  if (m_tiles > 65535) return IX_ERR_SIZE;
  dim3 grid((N + GT_N - 1) / GT_N, m_tiles);
  const int Ms = offsets ? 0 : M;
#define IX_GG(TA, TO, D)                                                                   \
  gemm_generic_kernel<TA, TO, D><<<grid, GT_THREADS, 0, stream>>>(                          \
      (const TA*)x, rows, offsets, (const TA*)w, (TO*)out, Ms, N, K, E, stride, N)
  if (in_dtype == IX_F32 && out_dtype == IX_F32) {
    if (dual) IX_GG(float, float, true); else IX_GG(float, float, false);
  } else if (in_dtype == IX_BF16 && out_dtype == IX_BF16) {
    if (dual) IX_GG(bf16, bf16, true); else IX_GG(bf16, bf16, false);
  } else if (in_dtype == IX_BF16 && out_dtype == IX_F32) {
    if (dual) IX_GG(bf16, float, true); else IX_GG(bf16, float, false);
  } else {
    return IX_ERR_DTYPE;
  }
#undef IX_GG
  return ix_launch_status();
}
