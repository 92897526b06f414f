// Weight-streaming matrix product for few rows: y = x . w^T where every weight
// matrix meets at most a few dozen activation rows (decode steps).  The work is
// bandwidth: each weight element is read once, with 16-byte loads straight from
// global memory into tensor-core fragments.
//
//   out[r, j] = sum_k x[src(r), k] * w[e(r), j, k]          (plain)
//   out[r, j] = silu(x . wg[e, j]) * (x . wu[e, j])          (DUAL: SwiGLU fused)
//
// Groups are the experts of a mixture (ragged row ranges from `offsets`, source
// rows from `rows`: the reference's GatherRows + GroupedGemmBf16Kernel<1> decode
// variant + SiluMulFused, src/backends/cuda/ops/moe.cu:223-231,324-392,
// src/backends/cuda/ops/layers.cu:512-529), or a single dense matrix with a few
// rows (E = 1), where the reference calls cuBLASLt.
//
// Mapping: the product is computed transposed, out^T = w . x^T, with
// mma.sync.m16n8k16: sixteen weight rows (output columns) are the M side, eight
// activation rows the N side.  A thread's 16-byte load of a weight row holds eight
// consecutive k; the same eight k of its activation row are loaded the same way,
// and both are fed to the same k-slots of two mma instructions, so no shuffle or
// shared-memory staging is needed (a dot product does not care in which order k is
// visited, as long as both operands agree).  A block owns 16 output columns of one
// group; its 8 warps split K and their partial sums are added through shared
// memory in warp order, so a row's result does not depend on which other rows
// share the tile.  Groups with more rows than one pass holds re-read their
// weights (through L2).
//
// Requires bf16 inputs and K a multiple of 8 (16-byte chunks); refuses otherwise.
#include "common.cuh"

#define SM_THREADS 256
#define SM_WARPS 8

__device__ __forceinline__ uint4 ld_stream16(const bf16* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void mma_bf16_16816(float* c, unsigned a0, unsigned a1, unsigned a2,
                                               unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TO, bool DUAL, int NT, int KSPLIT>
__global__ void __launch_bounds__(SM_THREADS, (NT >= 4 || (NT >= 2 && KSPLIT == 1)) ? 1 : 2)
gemm_small_m_kernel(const bf16* __restrict__ x, const int* __restrict__ rows,
                    const int* __restrict__ offsets, const bf16* __restrict__ w,
                    TO* __restrict__ out, int M_single, int N, int K, long long w_expert_stride,
                    int offsets_settled) {
  constexpr int TILES = SM_WARPS / KSPLIT;        // 16-column tiles per block
  // k-steps kept in flight per warp: deep when a warp streams all of K for its tile,
  // shallower when K is split over warps (more warps resident instead)
  constexpr int D = KSPLIT == 1 ? (DUAL ? 4 : (NT >= 4 ? 4 : 8)) : (DUAL ? 2 : (NT >= 4 ? 2 : 4));
  __shared__ float red[KSPLIT > 1 ? (DUAL ? 2 : 1) : 1][KSPLIT > 1 ? SM_WARPS : 1]
                      [KSPLIT > 1 ? NT : 1][4][32];
  const int e = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tile = warp / KSPLIT, ks = warp % KSPLIT;
  const int j0 = (blockIdx.x * TILES + tile) * 16;
  const int ja = j0 + g, jb = j0 + g + 8;
  const bool ja_ok = ja < N, jb_ok = jb < N;
  const bf16* wbase = w + (size_t)e * w_expert_stride;
  const bf16* wa = wbase + (size_t)(ja_ok ? ja : 0) * K;
  const bf16* wb = wbase + (size_t)(jb_ok ? jb : 0) * K;
  const bf16* ua = wa + (size_t)N * K;   // up rows follow the gate rows (DUAL)
  const bf16* ub = wb + (size_t)N * K;
  const int ksteps = (K + 31) >> 5;
  const int my_steps = ksteps > ks ? (ksteps - ks + KSPLIT - 1) / KSPLIT : 0;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // a ring of D k-steps in registers: weights and the matching activations
  uint4 va[D], vb[D], vua[DUAL ? D : 1], vub[DUAL ? D : 1], vx[D][NT];
  auto fetch_w = [&](int u, int idx) {
    const int kb = (ks + idx * KSPLIT) * 32 + t * 8;
    const bool kok = idx < my_steps && kb < K;
    va[u] = (kok && ja_ok) ? ld_stream16(wa + kb) : zero;
    vb[u] = (kok && jb_ok) ? ld_stream16(wb + kb) : zero;
    if (DUAL) {
      vua[u] = (kok && ja_ok) ? ld_stream16(ua + kb) : zero;
      vub[u] = (kok && jb_ok) ? ld_stream16(ub + kb) : zero;
    }
  };
  // Weights are never written on the device, so the first loads of the weight stream can
  // go out before the wait on the predecessor in the stream and be in flight while it
  // drains: always for a single matrix (it is wanted whatever the predecessor wrote), and
  // for groups when the caller says that `offsets` was written at least two launches
  // back (the predecessor itself waited for that launch before it let this one start).
  const bool early = offsets == nullptr || offsets_settled != 0;
  int lo = 0, hi = M_single;
  if (early) {
    if (offsets) {
      lo = offsets[e];
      hi = offsets[e + 1];
    }
    if (lo >= hi) return;
#pragma unroll
    for (int u = 0; u < D; ++u) fetch_w(u, u);
  }
  IX_PDL_WAIT();
  if (!early) {
    lo = offsets[e];
    hi = offsets[e + 1];
    if (lo >= hi) return;
  }

  for (int r0 = lo; r0 < hi; r0 += 8 * NT) {
    const bf16* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int r = r0 + i * 8 + g;
      xok[i] = r < hi;
      const size_t src = xok[i] ? (rows ? (size_t)rows[r] : (size_t)r) : 0;
      xrow[i] = x + src * K;
    }
    float acc[NT][4], acc2[DUAL ? NT : 1][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc[i][c] = 0.f;
        if (DUAL) acc2[i][c] = 0.f;
      }
    auto fetch_x = [&](int u, int idx) {
      const int kb = (ks + idx * KSPLIT) * 32 + t * 8;
      const bool kok = idx < my_steps && kb < K;
#pragma unroll
      for (int i = 0; i < NT; ++i)
        vx[u][i] = (kok && xok[i]) ? *reinterpret_cast<const uint4*>(xrow[i] + kb) : zero;
    };
    auto fetch = [&](int u, int idx) {
      fetch_w(u, idx);
      fetch_x(u, idx);
    };
    if (early && r0 == lo) {
#pragma unroll
      for (int u = 0; u < D; ++u) fetch_x(u, u);
    } else {
#pragma unroll
      for (int u = 0; u < D; ++u) fetch(u, u);
    }
    for (int base = 0; base < my_steps; base += D) {
#pragma unroll
      for (int u = 0; u < D; ++u) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          mma_bf16_16816(acc[i], va[u].x, vb[u].x, va[u].y, vb[u].y, vx[u][i].x, vx[u][i].y);
          mma_bf16_16816(acc[i], va[u].z, vb[u].z, va[u].w, vb[u].w, vx[u][i].z, vx[u][i].w);
          if (DUAL) {
            mma_bf16_16816(acc2[i], vua[u].x, vub[u].x, vua[u].y, vub[u].y, vx[u][i].x,
                           vx[u][i].y);
            mma_bf16_16816(acc2[i], vua[u].z, vub[u].z, vua[u].w, vub[u].w, vx[u][i].z,
                           vx[u][i].w);
          }
        }
        fetch(u, base + u + D);   // zeros beyond the last step
      }
    }
    if (KSPLIT == 1) {
      // this warp holds complete sums: c0,c1 -> (column g, rows 2t, 2t+1); c2,c3 -> column g+8
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int j = (c & 2) ? jb : ja;
          const int r = r0 + i * 8 + 2 * t + (c & 1);
          if (j < N && r < hi) {
            float v = acc[i][c];
            if (DUAL) v = v / (1.0f + __expf(-v)) * acc2[i][c];
            out[(size_t)r * N + j] = from_f32<TO>(v);
          }
        }
    } else {
      __syncthreads();   // the previous pass has read its sums
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          red[0][warp][i][c][lane] = acc[i][c];
          if (DUAL) red[DUAL ? 1 : 0][warp][i][c][lane] = acc2[i][c];
        }
      __syncthreads();
      for (int idx = threadIdx.x; idx < TILES * NT * 128; idx += SM_THREADS) {
        const int l = idx & 31, c = (idx >> 5) & 3, i = (idx >> 7) % NT, ti = idx / (NT * 128);
        float v = 0.f, v2 = 0.f;
#pragma unroll
        for (int q = 0; q < KSPLIT; ++q) {
          v += red[0][ti * KSPLIT + q][i][c][l];
          if (DUAL) v2 += red[DUAL ? 1 : 0][ti * KSPLIT + q][i][c][l];
        }
        const int gg = l >> 2, tt = l & 3;
        const int j = (blockIdx.x * TILES + ti) * 16 + ((c & 2) ? gg + 8 : gg);
        const int r = r0 + i * 8 + 2 * tt + (c & 1);
        if (j < N && r < hi) {
          if (DUAL) v = v / (1.0f + __expf(-v)) * v2;
          out[(size_t)r * N + j] = from_f32<TO>(v);
        }
      }
    }
  }
}

template <typename TO, bool DUAL, int NT, int KSPLIT>
static int launch_small_m2(const void* x, const int* rows, const int* offsets, const void* w,
                           void* out, int M, int N, int K, int E, int settled,
                           cudaStream_t stream) {
  if (E > 65535) return IX_ERR_SIZE;
  const long long w_rows = DUAL ? 2LL * N : N;
  constexpr int TILES = SM_WARPS / KSPLIT;
  dim3 grid((N + 16 * TILES - 1) / (16 * TILES), E);
  ix_launch(gemm_small_m_kernel<TO, DUAL, NT, KSPLIT>, grid, dim3(SM_THREADS), 0, stream,
            (const bf16*)x, rows, offsets, (const bf16*)w, (TO*)out, offsets ? 0 : M, N, K,
            w_rows * K, settled);
  return ix_launch_status();
}

template <typename TO, bool DUAL, int NT>
static int launch_small_m(const void* x, const int* rows, const int* offsets, const void* w,
                          void* out, int M, int N, int K, int E, int active_groups, int settled,
                          cudaStream_t stream) {
  // enough warps to keep every SM streaming: split K over warps when there are few tiles
  const long long tiles = (long long)((N + 15) / 16) * (active_groups > 0 ? active_groups : 1);
  int ksplit = 1;
  while (ksplit < 8 && tiles * ksplit < 148 * 8) ksplit *= 2;
  if (ksplit == 1)
    return launch_small_m2<TO, DUAL, NT, 1>(x, rows, offsets, w, out, M, N, K, E, settled, stream);
  if (ksplit == 2)
    return launch_small_m2<TO, DUAL, NT, 2>(x, rows, offsets, w, out, M, N, K, E, settled, stream);
  if (ksplit == 4)
    return launch_small_m2<TO, DUAL, NT, 4>(x, rows, offsets, w, out, M, N, K, E, settled, stream);
  return launch_small_m2<TO, DUAL, NT, 8>(x, rows, offsets, w, out, M, N, K, E, settled, stream);
}

// x: [*, K] bf16; w: [E, N (or 2N when dual), K] bf16; out: [rows, N] bf16 or fp32.
// offsets == null: one matrix (E must be 1) with M rows.  rows_per_pass: 8, 16 or 32
// activation rows handled per pass over a group's weights.  active_groups: how many
// groups are expected to have rows (a hint for how to spread the work; 0 = all).
// offsets_settled: nonzero when `offsets` was written at least two launches back in the
// stream, which lets a grouped launch start its weight stream before its wait.
IX_API int ix_gemm_small_m(const void* x, const int* rows, const int* offsets, const void* w,
                           void* out, int out_dtype, int dual, int M, int N, int K, int E,
                           int rows_per_pass, int active_groups, int offsets_settled,
                           cudaStream_t stream) {
  if (N <= 0 || K <= 0 || E <= 0) return IX_ERR_SIZE;
  if (K % 8 != 0) return IX_ERR_UNSUPPORTED;
  if (!offsets && E != 1) return IX_ERR_SIZE;
  if (!offsets && M <= 0) return IX_OK;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return IX_ERR_ALIGN;
  const int nt = rows_per_pass > 16 ? 4 : (rows_per_pass > 8 ? 2 : 1);
  if (active_groups <= 0 || active_groups > E) active_groups = E;
#define IX_SM(TO, D)                                                                          \
  do {                                                                                        \
    if (nt == 4) return launch_small_m<TO, D, 4>(x, rows, offsets, w, out, M, N, K, E, active_groups, offsets_settled, stream); \
    if (nt == 2) return launch_small_m<TO, D, 2>(x, rows, offsets, w, out, M, N, K, E, active_groups, offsets_settled, stream); \
    return launch_small_m<TO, D, 1>(x, rows, offsets, w, out, M, N, K, E, active_groups, offsets_settled, stream); \
  } while (0)
  if (out_dtype == IX_BF16) {
    if (dual) IX_SM(bf16, true);
    IX_SM(bf16, false);
  }
  if (out_dtype == IX_F32) {
    if (dual) IX_SM(float, true);
    IX_SM(float, false);
  }
#undef IX_SM
  return IX_ERR_DTYPE;
}
