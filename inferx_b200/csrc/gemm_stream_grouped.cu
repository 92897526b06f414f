// Grouped weight-streaming product for decode steps, persistent form.
//
//   out[r, j] = sum_k x[src(r), k] * w[e(r), j, k]          (plain)
//   out[r, j] = silu(x . wg[e, j]) * (x . wu[e, j])          (DUAL: SwiGLU fused)
//
// Same operands, same transposed mma.sync mapping and 16-byte loads straight into
// fragments as gemm_small_m.cu (the reference's GatherRows + GroupedGemmBf16Kernel<1>
// decode variant + SiluMulFused, src/backends/cuda/ops/moe.cu:223-231,324-392,
// src/backends/cuda/ops/layers.cu:512-529).  What differs is how the work is spread.
// With a handful of tokens only some experts have rows, and a grid of one block per
// (expert, column tile) is a wave and a bit of short-lived blocks, each of which
// starts its stream cold.  Here two blocks per SM stay for the whole launch: a block
// lists the experts that have rows, takes an equal share of the list of (active
// expert, 16-column tile) items, and walks it; its eight warps split K of every item
// (warp w takes k-steps w, w + 8, ...) and add their partial sums through shared
// memory in warp order, and a warp's ring of loads runs on into the next item while
// the current one is being finished, so the stream from HBM never stops at an item's
// edge.  A row's result is formed the same way whatever else is in the batch.
//
// Requires bf16, K a multiple of 8 and at least 256, E <= 1024; experts with more
// than 8 * NT rows re-read their weights per pass (through L2).
#include "common.cuh"

#define GS_THREADS 256
#define GS_WARPS 8
#define GS_MAX_EXPERTS 1024

__device__ __forceinline__ uint4 gs_ld_stream16(const bf16* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ void gs_mma(float* c, unsigned a0, unsigned a1, unsigned a2,
                                       unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Where a warp stands in its sequence of k-steps: item (tile of an active expert),
// pass over the expert's rows, k-step of the pass; and what it needs to load there.
template <int NT> struct GsCursor {
  int tile, r0, q, hi;
  bool valid;
  const bf16 *wa, *wb;          // weight rows g and g + 8 of the tile (gate rows when DUAL)
  const bf16* xrow[NT];
  bool ja_ok, jb_ok, xok[NT];
};

template <bool DUAL, int NT>
__global__ void __launch_bounds__(GS_THREADS, 2)
gemm_stream_grouped_kernel(const bf16* __restrict__ x, const int* __restrict__ rows,
                           const int* __restrict__ offsets, const bf16* __restrict__ w,
                           bf16* __restrict__ out, int N, int K, int E,
                           long long w_expert_stride) {
  constexpr int D = DUAL ? 3 : (NT > 1 ? 4 : 6);      // k-steps in flight per warp
  __shared__ int act[GS_MAX_EXPERTS];
  __shared__ int n_act_s;
  __shared__ float red[2][DUAL ? 2 : 1][GS_WARPS][NT][4][32];
  IX_PDL_WAIT();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  if (warp == 0) {
    int base = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const bool on = e < E && offsets[e + 1] > offsets[e];
      const unsigned m = __ballot_sync(0xffffffffu, on);
      if (on) act[base + __popc(m & ((1u << lane) - 1u))] = e;
      base += __popc(m);
    }
    if (lane == 0) n_act_s = base;
  }
  __syncthreads();
  const int tiles_per_e = (N + 15) >> 4;
  const long long total = (long long)n_act_s * tiles_per_e;
  const int t_begin = (int)(total * blockIdx.x / gridDim.x);
  const int t_end = (int)(total * (blockIdx.x + 1) / gridDim.x);
  const int ksteps = (K + 31) >> 5;
  const int my_steps = (ksteps - warp + GS_WARPS - 1) / GS_WARPS;   // >= 1: K >= 256
  const size_t up_off = (size_t)N * K;     // up rows follow the gate rows (DUAL)
  const uint4 zero = make_uint4(0, 0, 0, 0);

  // position a cursor at the start of (tile, pass); r0 < 0 means the first pass
  auto enter = [&](GsCursor<NT>& c) {
    c.q = 0;
    c.valid = c.tile < t_end;
    if (!c.valid) return;
    const int a = c.tile / tiles_per_e, j = c.tile - a * tiles_per_e;
    const int e = act[a];
    const int lo = offsets[e];
    c.hi = offsets[e + 1];
    if (c.r0 < 0) c.r0 = lo;
    const int ja = j * 16 + g, jb = ja + 8;
    c.ja_ok = ja < N;
    c.jb_ok = jb < N;
    const bf16* wbase = w + (size_t)e * w_expert_stride;
    c.wa = wbase + (size_t)(c.ja_ok ? ja : 0) * K;
    c.wb = wbase + (size_t)(c.jb_ok ? jb : 0) * K;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int r = c.r0 + i * 8 + g;
      c.xok[i] = r < c.hi;
      const size_t src = c.xok[i] ? (rows ? (size_t)rows[r] : (size_t)r) : 0;
      c.xrow[i] = x + src * K;
    }
  };
  // one k-step further; true when that was the last step of an item's pass
  auto advance = [&](GsCursor<NT>& c) {
    if (++c.q < my_steps) return false;
    c.r0 += 8 * NT;
    if (c.r0 >= c.hi) {
      c.tile += 1;
      c.r0 = -1;
    }
    return true;
  };

  uint4 va[D], vb[D], vua[DUAL ? D : 1], vub[DUAL ? D : 1], vx[D][NT];
  auto fetch = [&](int u, const GsCursor<NT>& c) {
    const int kb = (warp + c.q * GS_WARPS) * 32 + t * 8;
    const bool kok = c.valid && kb < K;
    va[u] = (kok && c.ja_ok) ? gs_ld_stream16(c.wa + kb) : zero;
    vb[u] = (kok && c.jb_ok) ? gs_ld_stream16(c.wb + kb) : zero;
    if (DUAL) {
      vua[u] = (kok && c.ja_ok) ? gs_ld_stream16(c.wa + up_off + kb) : zero;
      vub[u] = (kok && c.jb_ok) ? gs_ld_stream16(c.wb + up_off + kb) : zero;
    }
#pragma unroll
    for (int i = 0; i < NT; ++i)
      vx[u][i] = (kok && c.xok[i]) ? *reinterpret_cast<const uint4*>(c.xrow[i] + kb) : zero;
  };

  GsCursor<NT> fc, cc;            // where loads are issued, where sums are formed
  fc.tile = cc.tile = t_begin;
  fc.r0 = cc.r0 = -1;
  enter(fc);
  enter(cc);
#pragma unroll
  for (int u = 0; u < D; ++u) {
    fetch(u, fc);
    if (fc.valid && advance(fc)) enter(fc);
  }
  float acc[NT][4], acc2[DUAL ? NT : 1][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      acc[i][c] = 0.f;
      if (DUAL) acc2[i][c] = 0.f;
    }
  int items_done = 0;
  while (cc.valid) {
#pragma unroll
    for (int u = 0; u < D; ++u) {
      if (cc.valid) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          gs_mma(acc[i], va[u].x, vb[u].x, va[u].y, vb[u].y, vx[u][i].x, vx[u][i].y);
          gs_mma(acc[i], va[u].z, vb[u].z, va[u].w, vb[u].w, vx[u][i].z, vx[u][i].w);
          if (DUAL) {
            gs_mma(acc2[i], vua[u].x, vub[u].x, vua[u].y, vub[u].y, vx[u][i].x, vx[u][i].y);
            gs_mma(acc2[i], vua[u].z, vub[u].z, vua[u].w, vub[u].w, vx[u][i].z, vx[u][i].w);
          }
        }
        // the slot is free: the next load of the ring goes out before anything else
        fetch(u, fc);
        if (fc.valid && advance(fc)) enter(fc);
        const int done_tile = cc.tile, done_r0 = cc.r0, done_hi = cc.hi;
        if (advance(cc)) {
          // the warps' partial sums of this (item, pass), added in warp order
          const int buf = items_done & 1;
#pragma unroll
          for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              red[buf][0][warp][i][c][lane] = acc[i][c];
              acc[i][c] = 0.f;
              if (DUAL) {
                red[buf][DUAL ? 1 : 0][warp][i][c][lane] = acc2[i][c];
                acc2[i][c] = 0.f;
              }
            }
          __syncthreads();
          if (threadIdx.x < NT * 128) {
            const int idx = threadIdx.x;
            const int l = idx & 31, c = (idx >> 5) & 3, i = idx >> 7;
            float v = 0.f, v2 = 0.f;
#pragma unroll
            for (int q = 0; q < GS_WARPS; ++q) {
              v += red[buf][0][q][i][c][l];
              if (DUAL) v2 += red[buf][DUAL ? 1 : 0][q][i][c][l];
            }
            const int a = done_tile / tiles_per_e, jt = done_tile - a * tiles_per_e;
            const int gg = l >> 2, tt = l & 3;
            const int j = jt * 16 + ((c & 2) ? gg + 8 : gg);
            const int r = done_r0 + i * 8 + 2 * tt + (c & 1);
            if (j < N && r < done_hi) {
              if (DUAL) v = v / (1.0f + __expf(-v)) * v2;
              out[(size_t)r * N + j] = __float2bfloat16_rn(v);
            }
          }
          ++items_done;
          enter(cc);
        }
      }
    }
  }
}

template <bool DUAL, int NT>
static int launch_stream_grouped(const void* x, const int* rows, const int* offsets,
                                 const void* w, void* out, int N, int K, int E,
                                 cudaStream_t stream) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms <= 0)
      sms = 148;
  }
  const long long w_rows = DUAL ? 2LL * N : N;
  ix_launch(gemm_stream_grouped_kernel<DUAL, NT>, dim3(2 * sms), dim3(GS_THREADS), 0, stream,
            (const bf16*)x, rows, offsets, (const bf16*)w, (bf16*)out, N, K, E, w_rows * K);
  return ix_launch_status();
}

// x: [*, K] bf16; rows: source row of each grouped row, or null when x is already
// grouped; offsets: [E + 1]; w: [E, N (or 2N when dual), K] bf16; out: [rows, N] bf16.
// rows_per_pass: 8 or 16 activation rows handled per pass over an expert's weights.
IX_API int ix_gemm_stream_grouped(const void* x, const int* rows, const int* offsets,
                                  const void* w, void* out, int dual, int N, int K, int E,
                                  int rows_per_pass, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || E <= 0 || offsets == nullptr) return IX_ERR_SIZE;
  if (K % 8 != 0 || K < 256 || E > GS_MAX_EXPERTS) return IX_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return IX_ERR_ALIGN;
  if (rows_per_pass > 8) {
    if (dual) return launch_stream_grouped<true, 2>(x, rows, offsets, w, out, N, K, E, stream);
    return launch_stream_grouped<false, 2>(x, rows, offsets, w, out, N, K, E, stream);
  }
  if (dual) return launch_stream_grouped<true, 1>(x, rows, offsets, w, out, N, K, E, stream);
  return launch_stream_grouped<false, 1>(x, rows, offsets, w, out, N, K, E, stream);
}
