// For a step of a few tokens: the fused Q/K/V projection with what follows it in the
// layer done in the product's epilogue: the Q/K/V biases, the rotation of Q and K by
// position, Q written densely, the rotated K and the V written into their cache pages.
// One launch where the step would otherwise run the weight-streaming product
// (gemm_small_m.cu) and then the split + rotate + append kernel (rope_cache.cu);
// the reference runs four (cuBLASLt, SplitQkvKernel, RopeKernel, AppendKvKernel:
// src/model/qwen2.cc:920-931, src/backends/cuda/ops/layers.cu:80-115,195-219,485-510).
//
// The product is the one of gemm_small_m.cu: out^T = w . x^T by mma.sync.m16n8k16,
// sixteen weight rows on the M side, eight tokens on the N side, weights streamed once
// from global memory through a ring of registers, K split over four warps whose partial
// sums are added in warp order.  What differs is which columns a block owns: the
// half-split rotation pairs dimension d of a head with d + head_dim/2, so a block takes
// sixteen dimensions of the first half of one head together with the sixteen that pair
// with them, and the thread that adds up one finishes both.
//
// The projection's result is rounded to bfloat16 before the bias is added, as it is
// when the product and the rotation are separate kernels with a bfloat16 tensor in
// between; the arithmetic after that is the rotation kernel's (fp32, accurate sincosf).
//
// Takes bf16, K a multiple of 8, head_dim a multiple of 32, a full rotation
// (rot == head_dim) or none (rot == 0), at most 16 tokens; refuses otherwise.
#include "common.cuh"

#define QP_THREADS 256
#define QP_KSPLIT 4
#define QP_D 4

__device__ __forceinline__ uint4 qp_ld_stream16(const bf16* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void qp_mma(float* c, unsigned a0, unsigned a1, unsigned a2,
                                       unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>
__global__ void __launch_bounds__(QP_THREADS, 2)
qkv_project_rope_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                        const float* __restrict__ bias, const int* __restrict__ positions,
                        const float* __restrict__ inv_freq, int rot,
                        const int* __restrict__ slots, bf16* __restrict__ q_out,
                        bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int page_size,
                        int T, int K, int heads, int kvh, int hd) {
  __shared__ float red[2 * QP_KSPLIT][NT][4][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tile = warp / QP_KSPLIT, ks = warp % QP_KSPLIT;
  const int half = hd >> 1;
  const int per_head = half >> 4;                  // blocks per head
  const int head = blockIdx.x / per_head;          // q heads, then k heads, then v heads
  const int d0 = (blockIdx.x - head * per_head) * 16;
  const int col0 = head * hd + d0 + tile * half;   // first of this warp's sixteen columns
  const bf16* wa = w + (size_t)(col0 + g) * K;
  const bf16* wb = w + (size_t)(col0 + g + 8) * K;
  const int ksteps = (K + 31) >> 5;
  const int my_steps = ksteps > ks ? (ksteps - ks + QP_KSPLIT - 1) / QP_KSPLIT : 0;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 va[QP_D], vb[QP_D], vx[QP_D][NT];
  auto fetch_w = [&](int u, int idx) {
    const int kb = (ks + idx * QP_KSPLIT) * 32 + t * 8;
    const bool kok = idx < my_steps && kb < K;
    va[u] = kok ? qp_ld_stream16(wa + kb) : zero;
    vb[u] = kok ? qp_ld_stream16(wb + kb) : zero;
  };
  // the weights are never written on the device: their first loads go out while the
  // preceding kernel drains
#pragma unroll
  for (int u = 0; u < QP_D; ++u) fetch_w(u, u);
  IX_PDL_WAIT();

  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int r = i * 8 + g;
    xok[i] = r < T;
    xrow[i] = x + (size_t)(xok[i] ? r : 0) * K;
  }
  auto fetch_x = [&](int u, int idx) {
    const int kb = (ks + idx * QP_KSPLIT) * 32 + t * 8;
    const bool kok = idx < my_steps && kb < K;
#pragma unroll
    for (int i = 0; i < NT; ++i)
      vx[u][i] = (kok && xok[i]) ? *reinterpret_cast<const uint4*>(xrow[i] + kb) : zero;
  };
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
#pragma unroll
  for (int u = 0; u < QP_D; ++u) fetch_x(u, u);
  for (int base = 0; base < my_steps; base += QP_D) {
#pragma unroll
    for (int u = 0; u < QP_D; ++u) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        qp_mma(acc[i], va[u].x, vb[u].x, va[u].y, vb[u].y, vx[u][i].x, vx[u][i].y);
        qp_mma(acc[i], va[u].z, vb[u].z, va[u].w, vb[u].w, vx[u][i].z, vx[u][i].w);
      }
      fetch_w(u, base + u + QP_D);   // zeros beyond the last step
      fetch_x(u, base + u + QP_D);
    }
  }
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) red[warp][i][c][lane] = acc[i][c];
  __syncthreads();

  // c0,c1 -> (column g, rows 2t, 2t+1); c2,c3 -> column g + 8
  const bool rotated = rot > 0 && head < heads + kvh;
  for (int idx = threadIdx.x; idx < NT * 128; idx += QP_THREADS) {
    const int l = idx & 31, c = (idx >> 5) & 3, i = idx >> 7;
    const int r = i * 8 + 2 * (l & 3) + (c & 1);
    if (r >= T) continue;
    float v1 = 0.f, v2 = 0.f;
#pragma unroll
    for (int q = 0; q < QP_KSPLIT; ++q) {
      v1 += red[q][i][c][l];
      v2 += red[QP_KSPLIT + q][i][c][l];
    }
    const int d1 = d0 + ((c & 2) ? (l >> 2) + 8 : (l >> 2));   // dimension in the first half
    const int d2 = d1 + half;
    const int c1 = head * hd + d1, c2 = head * hd + d2;
    // the projection as a bfloat16 tensor, then bias and rotation in fp32
    float x1 = __bfloat162float(__float2bfloat16_rn(v1));
    float x2 = __bfloat162float(__float2bfloat16_rn(v2));
    if (bias) {
      x1 += bias[c1];
      x2 += bias[c2];
    }
    float o1 = x1, o2 = x2;
    if (rotated) {
      float sn, cs;
      sincosf((float)positions[r] * inv_freq[d1], &sn, &cs);
      o1 = x1 * cs - x2 * sn;
      o2 = x2 * cs + x1 * sn;
    }
    const bf16 b1 = __float2bfloat16_rn(o1), b2 = __float2bfloat16_rn(o2);
    if (head < heads) {
      bf16* o = q_out + ((size_t)r * heads + head) * hd;
      o[d1] = b1;
      o[d2] = b2;
    } else {
      const bool is_k = head < heads + kvh;
      const int kh = is_k ? head - heads : head - heads - kvh;
      bf16* cache = is_k ? k_cache : v_cache;
      const int slot = slots[r];
      if (slot >= 0) {
        const int page = slot / page_size, off = slot - page * page_size;
        bf16* o = cache + (((size_t)page * kvh + kh) * page_size + off) * hd;
        o[d1] = b1;
        o[d2] = b2;
      }
    }
  }
}

IX_API int ix_qkv_project_rope_applies(int T, int K, int heads, int kvh, int hd, int rot) {
  if (T <= 0 || T > 16 || K <= 0 || K % 8 != 0) return 0;
  if (heads <= 0 || kvh <= 0 || hd <= 0 || hd % 32 != 0) return 0;
  if (rot != 0 && rot != hd) return 0;
  return 1;
}

// x [T, K] bf16; w [(heads + 2 kvh) * hd, K] bf16 (q rows, k rows, v rows); bias fp32 of
// that many entries or null; q_out [T, heads, hd]; caches [pages, kvh, page_size, hd];
// slots [T].
IX_API int ix_qkv_project_rope_append(const void* x, const void* w, const float* bias,
                                      const int* positions, const float* inv_freq, int rot,
                                      const int* slots, void* q_out, void* k_cache,
                                      void* v_cache, int page_size, int T, int K, int heads,
                                      int kvh, int hd, cudaStream_t stream) {
  if (!ix_qkv_project_rope_applies(T, K, heads, kvh, hd, rot)) return IX_ERR_UNSUPPORTED;
  if (!x || !w || !positions || !slots || !q_out || !k_cache || !v_cache || page_size <= 0)
    return IX_ERR_SIZE;
  if (rot > 0 && !inv_freq) return IX_ERR_SIZE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return IX_ERR_ALIGN;
  const long long blocks = (long long)(heads + 2 * kvh) * (hd / 32);
  if (blocks > 0x7fffffffLL) return IX_ERR_SIZE;
  if (T <= 8)
    ix_launch(qkv_project_rope_kernel<1>, dim3((unsigned)blocks), dim3(QP_THREADS), 0, stream,
              (const bf16*)x, (const bf16*)w, bias, positions, inv_freq, rot, slots,
              (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, page_size, T, K, heads, kvh, hd);
  else
    ix_launch(qkv_project_rope_kernel<2>, dim3((unsigned)blocks), dim3(QP_THREADS), 0, stream,
              (const bf16*)x, (const bf16*)w, bias, positions, inv_freq, rot, slots,
              (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, page_size, T, K, heads, kvh, hd);
  return ix_launch_status();
}
