// Paged causal attention for prompt portions (and any batch that is not all
// single tokens): tensor-core tiles over the paged cache, online softmax.
//
// One block of 4 warps owns 64 consecutive queries of one sequence and one head
// (16 queries per warp).  It walks the keys the tile can see in tiles of 64 keys
// aligned to absolute positions, double-buffered through shared memory with
// cp.async (each key row is fetched from its page with 16-byte copies, so any
// page size works), computes S = Q K^T with mma.sync.m16n8k16 (bf16 in, fp32
// out), applies the causal and window mask by position, keeps the running max and
// sum per query row in fp32 (exp2 on scores pre-scaled by log2 e), and
// accumulates O += P V with P rounded to bf16 as the reference's FlashInfer
// prefill does (src/backends/cuda/ops/flashinfer_prefill.cu:294-343; semantics of
// PagedAttentionWithLseKernel, src/backends/cuda/ops/layers.cu:329-407).  The
// batch is ragged: sequences bring different numbers of queries (cu_q) starting
// at different positions (q_pos0); a sequence with a single query is a tile with
// one valid row.  A query's result depends on its own keys only: tiles are
// aligned to positions, and keys outside its span contribute exact zeros.
//
// Sizes: bf16, head_dim 64 or 128; everything else is refused with
// IX_ERR_UNSUPPORTED and the caller uses the general kernel.
#include "common.cuh"

#define PF_BM 64
#define PF_BN 64
#define PF_THREADS 128

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                            const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2,
                                                  unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
__device__ __forceinline__ void mma16816(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// byte offset of 16-byte chunk `c` of row `r` in a tile with CH chunks per row
template <int CH> __device__ __forceinline__ int swz(int r, int c) {
  return (r * CH + (c ^ (r & 7))) * 16;
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc,
                    const bf16* __restrict__ vc, const int* __restrict__ block_table,
                    const int* __restrict__ cu_q, const int* __restrict__ q_pos0,
                    bf16* __restrict__ out, int S, int heads, int kvh, int page_size,
                    int page_shift, int maxb, int window, float scale_log2e) {
  constexpr int CH = HD / 8;            // 16-byte chunks per row
  constexpr int KS = HD / 16;           // k-steps of Q K^T
  constexpr int DT = HD / 8;            // n-tiles of the output
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Qs = smem;                               // [BM][HD]
  unsigned char* Ks = Qs + PF_BM * HD * 2;                // [2][BN][HD]
  unsigned char* Vs = Ks + 2 * PF_BN * HD * 2;            // [2][BN][HD]

  // which sequence and which 64-query tile of it
  // blocks are handed out in launch order; the tiles with the most keys to walk (the
  // last queries of a sequence) come first, all heads of a tile together, so that the
  // short tiles fill the end of the grid
  int s = 0, tile = gridDim.y - 1 - blockIdx.y;
  {
    bool found = false;
    for (int ss = 0; ss < S; ++ss) {
      const int n = cu_q[ss + 1] - cu_q[ss];
      const int tiles = (n + PF_BM - 1) / PF_BM;
      if (tile < tiles) { s = ss; found = true; break; }
      tile -= tiles;
    }
    if (!found) return;
  }
  const int h = blockIdx.x;
  const int kh = h / (heads / kvh);
  const int tok0 = cu_q[s];
  const int nq = cu_q[s + 1] - tok0;
  const int q0 = tile * PF_BM;
  const int rows_valid = min(PF_BM, nq - q0);
  const int pos0 = q_pos0[s] + q0;               // position of the tile's first query
  const int pmax = pos0 + rows_valid - 1;
  const int kv_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kv_hi = pmax + 1;
  const int kt0 = (kv_lo / PF_BN) * PF_BN;
  const int n_tiles = (kv_hi - kt0 + PF_BN - 1) / PF_BN;
  const int* bt = block_table + (size_t)s * maxb;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  // Q tile -> shared
  for (int idx = tid; idx < PF_BM * CH; idx += PF_THREADS) {
    const int r = idx / CH, c = idx - r * CH;
    const bool ok = r < rows_valid;
    const bf16* src = q + ((size_t)(tok0 + q0 + (ok ? r : 0)) * heads + h) * HD + c * 8;
    cp_async16(Qs + swz<CH>(r, c), src, ok);
  }
  auto load_kv = [&](int it, int stage) {
    const int kbase = kt0 + it * PF_BN;
    unsigned char* kd = Ks + stage * PF_BN * HD * 2;
    unsigned char* vd = Vs + stage * PF_BN * HD * 2;
    for (int idx = tid; idx < PF_BN * CH; idx += PF_THREADS) {
      const int r = idx / CH, c = idx - r * CH;
      const int kp = kbase + r;
      const bool ok = kp >= kv_lo && kp < kv_hi;
      size_t off = 0;
      if (ok) {
        const int pi = page_shift >= 0 ? (kp >> page_shift) : (kp / page_size);
        const int po = page_shift >= 0 ? (kp & (page_size - 1)) : (kp % page_size);
        off = (((size_t)bt[pi] * kvh + kh) * page_size + po) * HD + c * 8;
      }
      cp_async16(kd + swz<CH>(r, c), kc + off, ok);
      cp_async16(vd + swz<CH>(r, c), vc + off, ok);
    }
  };
  load_kv(0, 0);
  cp_async_commit();

  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  unsigned qf[KS][4];
  const int row_a = warp * 16 + g, row_b = row_a + 8;     // this thread's two query rows
  const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_tiles) load_kv(it + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = kk * 2 + (lane >> 4);
        ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], Qs + swz<CH>(r, c));
      }
    }
    const unsigned char* kt = Ks + stage * PF_BN * HD * 2;
    const unsigned char* vt = Vs + stage * PF_BN * HD * 2;
    const int kbase = kt0 + it * PF_BN;

    float sc[PF_BN / 8][4];
#pragma unroll
    for (int j = 0; j < PF_BN / 8; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) sc[j][c] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
      for (int j = 0; j < PF_BN / 8; j += 2) {
        unsigned b0, b1, b2, b3;
        const int r = (j + (lane >> 4)) * 8 + (lane & 7);
        const int c = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b0, b1, b2, b3, kt + swz<CH>(r, c));
        mma16816(sc[j], qf[kk], b0, b1);
        mma16816(sc[j + 1], qf[kk], b2, b3);
      }
    }
    // scale, mask by position, row max
    const bool need_mask = (kbase + PF_BN - 1 > pos0) || (window > 0 && kbase < pmax - window + 1)
                           || kbase < kv_lo;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < PF_BN / 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v = sc[j][c] * scale_log2e;
        if (need_mask) {
          const int kp = kbase + j * 8 + 2 * t + (c & 1);
          const int pos = (c & 2) ? pos_b : pos_a;
          const bool vis = kp <= pos && (window <= 0 || kp >= pos - window + 1);
          if (!vis) v = -INFINITY;
        }
        sc[j][c] = v;
        mx[c >> 1] = fmaxf(mx[c >> 1], v);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = fast_exp2(m_run[r] - m_use[r]);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int j = 0; j < DT; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
    unsigned pf[PF_BN / 16][4];
#pragma unroll
    for (int j = 0; j < PF_BN / 8; ++j) {
      const float p0 = fast_exp2(sc[j][0] - m_use[0]);
      const float p1 = fast_exp2(sc[j][1] - m_use[0]);
      const float p2 = fast_exp2(sc[j][2] - m_use[1]);
      const float p3 = fast_exp2(sc[j][3] - m_use[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < PF_BN / 16; ++kk) {
#pragma unroll
      for (int jd = 0; jd < DT; jd += 2) {
        unsigned b0, b1, b2, b3;
        const int r = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int c = jd + (lane >> 4);
        ldmatrix_x4_trans(b0, b1, b2, b3, vt + swz<CH>(r, c));
        mma16816(o[jd], pf[kk], b0, b1);
        mma16816(o[jd + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads();   // everyone is done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // finish the row sums across the quad and write
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv_a = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
  const float inv_b = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
#pragma unroll
  for (int j = 0; j < DT; ++j) {
    const int d = j * 8 + 2 * t;
    if (row_a < rows_valid) {
      bf16* dst = out + ((size_t)(tok0 + q0 + row_a) * heads + h) * HD + d;
      *reinterpret_cast<unsigned*>(dst) = pack_bf16(o[j][0] * inv_a, o[j][1] * inv_a);
    }
    if (row_b < rows_valid) {
      bf16* dst = out + ((size_t)(tok0 + q0 + row_b) * heads + h) * HD + d;
      *reinterpret_cast<unsigned*>(dst) = pack_bf16(o[j][2] * inv_b, o[j][3] * inv_b);
    }
  }
}

template <int HD>
static int launch_prefill(const void* q, const void* kc, const void* vc, const int* bt,
                          const int* cu_q, const int* q_pos0, void* out, int T, int S, int heads,
                          int kvh, int page_size, int maxb, int window, float scale,
                          cudaStream_t stream) {
  const size_t smem = (size_t)(PF_BM + 4 * PF_BN) * HD * 2;
  auto kern = attn_prefill_kernel<HD>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int tiles = (T + PF_BM - 1) / PF_BM + S;   // every sequence can add one partial tile
  if (tiles > 65535) return IX_ERR_SIZE;
  dim3 grid(heads, tiles);
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
  kern<<<grid, PF_THREADS, smem, stream>>>((const bf16*)q, (const bf16*)kc, (const bf16*)vc, bt,
                                           cu_q, q_pos0, (bf16*)out, S, heads, kvh, page_size,
                                           page_shift, maxb, window,
                                           scale * 1.4426950408889634f);
  return ix_launch_status();
}

IX_API int ix_paged_attention_prefill(const void* q, const void* k_cache, const void* v_cache,
                                      const int* block_table, const int* cu_q, const int* q_pos0,
                                      void* out, int act_dtype, int T, int S, int heads, int kvh,
                                      int hd, int page_size, int max_blocks, int window,
                                      float scale, cudaStream_t stream) {
  if (T <= 0 || S <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || heads % kvh != 0 || page_size <= 0 || max_blocks <= 0 ||
      window < 0)
    return IX_ERR_SIZE;
  if (act_dtype != IX_BF16) return IX_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15)
    return IX_ERR_ALIGN;
  if (hd == 128)
    return launch_prefill<128>(q, k_cache, v_cache, block_table, cu_q, q_pos0, out, T, S, heads,
                               kvh, page_size, max_blocks, window, scale, stream);
  if (hd == 64)
    return launch_prefill<64>(q, k_cache, v_cache, block_table, cu_q, q_pos0, out, T, S, heads,
                              kvh, page_size, max_blocks, window, scale, stream);
  return IX_ERR_UNSUPPORTED;
}
