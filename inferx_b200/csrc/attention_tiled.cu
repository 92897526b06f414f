// Paged causal attention on the CUDA cores, tiled: 32 queries of one (sequence, head)
// against tiles of 64 keys held in shared memory, fp32 arithmetic throughout with the
// accurate expf.  The prompt-sized counterpart of attention_generic.cu (one block per
// (token, head), which re-reads every key for every query): the attention of the
// 32-bit path for prompt portions, and of the bfloat16 path for head sizes the
// tensor-core kernels do not take.  Reference behaviour as in attention_generic.cu
// (src/backends/cuda/ops/layers.cu:256-318, 329-407): a query at position p sees keys
// max(0, p - window + 1) .. p, score = (q . k) * scale, softmax with max subtraction,
// kv head = head / group.
//
// Key tiles start at multiples of 64 of the absolute position, and a query's running
// maximum and sum are updated once per tile, so what a query computes does not depend
// on how its sequence was cut into portions or on what else is in the batch.
//
// Takes any element type, head sizes that are a multiple of 4 up to 256, any page size.
#include "common.cuh"

#define TA_BQ 32
#define TA_BK 64
#define TA_THREADS 256

template <typename TA> struct TaLoad4;
template <> struct TaLoad4<float> {
  static __device__ __forceinline__ float4 load(const float* p) {
    return *reinterpret_cast<const float4*>(p);
  }
  static __device__ __forceinline__ void store(float* p, float4 v) {
    *reinterpret_cast<float4*>(p) = v;
  }
};
template <> struct TaLoad4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    uint2 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
    h[0] = __floats2bfloat162_rn(v.x, v.y);
    h[1] = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

template <typename TA>
__global__ void __launch_bounds__(TA_THREADS)
paged_attention_tiled_kernel(const TA* __restrict__ q, const TA* __restrict__ kc,
                             const TA* __restrict__ vc, const int* __restrict__ block_table,
                             const int* __restrict__ cu_q, const int* __restrict__ q_pos0,
                             TA* __restrict__ out, int S, int heads, int kvh, int hd,
                             int page_size, int max_blocks, int window, float scale) {
  extern __shared__ __align__(16) float tsm[];
  const int ld = hd + 4;                         // row pitch: 16-byte rows, no bank conflicts
  float* Qs = tsm;                               // [TA_BQ][ld]
  float* Ks = Qs + TA_BQ * ld;                   // [TA_BK][ld]
  float* Vs = Ks + TA_BK * ld;                   // [TA_BK][ld]
  float* Ps = Vs + TA_BK * ld;                   // [TA_BQ][TA_BK + 4]
  float* m_run = Ps + TA_BQ * (TA_BK + 4);       // [TA_BQ]
  float* l_run = m_run + TA_BQ;
  float* corr = l_run + TA_BQ;

  // which sequence and which 32-query tile of it
  int s = -1, tile = blockIdx.y;
  for (int ss = 0; ss < S; ++ss) {
    const int tiles = (cu_q[ss + 1] - cu_q[ss] + TA_BQ - 1) / TA_BQ;
    if (tile < tiles) { s = ss; break; }
    tile -= tiles;
  }
  if (s < 0) return;
  const int h = blockIdx.x;
  const int kh = h / (heads / kvh);
  const int tok0 = cu_q[s] + tile * TA_BQ;
  const int rows_valid = min(TA_BQ, cu_q[s + 1] - tok0);
  const int pos0 = q_pos0[s] + tile * TA_BQ;     // position of the tile's first query
  const int kv_hi = pos0 + rows_valid;           // one past the last visible key
  const int kv_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int* bt = block_table + (size_t)s * max_blocks;
  const int tid = threadIdx.x;
  const int chunks = hd >> 2;

  for (int idx = tid; idx < TA_BQ * chunks; idx += TA_THREADS) {
    const int r = idx / chunks, c = idx - r * chunks;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows_valid) v = TaLoad4<TA>::load(q + ((size_t)(tok0 + r) * heads + h) * hd + 4 * c);
    *reinterpret_cast<float4*>(Qs + r * ld + 4 * c) = v;
  }
  if (tid < TA_BQ) {
    m_run[tid] = -INFINITY;
    l_run[tid] = 0.f;
  }

  // scores: thread (sq, sk) of 16 x 16 owns queries sq, sq + 16 and keys sk + 16 j
  const int sq = tid >> 4, sk = tid & 15;
  // output: warp w owns queries 4 w .. 4 w + 3, lane l the dimensions 4 l + 128 j
  const int ow = tid >> 5, ol = tid & 31;
  float acc[4][2][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;

  for (int kv0 = kv_lo & ~(TA_BK - 1); kv0 < kv_hi; kv0 += TA_BK) {
    __syncthreads();                             // the previous tile has been used
    for (int idx = tid; idx < TA_BK * chunks; idx += TA_THREADS) {
      const int r = idx / chunks, c = idx - r * chunks;
      const int kp = kv0 + r;
      float4 kv4 = make_float4(0.f, 0.f, 0.f, 0.f), vv4 = kv4;
      if (kp >= kv_lo && kp < kv_hi) {
        const int page = bt[kp / page_size];
        if (page >= 0) {
          const size_t row = (((size_t)page * kvh + kh) * page_size + kp % page_size) * hd;
          kv4 = TaLoad4<TA>::load(kc + row + 4 * c);
          vv4 = TaLoad4<TA>::load(vc + row + 4 * c);
        }
      }
      *reinterpret_cast<float4*>(Ks + r * ld + 4 * c) = kv4;
      *reinterpret_cast<float4*>(Vs + r * ld + 4 * c) = vv4;
    }
    __syncthreads();

    float sc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
    for (int c = 0; c < chunks; ++c) {
      float4 qa[2], kb[4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        qa[i] = *reinterpret_cast<const float4*>(Qs + (sq + 16 * i) * ld + 4 * c);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        kb[j] = *reinterpret_cast<const float4*>(Ks + (sk + 16 * j) * ld + 4 * c);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sc[i][j] = fmaf(qa[i].x, kb[j].x, sc[i][j]);
          sc[i][j] = fmaf(qa[i].y, kb[j].y, sc[i][j]);
          sc[i][j] = fmaf(qa[i].z, kb[j].z, sc[i][j]);
          sc[i][j] = fmaf(qa[i].w, kb[j].w, sc[i][j]);
        }
    }
    // mask, running maximum, probabilities
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = sq + 16 * i;
      const int qp = pos0 + r;
      const int first = window > 0 ? max(0, qp - window + 1) : 0;
      float tm = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kp = kv0 + sk + 16 * j;
        const bool seen = r < rows_valid && kp <= qp && kp >= first;
        sc[i][j] = seen ? sc[i][j] * scale : -INFINITY;
        tm = fmaxf(tm, sc[i][j]);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
      const float m_old = m_run[r];
      const float m_new = fmaxf(m_old, tm);
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = m_new == -INFINITY ? 0.f : expf(sc[i][j] - m_new);
        Ps[r * (TA_BK + 4) + sk + 16 * j] = p;
        psum += p;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
      __syncwarp();
      if (sk == 0) {
        const float cr = m_new == -INFINITY ? 1.f : expf(m_old - m_new);   // 0 at the first tile
        corr[r] = cr;
        l_run[r] = l_run[r] * cr + psum;
        m_run[r] = m_new;
      }
    }
    __syncthreads();

    // O = O * corr + P V
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float cr = corr[4 * ow + i];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][j][c] *= cr;
    }
    for (int k = 0; k < TA_BK; ++k) {
      float p[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) p[i] = Ps[(4 * ow + i) * (TA_BK + 4) + k];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int d = 4 * ol + 128 * j;
        if (d < hd) {
          const float4 v4 = *reinterpret_cast<const float4*>(Vs + k * ld + d);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[i][j][0] = fmaf(p[i], v4.x, acc[i][j][0]);
            acc[i][j][1] = fmaf(p[i], v4.y, acc[i][j][1]);
            acc[i][j][2] = fmaf(p[i], v4.z, acc[i][j][2]);
            acc[i][j][3] = fmaf(p[i], v4.w, acc[i][j][3]);
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 4 * ow + i;
    if (r >= rows_valid) continue;
    const float inv_l = 1.0f / l_run[r];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int d = 4 * ol + 128 * j;
      if (d < hd)
        TaLoad4<TA>::store(out + ((size_t)(tok0 + r) * heads + h) * hd + d,
                           make_float4(acc[i][j][0] * inv_l, acc[i][j][1] * inv_l,
                                       acc[i][j][2] * inv_l, acc[i][j][3] * inv_l));
    }
  }
}

IX_API int ix_paged_attention_tiled_applies(int hd) { return hd > 0 && hd % 4 == 0 && hd <= 256; }

// q, out: [T, heads, hd]; caches [pages, kvh, page_size, hd]; block_table [S, max_blocks];
// cu_q [S + 1]: token range of each sequence; q_pos0 [S]: position of its first token here.
IX_API int ix_paged_attention_tiled(const void* q, const void* k_cache, const void* v_cache,
                                    const int* block_table, const int* cu_q, const int* q_pos0,
                                    void* out, int act_dtype, int T, int S, int heads, int kvh,
                                    int hd, int page_size, int max_blocks, int window,
                                    float scale, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (S <= 0 || heads <= 0 || kvh <= 0 || heads % kvh != 0 || page_size <= 0 || max_blocks <= 0 ||
      window < 0)
    return IX_ERR_SIZE;
  if (!ix_paged_attention_tiled_applies(hd)) return IX_ERR_UNSUPPORTED;
  if ((T + TA_BQ - 1) / TA_BQ + S > 65535) return IX_ERR_SIZE;
  const int esize = act_dtype == IX_F32 ? 4 : 2;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % (4 * esize))
    return IX_ERR_ALIGN;
  const int ld = hd + 4;
  const size_t smem = ((size_t)(TA_BQ + 2 * TA_BK) * ld + TA_BQ * (TA_BK + 4) + 3 * TA_BQ) * 4;
  dim3 grid(heads, (T + TA_BQ - 1) / TA_BQ + S);   // every sequence can add a partial tile
  IX_DISPATCH_DTYPE(act_dtype, TA, {
    auto kern = paged_attention_tiled_kernel<TA>;
    if (smem > 48 * 1024) {
      cudaError_t e =
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kern<<<grid, TA_THREADS, smem, stream>>>((const TA*)q, (const TA*)k_cache, (const TA*)v_cache,
                                             block_table, cu_q, q_pos0, (TA*)out, S, heads, kvh,
                                             hd, page_size, max_blocks, window, scale);
  });
  return ix_launch_status();
}
