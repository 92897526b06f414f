// Paged attention for decode steps: every sequence brings one query.
//
// The work is bandwidth: each key and value is read once and used for one dot
// product per query head.  The keys of a sequence are split across thread blocks
// (split-KV), each block streams its range with 16-byte loads kept many deep in
// flight, keeps an online softmax per warp, and writes an unnormalised partial
// (o, max, sum); a second small kernel merges the partials.  Query heads that
// share a KV head are handled by the same block so that the cache is read once
// for the group (GQA packing).  Scores, maxima, sums and the output accumulate
// in fp32; exp is exp2 on scores pre-multiplied by log2(e).
//
// Reference behaviour: FlashInfer's BatchDecodeWithPagedKVCache as the reference
// calls it (src/backends/cuda/ops/flashinfer_attention.cu:340-343), i.e. the same
// result as PagedAttentionKernel (src/backends/cuda/ops/layers.cu:256-318) with
// the window of layers.cu:346-354 for a query at position kv_len - 1.
//
// Sizes: head_dim such that head_dim * sizeof(T) / 16 is a power of two <= 32 and
// instantiated below (64, 128, 256 for bf16; 64, 128 for fp32); other head sizes
// are refused with IX_ERR_UNSUPPORTED and the caller uses the general kernel.
// Scratch: partial outputs [S, heads, splits, head_dim] and (max, sum)
// [S, heads, splits, 2], fp32, provided by the caller.
#include "common.cuh"

#define DEC_THREADS 128
#define DEC_WARPS 4
#define DEC_U 4

template <typename TA> struct Vec16;
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(p[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x);
    f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z);
    f[3] = __uint_as_float(r.w);
  }
};

template <bool FAST> __device__ __forceinline__ float ix_exp2(float x) {
  if (FAST) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  return exp2f(x);
}

template <typename TA, int HD, int G, bool FAST, bool POW2>
__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_split_kernel(const TA* __restrict__ q, const TA* __restrict__ kc,
                         const TA* __restrict__ vc, const int* __restrict__ block_table,
                         const int* __restrict__ kv_len, float* __restrict__ part_o,
                         float* __restrict__ part_ml, TA* __restrict__ out, int heads, int kvh,
                         int page_size, int page_shift, int maxb, int window, float scale_log2e,
                         int splits) {
  constexpr int EPL = Vec16<TA>::N;   // elements per 16-byte load
  constexpr int LPK = HD / EPL;       // lanes that share one key
  constexpr int KPI = 32 / LPK;       // keys per warp per load
  constexpr int KB = KPI * DEC_U;     // keys per warp per iteration
  static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head size not supported");
  __shared__ float sm_acc[G][DEC_WARPS][HD];
  __shared__ float sm_m[G][DEC_WARPS];
  __shared__ float sm_l[G][DEC_WARPS];

  const int split = blockIdx.x, s = blockIdx.z;
  const int rep = heads / kvh;
  const int groups_per_kv = rep / G;
  const int kh = blockIdx.y / groups_per_kv;
  const int h0 = kh * rep + (blockIdx.y % groups_per_kv) * G;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPK, c = lane % LPK;

  const int len = kv_len[s];
  const int start = window > 0 ? max(0, len - window) : 0;
  const int n = len - start;
  int chunk = (n + splits - 1) / splits;
  chunk = (chunk + KB - 1) / KB * KB;
  const int k0 = start + split * chunk;
  const int k1 = min(len, k0 + chunk);
  const int* bt = block_table + (size_t)s * maxb;

  float qreg[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 raw = *reinterpret_cast<const uint4*>(q + ((size_t)s * heads + h0 + g) * HD +
                                                       c * EPL);
    Vec16<TA>::unpack(raw, qreg[g]);
#pragma unroll
    for (int e = 0; e < EPL; ++e) qreg[g][e] *= scale_log2e;
  }
  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }

  for (int kb = k0 + warp * KB; kb < k1; kb += DEC_WARPS * KB) {
    uint4 kraw[DEC_U], vraw[DEC_U];
    bool valid[DEC_U];
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) {
      const int kidx = kb + u * KPI + sub;
      valid[u] = kidx < k1;
      kraw[u] = make_uint4(0, 0, 0, 0);
      vraw[u] = make_uint4(0, 0, 0, 0);
      if (valid[u]) {
        // a runtime integer division costs more than the dot product it feeds
        const int pi = POW2 ? (kidx >> page_shift) : (kidx / page_size);
        const int po = POW2 ? (kidx & (page_size - 1)) : (kidx % page_size);
        const int page = bt[pi];
        const size_t off = (((size_t)page * kvh + kh) * page_size + po) * HD + c * EPL;
        kraw[u] = *reinterpret_cast<const uint4*>(kc + off);
        vraw[u] = *reinterpret_cast<const uint4*>(vc + off);
      }
    }
    float kf[DEC_U][EPL];
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) Vec16<TA>::unpack(kraw[u], kf[u]);
    float sc[G][DEC_U];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int u = 0; u < DEC_U; ++u) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) d += qreg[g][e] * kf[u][e];
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        sc[g][u] = valid[u] ? d : -INFINITY;
      }
    float vf[DEC_U][EPL];
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) Vec16<TA>::unpack(vraw[u], vf[u]);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float m_new = m[g];
#pragma unroll
      for (int u = 0; u < DEC_U; ++u) m_new = fmaxf(m_new, sc[g][u]);
      if (m_new == -INFINITY) continue;
      const float corr = ix_exp2<FAST>(m[g] - m_new);
      float p[DEC_U], psum = 0.f;
#pragma unroll
      for (int u = 0; u < DEC_U; ++u) {
        p[u] = ix_exp2<FAST>(sc[g][u] - m_new);
        psum += p[u];
      }
      l[g] = l[g] * corr + psum;
      m[g] = m_new;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        float a = acc[g][e] * corr;
#pragma unroll
        for (int u = 0; u < DEC_U; ++u) a += p[u] * vf[u][e];
        acc[g][e] = a;
      }
    }
  }

  // merge the key sub-groups of the warp (lanes with the same c)
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int o = 16; o >= LPK; o >>= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], mo);
      const float ca = mn == -INFINITY ? 0.f : ix_exp2<FAST>(m[g] - mn);
      const float cb = mn == -INFINITY ? 0.f : ix_exp2<FAST>(mo - mn);
      l[g] = l[g] * ca + lo * cb;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
        acc[g][e] = acc[g][e] * ca + ao * cb;
      }
      m[g] = mn;
    }
    if (sub == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) sm_acc[g][warp][c * EPL + e] = acc[g][e];
      if (c == 0) {
        sm_m[g][warp] = m[g];
        sm_l[g][warp] = l[g];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += DEC_THREADS) {
    const int g = idx / HD, d = idx - g * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[g][w]);
    float o = 0.f, L = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float cw = ix_exp2<FAST>(sm_m[g][w] - M);
        o += sm_acc[g][w][d] * cw;
        L += sm_l[g][w] * cw;
      }
    }
    const size_t hrow = (size_t)s * heads + h0 + g;
    if (splits == 1) {
      out[hrow * HD + d] = from_f32<TA>(L > 0.f ? o / L : 0.f);
    } else {
      part_o[(hrow * splits + split) * HD + d] = o;
      if (d == 0) {
        part_ml[(hrow * splits + split) * 2] = M;
        part_ml[(hrow * splits + split) * 2 + 1] = L;
      }
    }
  }
}

template <typename TA, bool FAST>
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml, TA* __restrict__ out,
                                         int hd, int splits) {
  const size_t hrow = blockIdx.x;   // s * heads + h
  const float* ml = part_ml + hrow * splits * 2;
  float M = -INFINITY;
  for (int j = 0; j < splits; ++j) M = fmaxf(M, ml[2 * j]);
  float L = 0.f;
  for (int j = 0; j < splits; ++j)
    if (ml[2 * j] != -INFINITY) L += ml[2 * j + 1] * ix_exp2<FAST>(ml[2 * j] - M);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int j = 0; j < splits; ++j)
      if (ml[2 * j] != -INFINITY)
        o += part_o[(hrow * splits + j) * hd + d] * ix_exp2<FAST>(ml[2 * j] - M);
    out[hrow * hd + d] = from_f32<TA>(L > 0.f ? o / L : 0.f);
  }
}

template <typename TA, int HD, bool FAST>
static int launch_decode(const void* q, const void* kc, const void* vc, const int* bt,
                         const int* kv_len, float* part_o, float* part_ml, void* out, int S,
                         int heads, int kvh, int page_size, int maxb, int window, float scale,
                         int splits, cudaStream_t stream) {
  const int rep = heads / kvh;
  const float sl2 = scale * 1.4426950408889634f;
  const int G = rep % 8 == 0 ? 8 : (rep % 4 == 0 ? 4 : (rep % 2 == 0 ? 2 : 1));
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
  dim3 grid(splits, kvh * (rep / G), S);
#define IX_DEC(GG)                                                                              \
  do {                                                                                          \
    if (page_shift >= 0)                                                                        \
      attn_decode_split_kernel<TA, HD, GG, FAST, true><<<grid, DEC_THREADS, 0, stream>>>(        \
          (const TA*)q, (const TA*)kc, (const TA*)vc, bt, kv_len, part_o, part_ml, (TA*)out,    \
          heads, kvh, page_size, page_shift, maxb, window, sl2, splits);                        \
    else                                                                                        \
      attn_decode_split_kernel<TA, HD, GG, FAST, false><<<grid, DEC_THREADS, 0, stream>>>(       \
          (const TA*)q, (const TA*)kc, (const TA*)vc, bt, kv_len, part_o, part_ml, (TA*)out,    \
          heads, kvh, page_size, page_shift, maxb, window, sl2, splits);                        \
  } while (0)
  if (G == 8) IX_DEC(8);
  else if (G == 4) IX_DEC(4);
  else if (G == 2) IX_DEC(2);
  else IX_DEC(1);
#undef IX_DEC
  int rc = ix_launch_status();
  if (rc != 0 || splits == 1) return rc;
  attn_decode_merge_kernel<TA, FAST><<<S * heads, HD >= 128 ? 128 : 64, 0, stream>>>(
      part_o, part_ml, (TA*)out, HD, splits);
  return ix_launch_status();
}

// The number of splits a caller should provide scratch for.
IX_API int ix_attn_decode_splits(int S, int heads, int kvh, int max_kv_len) {
  const int rep = heads / (kvh > 0 ? kvh : 1);
  const int G = rep % 8 == 0 ? 8 : (rep % 4 == 0 ? 4 : (rep % 2 == 0 ? 2 : 1));
  const long long base = (long long)S * kvh * (rep / G);
  const int target = 148 * 6;
  long long splits = (target + base - 1) / base;
  const int max_by_len = (max_kv_len + 255) / 256;
  if (splits > max_by_len) splits = max_by_len;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  return (int)splits;
}

IX_API int ix_paged_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                                     const int* block_table, const int* kv_len, float* part_o,
                                     float* part_ml, void* out, int act_dtype, int S, int heads,
                                     int kvh, int hd, int page_size, int max_blocks, int window,
                                     float scale, int splits, cudaStream_t stream) {
  if (S <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || heads % kvh != 0 || page_size <= 0 || max_blocks <= 0 ||
      window < 0 || splits < 1)
    return IX_ERR_SIZE;
  if (kvh * (heads / kvh) > 65535 || S > 65535) return IX_ERR_SIZE;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return IX_ERR_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return IX_ERR_ALIGN;
#define IX_DEC_HD(TA, HDV, FAST)                                                               \
  return launch_decode<TA, HDV, FAST>(q, k_cache, v_cache, block_table, kv_len, part_o, part_ml, \
                                      out, S, heads, kvh, page_size, max_blocks, window, scale,  \
                                      splits, stream)
  if (act_dtype == IX_BF16) {
    if (hd == 64) IX_DEC_HD(bf16, 64, true);
    if (hd == 128) IX_DEC_HD(bf16, 128, true);
    if (hd == 256) IX_DEC_HD(bf16, 256, true);
    return IX_ERR_UNSUPPORTED;
  }
  if (act_dtype == IX_F32) {
    if (hd == 64) IX_DEC_HD(float, 64, false);
    if (hd == 128) IX_DEC_HD(float, 128, false);
    return IX_ERR_UNSUPPORTED;
  }
#undef IX_DEC_HD
  return IX_ERR_DTYPE;
}
