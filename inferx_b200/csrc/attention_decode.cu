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
  IX_PDL_WAIT();
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

// ---------------------------------------------------------------------------
// Tensor-core form of the split kernel (bf16, head_dim 64 or 128).  The scalar
// kernel above spends several instructions per byte on unpacking and shuffles and
// cannot keep up with HBM; here a block's four warps share 64-key tiles that
// cp.async streams through a three-stage ring in shared memory, each warp takes 16
// keys of the tile, computes S = Q K^T and O += P V with mma.sync.m16n8k16 (the up
// to 16 query heads of the KV head are the M side) and keeps its own online
// softmax; the warps' partials are merged through shared memory at the end.
// Same scratch layout and merge kernel as the scalar form.
// ---------------------------------------------------------------------------
#define DM_BN 64
#define DM_STAGES 2

__device__ __forceinline__ void dm_cp16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void dm_ldsm(unsigned* r, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void dm_ldsm_t(unsigned* r, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void dm_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <int CH> __device__ __forceinline__ int dm_swz(int r, int c) {
  return (r * CH + (c ^ (r & 7))) * 16;
}

template <int HD, bool POW2>
__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc,
                       const bf16* __restrict__ vc, const int* __restrict__ block_table,
                       const int* __restrict__ kv_len, float* __restrict__ part_o,
                       float* __restrict__ part_ml, bf16* __restrict__ out, int heads, int kvh,
                       int page_size, int page_shift, int maxb, int window, float scale_log2e,
                       int splits) {
  constexpr int CH = HD / 8, KS = HD / 16, DT = HD / 8;
  constexpr int TILE_BYTES = DM_BN * HD * 2;
  extern __shared__ __align__(128) unsigned char dsm[];
  unsigned char* Qs = dsm;                                   // [16][HD]
  unsigned char* Ks = Qs + 16 * HD * 2;                      // [STAGES][64][HD]
  unsigned char* Vs = Ks + DM_STAGES * TILE_BYTES;           // [STAGES][64][HD]
  __shared__ float sm_m[DEC_WARPS][16];
  __shared__ float sm_l[DEC_WARPS][16];
  IX_PDL_WAIT();

  const int split = blockIdx.x, s = blockIdx.z;
  const int rep = heads / kvh;
  const int row_groups = (rep + 15) / 16;
  const int kh = blockIdx.y / row_groups;
  const int qrow0 = (blockIdx.y % row_groups) * 16;
  const int rows_valid = min(16, rep - qrow0);
  const int h0 = kh * rep + qrow0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  const int len = kv_len[s];
  const int start = window > 0 ? max(0, len - window) : 0;
  const int n = len - start;
  int chunk = (n + splits - 1) / splits;
  chunk = (chunk + DM_BN - 1) / DM_BN * DM_BN;
  const int k0 = start + split * chunk;
  const int k1 = min(len, k0 + chunk);
  const int n_tiles = k1 > k0 ? (k1 - k0 + DM_BN - 1) / DM_BN : 0;
  const int* bt = block_table + (size_t)s * maxb;

  for (int idx = tid; idx < 16 * CH; idx += DEC_THREADS) {
    const int r = idx / CH, c = idx - r * CH;
    const bool ok = r < rows_valid;
    dm_cp16(Qs + dm_swz<CH>(r, c), q + ((size_t)s * heads + h0 + (ok ? r : 0)) * HD + c * 8, ok);
  }
  auto load_kv = [&](int it) {
    if (it < n_tiles) {
      const int stage = it % DM_STAGES;
      const int kbase = k0 + it * DM_BN;
      unsigned char* kd = Ks + stage * TILE_BYTES;
      unsigned char* vd = Vs + stage * TILE_BYTES;
      for (int idx = tid; idx < DM_BN * CH; idx += DEC_THREADS) {
        const int r = idx / CH, c = idx - r * CH;
        const int kp = kbase + r;
        const bool ok = kp < k1;
        size_t off = 0;
        if (ok) {
          const int pi = POW2 ? (kp >> page_shift) : (kp / page_size);
          const int po = POW2 ? (kp & (page_size - 1)) : (kp % page_size);
          off = (((size_t)bt[pi] * kvh + kh) * page_size + po) * HD + c * 8;
        }
        dm_cp16(kd + dm_swz<CH>(r, c), kc + off, ok);
        dm_cp16(vd + dm_swz<CH>(r, c), vc + off, ok);
      }
    }
    asm volatile("cp.async.commit_group;");
  };
  load_kv(0);

  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  unsigned qf[KS][4];

  for (int it = 0; it < n_tiles; ++it) {
    load_kv(it + 1);
    asm volatile("cp.async.wait_group 1;");
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < KS; ++kk)
        dm_ldsm(qf[kk], Qs + dm_swz<CH>((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));
    }
    const int stage = it % DM_STAGES;
    const unsigned char* kt = Ks + stage * TILE_BYTES;
    const unsigned char* vt = Vs + stage * TILE_BYTES;
    const int kw = k0 + it * DM_BN + warp * 16;      // first key of this warp's 16
    if (kw < k1) {
      float sc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[j][c] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
        unsigned b[4];
        dm_ldsm(b, kt + dm_swz<CH>(warp * 16 + (lane >> 4) * 8 + (lane & 7),
                                   kk * 2 + ((lane >> 3) & 1)));
        dm_mma(sc[0], qf[kk], b[0], b[1]);
        dm_mma(sc[1], qf[kk], b[2], b[3]);
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int kp = kw + j * 8 + 2 * t + (c & 1);
          const float v = kp < k1 ? sc[j][c] * scale_log2e : -INFINITY;
          sc[j][c] = v;
          mx[c >> 1] = fmaxf(mx[c >> 1], v);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;
        corr[r] = ix_exp2<true>(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= corr[r];
      }
#pragma unroll
      for (int j = 0; j < DT; ++j) {
        o[j][0] *= corr[0]; o[j][1] *= corr[0];
        o[j][2] *= corr[1]; o[j][3] *= corr[1];
      }
      unsigned pf[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = ix_exp2<true>(sc[j][0] - m_use[0]);
        const float p1 = ix_exp2<true>(sc[j][1] - m_use[0]);
        const float p2 = ix_exp2<true>(sc[j][2] - m_use[1]);
        const float p3 = ix_exp2<true>(sc[j][3] - m_use[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi = __floats2bfloat162_rn(p2, p3);
        pf[j * 2 + 0] = *reinterpret_cast<unsigned*>(&lo);
        pf[j * 2 + 1] = *reinterpret_cast<unsigned*>(&hi);
      }
#pragma unroll
      for (int jd = 0; jd < DT; jd += 2) {
        unsigned b[4];
        dm_ldsm_t(b, vt + dm_swz<CH>(warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7),
                                     jd + (lane >> 4)));
        dm_mma(o[jd], pf, b[0], b[1]);
        dm_mma(o[jd + 1], pf, b[2], b[3]);
      }
    }
    __syncthreads();   // the stage may be refilled
  }
  asm volatile("cp.async.wait_group 0;");
  __syncthreads();

  // merge the four warps (each saw different keys); stage memory is free now
  float* sm_o = reinterpret_cast<float*>(Ks);     // [DEC_WARPS][16][HD]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  if (t == 0) {
    sm_m[warp][g] = m_run[0];     sm_l[warp][g] = l_run[0];
    sm_m[warp][g + 8] = m_run[1]; sm_l[warp][g + 8] = l_run[1];
  }
#pragma unroll
  for (int j = 0; j < DT; ++j) {
    const int d = j * 8 + 2 * t;
    sm_o[(warp * 16 + g) * HD + d] = o[j][0];
    sm_o[(warp * 16 + g) * HD + d + 1] = o[j][1];
    sm_o[(warp * 16 + g + 8) * HD + d] = o[j][2];
    sm_o[(warp * 16 + g + 8) * HD + d + 1] = o[j][3];
  }
  __syncthreads();
  for (int idx = tid; idx < rows_valid * HD; idx += DEC_THREADS) {
    const int r = idx / HD, d = idx - r * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][r]);
    float ov = 0.f, L = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float cw = ix_exp2<true>(sm_m[w][r] - M);   // exp2(-inf) = 0 for idle warps
        ov += sm_o[(w * 16 + r) * HD + d] * cw;
        L += sm_l[w][r] * cw;
      }
    }
    const size_t hrow = (size_t)s * heads + h0 + r;
    if (splits == 1) {
      out[hrow * HD + d] = __float2bfloat16_rn(L > 0.f ? ov / L : 0.f);
    } else {
      part_o[(hrow * splits + split) * HD + d] = ov;
      if (d == 0) {
        part_ml[(hrow * splits + split) * 2] = M;
        part_ml[(hrow * splits + split) * 2 + 1] = L;
      }
    }
  }
}

template <int HD>
static int launch_decode_mma(const void* q, const void* kc, const void* vc, const int* bt,
                             const int* kv_len, float* part_o, float* part_ml, void* out, int S,
                             int heads, int kvh, int page_size, int maxb, int window, float scale,
                             int splits, cudaStream_t stream) {
  const int rep = heads / kvh;
  const float sl2 = scale * 1.4426950408889634f;
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {}
  const int smem = 16 * HD * 2 + 2 * DM_STAGES * DM_BN * HD * 2;
  dim3 grid(splits, kvh * ((rep + 15) / 16), S);
  cudaError_t e;
  if (page_shift >= 0) {
    auto kern = attn_decode_mma_kernel<HD, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    ix_launch(kern, grid, dim3(DEC_THREADS), smem, stream, (const bf16*)q, (const bf16*)kc,
              (const bf16*)vc, bt, kv_len, part_o, part_ml, (bf16*)out, heads, kvh, page_size,
              page_shift, maxb, window, sl2, splits);
  } else {
    auto kern = attn_decode_mma_kernel<HD, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    ix_launch(kern, grid, dim3(DEC_THREADS), smem, stream, (const bf16*)q, (const bf16*)kc,
              (const bf16*)vc, bt, kv_len, part_o, part_ml, (bf16*)out, heads, kvh, page_size,
              page_shift, maxb, window, sl2, splits);
  }
  int rc = ix_launch_status();
  if (rc != 0 || splits == 1) return rc;
  ix_launch(attn_decode_merge_kernel<bf16, true>, dim3(S * heads), dim3(HD >= 128 ? 128 : 64), 0,
            stream, (const float*)part_o, (const float*)part_ml, (bf16*)out, HD, splits);
  return ix_launch_status();
}

// One wave: with `per_sm` blocks resident on each of the 148 SMs, aim for at most
// 148 * per_sm blocks and let each of them walk a long range of keys; a grid a little
// larger than a wave would leave most SMs idle during its last wave.
static int decode_splits(int S, int heads, int kvh, int max_kv_len, int per_sm) {
  const int rep = heads / (kvh > 0 ? kvh : 1);
  const long long base = (long long)S * kvh * ((rep + 15) / 16);
  const int slots = 148 * per_sm;
  const int max_by_len = (max_kv_len + 127) / 128;   // at least two 64-key tiles per block
  long long splits;
  if (base < slots) {
    splits = slots / base;
  } else {
    // More blocks than one wave holds.  A last wave that fills at least half of the
    // places still saturates the memory system and simply ends sooner; a thinner one
    // runs as long as a half-full one would (320 blocks on 296 places: the last 24 cost
    // as much as 148).  Splitting the keys a few ways evens that out and pays for the
    // merge it adds: take the count, up to four, with the least such waste, charging two
    // per cent for each extra split.
    splits = 1;
    double best = 0.0;
    for (int s = 1; s <= 4; ++s) {
      const long long blocks = base * s;
      const long long full = blocks / slots;
      const double rest = (double)(blocks - full * slots) / (double)slots;
      const double ideal = (double)full + rest;
      const double cost = (double)full + (rest > 0.0 ? (rest < 0.5 ? 0.5 : rest) : 0.0);
      const double score = ideal / cost * (1.0 - 0.02 * (s - 1));
      if (score > best + 1e-9) {
        best = score;
        splits = s;
      }
    }
  }
  if (splits > max_by_len) splits = max_by_len;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  return (int)splits;
}

// The number of splits a caller should provide scratch for: the cp.async-fed and
// scalar kernels (three blocks per SM) and the TMA-fed kernel (two, with a deeper ring).
IX_API int ix_attn_decode_splits(int S, int heads, int kvh, int max_kv_len) {
  return decode_splits(S, heads, kvh, max_kv_len, 3);
}
IX_API int ix_attn_decode_tma_splits(int S, int heads, int kvh, int max_kv_len) {
  return decode_splits(S, heads, kvh, max_kv_len, 2);
}

// variant 0: the tensor-core kernel where it applies (bf16, head_dim 64/128), else the
// scalar kernel; variant 1: always the scalar kernel.
static int decode_dispatch(const void* q, const void* k_cache, const void* v_cache,
                           const int* block_table, const int* kv_len, float* part_o,
                           float* part_ml, void* out, int act_dtype, int S, int heads, int kvh,
                           int hd, int page_size, int max_blocks, int window, float scale,
                           int splits, int variant, cudaStream_t stream) {
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
  if (act_dtype == IX_BF16 && variant == 0 && (hd == 64 || hd == 128)) {
    if (hd == 128)
      return launch_decode_mma<128>(q, k_cache, v_cache, block_table, kv_len, part_o, part_ml, out,
                                    S, heads, kvh, page_size, max_blocks, window, scale, splits,
                                    stream);
    return launch_decode_mma<64>(q, k_cache, v_cache, block_table, kv_len, part_o, part_ml, out, S,
                                 heads, kvh, page_size, max_blocks, window, scale, splits, stream);
  }
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

IX_API int ix_paged_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                                     const int* block_table, const int* kv_len, float* part_o,
                                     float* part_ml, void* out, int act_dtype, int S, int heads,
                                     int kvh, int hd, int page_size, int max_blocks, int window,
                                     float scale, int splits, cudaStream_t stream) {
  return decode_dispatch(q, k_cache, v_cache, block_table, kv_len, part_o, part_ml, out, act_dtype,
                         S, heads, kvh, hd, page_size, max_blocks, window, scale, splits, 0, stream);
}

IX_API int ix_paged_attention_decode_scalar(const void* q, const void* k_cache,
                                            const void* v_cache, const int* block_table,
                                            const int* kv_len, float* part_o, float* part_ml,
                                            void* out, int act_dtype, int S, int heads, int kvh,
                                            int hd, int page_size, int max_blocks, int window,
                                            float scale, int splits, cudaStream_t stream) {
  return decode_dispatch(q, k_cache, v_cache, block_table, kv_len, part_o, part_ml, out, act_dtype,
                         S, heads, kvh, hd, page_size, max_blocks, window, scale, splits, 1, stream);
}

// The TMA-fed form (attention_decode_tma.cu) followed by the same merge.  bf16,
// head_dim 64/128, page_size a power of two from 8 to 64; num_pages is the first
// extent of the cache tensors.
extern "C" int ix_attn_decode_tma_applies(int hd, int page_size);
extern "C" int ix_attn_decode_tma_partials(const void* q, const void* kc, const void* vc,
                                           int num_pages, const int* bt, const int* kv_len,
                                           float* part_o, float* part_ml, void* out, int S,
                                           int heads, int kvh, int hd, int page_size, int maxb,
                                           int window, float scale, int splits, int* status,
                                           cudaStream_t stream);

IX_API int ix_paged_attention_decode_tma(const void* q, const void* k_cache, const void* v_cache,
                                         int num_pages, const int* block_table,
                                         const int* kv_len, float* part_o, float* part_ml,
                                         void* out, int S, int heads, int kvh, int hd,
                                         int page_size, int max_blocks, int window, float scale,
                                         int splits, int* status, cudaStream_t stream) {
  if (S <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || heads % kvh != 0 || max_blocks <= 0 || window < 0 || splits < 1)
    return IX_ERR_SIZE;
  if (kvh * ((heads / kvh + 15) / 16) > 65535 || S > 65535) return IX_ERR_SIZE;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return IX_ERR_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return IX_ERR_ALIGN;
  if (!ix_attn_decode_tma_applies(hd, page_size)) return IX_ERR_UNSUPPORTED;
  int rc = ix_attn_decode_tma_partials(q, k_cache, v_cache, num_pages, block_table, kv_len, part_o,
                                       part_ml, out, S, heads, kvh, hd, page_size, max_blocks,
                                       window, scale, splits, status, stream);
  if (rc != 0 || splits == 1) return rc;
  ix_launch(attn_decode_merge_kernel<bf16, true>, dim3(S * heads), dim3(hd >= 128 ? 128 : 64), 0,
            stream, (const float*)part_o, (const float*)part_ml, (bf16*)out, hd, splits);
  return ix_launch_status();
}
