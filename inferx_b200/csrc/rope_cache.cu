// Fused: split the QKV projection row, add the Q/K/V biases, rotate Q and K by
// position (half-split / NeoX pairing over the first `rot` dims of each head),
// write Q densely and write the rotated K and the V into the paged cache.
//
// Reference behaviour, as separate kernels: SplitQkvKernel
// (src/backends/cuda/ops/layers.cu:485-510), RopeKernel (layers.cu:80-115) and
// AppendKvKernel (layers.cu:195-219); rotated keys are what the cache holds
// (src/model/qwen2.cc:928-931).  The angle pos * inv_freq and its sine and
// cosine are computed in fp32 with the accurate sincosf; inv_freq comes from the
// position-encoding part as a table, so a scaled or partial rotary encoding
// needs no other kernel.
//
// Cache layout: [pages, kv_heads, page_size, head_dim]; slot = page * page_size + offset.
#include "common.cuh"
#include "elementwise_vec.cuh"

template <typename TA>
__global__ void qkv_rope_append_kernel(const TA* __restrict__ qkv, const float* __restrict__ bias,
                                       const int* __restrict__ positions,
                                       const float* __restrict__ inv_freq, int rot,
                                       const int* __restrict__ slots, TA* __restrict__ q_out,
                                       TA* __restrict__ k_cache, TA* __restrict__ v_cache,
                                       int page_size, TA* __restrict__ k_out,
                                       TA* __restrict__ v_out, int heads, int kvh, int hd) {
  extern __shared__ float trig[];  // cos[rot/2], sin[rot/2]
  const int t = blockIdx.x;
  const int half = rot >> 1;
  float* cs = trig;
  float* sn = trig + half;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[j], &s, &c);
    cs[j] = c;
    sn[j] = s;
  }
  __syncthreads();

  const int width = (heads + 2 * kvh) * hd;
  const TA* in = qkv + (size_t)t * width;
  const int slot = slots ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot % page_size : 0;

  // Q and K heads: rotated
  const int qk_elems = (heads + kvh) * hd;
  for (int idx = threadIdx.x; idx < qk_elems; idx += blockDim.x) {
    const int head = idx / hd;
    const int d = idx - head * hd;
    const int col = idx;  // q heads then k heads are contiguous in the fused row
    float x = to_f32(in[col]);
    if (bias) x += bias[col];
    float val = x;
    if (d < rot) {
      const int j = d < half ? d : d - half;
      const int pcol = d < half ? col + half : col - half;
      float xp = to_f32(in[pcol]);
      if (bias) xp += bias[pcol];
      val = d < half ? x * cs[j] - xp * sn[j] : x * cs[j] + xp * sn[j];
    }
    const TA v = from_f32<TA>(val);
    if (head < heads) {
      q_out[(size_t)t * heads * hd + idx] = v;
    } else {
      const int kh = head - heads;
      if (k_out) k_out[((size_t)t * kvh + kh) * hd + d] = v;
      if (slot >= 0 && k_cache)
        k_cache[(((size_t)page * kvh + kh) * page_size + off) * hd + d] = v;
    }
  }
  // V heads: bias only
  const int v_elems = kvh * hd;
  const int vbase = (heads + kvh) * hd;
  for (int idx = threadIdx.x; idx < v_elems; idx += blockDim.x) {
    const int kh = idx / hd;
    const int d = idx - kh * hd;
    float x = to_f32(in[vbase + idx]);
    if (bias) x += bias[vbase + idx];
    const TA v = from_f32<TA>(x);
    if (v_out) v_out[(size_t)t * v_elems + idx] = v;
    if (slot >= 0 && v_cache)
      v_cache[(((size_t)page * kvh + kh) * page_size + off) * hd + d] = v;
  }
}

// bf16, head_dim a multiple of 8 and rot a multiple of 16: every thread handles 8
// consecutive dims (one 16-byte chunk) of the first rotary half together with the
// matching chunk of the second half, or one pass-through chunk.  Same arithmetic
// as the scalar kernel.
__global__ void __launch_bounds__(256)
qkv_rope_append_bf16_vec_kernel(const bf16* __restrict__ qkv, const float* __restrict__ bias,
                                const int* __restrict__ positions,
                                const float* __restrict__ inv_freq, int rot,
                                const int* __restrict__ slots, bf16* __restrict__ q_out,
                                bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                int page_size, bf16* __restrict__ k_out, bf16* __restrict__ v_out,
                                int heads, int kvh, int hd) {
  extern __shared__ float trig[];
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int half = rot >> 1;
  float* cs = trig;
  float* sn = trig + half;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[j], &s, &c);
    cs[j] = c;
    sn[j] = s;
  }
  __syncthreads();
  const int width = (heads + 2 * kvh) * hd;
  const bf16* in = qkv + (size_t)t * width;
  const int slot = slots ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot % page_size : 0;
  const int pair_chunks = half >> 3;                 // chunk pairs in the rotary part
  const int pass_chunks = (hd - rot) >> 3;           // chunks that are only biased
  const int per_head = pair_chunks + pass_chunks;
  const int qk_items = (heads + kvh) * per_head;
  const int v_items = kvh * (hd >> 3);

  auto load = [&](int col, float* f) {
    bf8_to_f32(*reinterpret_cast<const uint4*>(in + col), f);
    if (bias) {
      const float4 a = *reinterpret_cast<const float4*>(bias + col);
      const float4 b = *reinterpret_cast<const float4*>(bias + col + 4);
      f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
      f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
    }
  };
  auto store_qk = [&](int head, int d, const float* f) {
    const uint4 v = f32_to_bf8(f);
    if (head < heads) {
      *reinterpret_cast<uint4*>(q_out + ((size_t)t * heads + head) * hd + d) = v;
    } else {
      const int kh = head - heads;
      if (k_out) *reinterpret_cast<uint4*>(k_out + ((size_t)t * kvh + kh) * hd + d) = v;
      if (slot >= 0 && k_cache)
        *reinterpret_cast<uint4*>(k_cache + (((size_t)page * kvh + kh) * page_size + off) * hd +
                                  d) = v;
    }
  };
  for (int idx = threadIdx.x; idx < qk_items + v_items; idx += blockDim.x) {
    if (idx < qk_items) {
      const int head = idx / per_head;
      const int c = idx - head * per_head;
      if (c < pair_chunks) {
        const int d1 = c * 8, d2 = d1 + half;
        float x1[8], x2[8], o1[8], o2[8];
        load(head * hd + d1, x1);
        load(head * hd + d2, x2);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float cc = cs[d1 + j], ss = sn[d1 + j];
          o1[j] = x1[j] * cc - x2[j] * ss;
          o2[j] = x2[j] * cc + x1[j] * ss;
        }
        store_qk(head, d1, o1);
        store_qk(head, d2, o2);
      } else {
        const int d = rot + (c - pair_chunks) * 8;
        float x[8];
        load(head * hd + d, x);
        store_qk(head, d, x);
      }
    } else {
      const int vi = idx - qk_items;
      const int kh = vi / (hd >> 3);
      const int d = (vi - kh * (hd >> 3)) * 8;
      float x[8];
      load((heads + kvh) * hd + kh * hd + d, x);
      const uint4 v = f32_to_bf8(x);
      if (v_out) *reinterpret_cast<uint4*>(v_out + ((size_t)t * kvh + kh) * hd + d) = v;
      if (slot >= 0 && v_cache)
        *reinterpret_cast<uint4*>(v_cache + (((size_t)page * kvh + kh) * page_size + off) * hd +
                                  d) = v;
    }
  }
}

IX_API int ix_qkv_rope_append(const void* qkv, const float* bias, const int* positions,
                              const float* inv_freq, int rot, const int* slots, void* q_out,
                              void* k_cache, void* v_cache, int page_size, void* k_out,
                              void* v_out, int act_dtype, int T, int heads, int kvh, int hd,
                              cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || hd <= 0 || page_size <= 0) return IX_ERR_SIZE;
  if (rot < 0 || rot > hd || (rot & 1)) return IX_ERR_SIZE;
  if (rot > 0 && inv_freq == nullptr) return IX_ERR_SIZE;
  const size_t smem = (size_t)rot * sizeof(float);
  if (smem > 48 * 1024) return IX_ERR_SMEM;
  const uintptr_t all = (uintptr_t)qkv | (uintptr_t)bias | (uintptr_t)q_out | (uintptr_t)k_cache |
                        (uintptr_t)v_cache | (uintptr_t)k_out | (uintptr_t)v_out;
  if (act_dtype == IX_BF16 && hd % 8 == 0 && rot % 16 == 0 && (all & 15) == 0) {
    const int items = (heads + kvh) * (rot / 16 + (hd - rot) / 8) + kvh * (hd / 8);
    const int threads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
    ix_launch(qkv_rope_append_bf16_vec_kernel, dim3(T), dim3(threads), smem, stream,
              (const bf16*)qkv, bias, positions, inv_freq, rot, slots, (bf16*)q_out,
              (bf16*)k_cache, (bf16*)v_cache, page_size, (bf16*)k_out, (bf16*)v_out, heads, kvh,
              hd);
    return ix_launch_status();
  }
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    (qkv_rope_append_kernel<TA><<<T, 256, smem, stream>>>(
                        (const TA*)qkv, bias, positions, inv_freq, rot, slots, (TA*)q_out,
                        (TA*)k_cache, (TA*)v_cache, page_size, (TA*)k_out, (TA*)v_out, heads, kvh,
                        hd)));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// Plain append of dense k, v rows [T, kv_heads, head_dim] into the paged cache
// (the reference's AppendKvKernel, layers.cu:195-219), for mixers whose position
// encoding is applied outside the fused kernel.  A negative slot is skipped.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void append_kv_kernel(const TA* __restrict__ k, const TA* __restrict__ v,
                                 const int* __restrict__ slots, TA* __restrict__ k_cache,
                                 TA* __restrict__ v_cache, int page_size, int kvh, int hd) {
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const int page = slot / page_size, off = slot % page_size;
  for (int idx = threadIdx.x; idx < kvh * hd; idx += blockDim.x) {
    const int kh = idx / hd, d = idx - kh * hd;
    const size_t dst = (((size_t)page * kvh + kh) * page_size + off) * hd + d;
    k_cache[dst] = k[(size_t)t * kvh * hd + idx];
    v_cache[dst] = v[(size_t)t * kvh * hd + idx];
  }
}

IX_API int ix_append_kv(const void* k, const void* v, const int* slots, void* k_cache,
                        void* v_cache, int page_size, int act_dtype, int T, int kvh, int hd,
                        cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (kvh <= 0 || hd <= 0 || page_size <= 0) return IX_ERR_SIZE;
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    (append_kv_kernel<TA><<<T, 256, 0, stream>>>(
                        (const TA*)k, (const TA*)v, slots, (TA*)k_cache, (TA*)v_cache, page_size,
                        kvh, hd)));
  return ix_launch_status();
}
