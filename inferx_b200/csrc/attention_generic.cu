// Paged causal attention with grouped KV heads and an optional sliding window,
// for any mix of prompt portions and single decoded tokens in one launch.
// This is the general kernel: any head size up to 512, any element type, fp32
// arithmetic throughout with the accurate expf.  It is the whole attention of
// the 32-bit path and the fallback of the bfloat16 path for shapes the tuned
// kernels refuse.
//
// Reference behaviour: PagedAttentionKernel / PagedAttentionWithLseKernel
// (src/backends/cuda/ops/layers.cu:256-318, 329-407): query at position p of a
// sequence sees keys max(0, p-window+1)..p (all of 0..p without a window),
// score = (q.k) * scale, softmax with max subtraction, kv head = head / group.
// Unlike the reference there is no cap on the number of keys: scores are
// consumed in tiles of 128 keys with an online softmax.  One block owns one
// (token, head); its arithmetic depends only on that token's own keys, never on
// what else is in the batch or on which pages hold the keys.
#include "common.cuh"

#define ATT_TILE 128
#define ATT_THREADS 128
#define ATT_MAX_DPT 4  // dims per thread: head_dim <= ATT_THREADS * ATT_MAX_DPT

template <typename TA>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_generic_kernel(const TA* __restrict__ q, const TA* __restrict__ kc,
                               const TA* __restrict__ vc, const int* __restrict__ block_table,
                               const int* __restrict__ seq_of_token,
                               const int* __restrict__ positions, TA* __restrict__ out, int heads,
                               int kvh, int hd, int page_size, int max_blocks, int window,
                               float scale) {
  extern __shared__ float smem[];
  float* qs = smem;        // [hd]
  float* sc = smem + hd;   // [ATT_TILE]
  const int t = blockIdx.x;
  const int h = blockIdx.y;
  const int s = seq_of_token[t];
  const int pos = positions[t];
  const int kh = h / (heads / kvh);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = ATT_THREADS / 32;
  const int* bt = block_table + (size_t)s * max_blocks;

  const TA* qrow = q + ((size_t)t * heads + h) * hd;
  for (int d = threadIdx.x; d < hd; d += ATT_THREADS) qs[d] = to_f32(qrow[d]);
  __syncthreads();

  float acc[ATT_MAX_DPT];
#pragma unroll
  for (int i = 0; i < ATT_MAX_DPT; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  const int start = window > 0 ? max(0, pos - window + 1) : 0;
  for (int tile0 = start; tile0 <= pos; tile0 += ATT_TILE) {
    const int n = min(ATT_TILE, pos + 1 - tile0);
    // scores: one warp per key, lanes over the head dimension
    for (int j = warp; j < n; j += nwarps) {
      const int kp = tile0 + j;
      const int page = bt[kp / page_size];
      const int off = kp % page_size;
      const TA* krow = kc + (((size_t)page * kvh + kh) * page_size + off) * hd;
      float dot = 0.f;
      for (int d = lane; d < hd; d += 32) dot += qs[d] * to_f32(krow[d]);
      dot = warp_sum(dot);
      if (lane == 0) sc[j] = dot * scale;
    }
    __syncthreads();
    float tm = -INFINITY;
    for (int j = 0; j < n; ++j) tm = fmaxf(tm, sc[j]);
    const float m_new = fmaxf(m, tm);
    const float corr = expf(m - m_new);  // 0 on the first tile (m = -inf)
    __syncthreads();
    for (int j = threadIdx.x; j < n; j += ATT_THREADS) sc[j] = expf(sc[j] - m_new);
    __syncthreads();
    float psum = 0.f;
    for (int j = 0; j < n; ++j) psum += sc[j];
    l = l * corr + psum;
    m = m_new;
#pragma unroll
    for (int i = 0; i < ATT_MAX_DPT; ++i) acc[i] *= corr;
    for (int j = 0; j < n; ++j) {
      const int kp = tile0 + j;
      const int page = bt[kp / page_size];
      const int off = kp % page_size;
      const TA* vrow = vc + (((size_t)page * kvh + kh) * page_size + off) * hd;
      const float p = sc[j];
#pragma unroll
      for (int i = 0; i < ATT_MAX_DPT; ++i) {
        const int d = threadIdx.x + i * ATT_THREADS;
        if (d < hd) acc[i] += p * to_f32(vrow[d]);
      }
    }
    __syncthreads();
  }
  TA* orow = out + ((size_t)t * heads + h) * hd;
  const float inv_l = 1.0f / l;
#pragma unroll
  for (int i = 0; i < ATT_MAX_DPT; ++i) {
    const int d = threadIdx.x + i * ATT_THREADS;
    if (d < hd) orow[d] = from_f32<TA>(acc[i] * inv_l);
  }
}

// The largest head size any attention kernel of this library takes (this one; the tuned
// kernels take fewer); a model is checked against it when it is built.
IX_API int ix_attention_max_head_dim() { return ATT_THREADS * ATT_MAX_DPT; }

IX_API int ix_paged_attention_generic(const void* q, const void* k_cache, const void* v_cache,
                                      const int* block_table, const int* seq_of_token,
                                      const int* positions, void* out, int act_dtype, int T,
                                      int heads, int kvh, int hd, int page_size, int max_blocks,
                                      int window, float scale, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || heads % kvh != 0 || page_size <= 0 || max_blocks <= 0)
    return IX_ERR_SIZE;
  if (hd <= 0 || hd > ATT_THREADS * ATT_MAX_DPT) return IX_ERR_SIZE;
  if (window < 0) return IX_ERR_SIZE;
  const size_t smem = (size_t)(hd + ATT_TILE) * sizeof(float);
  if (heads > 65535) return IX_ERR_SIZE;
  dim3 grid(T, heads);
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    (paged_attention_generic_kernel<TA><<<grid, ATT_THREADS, smem, stream>>>(
                        (const TA*)q, (const TA*)k_cache, (const TA*)v_cache, block_table,
                        seq_of_token, positions, (TA*)out, heads, kvh, hd, page_size, max_blocks,
                        window, scale)));
  return ix_launch_status();
}
