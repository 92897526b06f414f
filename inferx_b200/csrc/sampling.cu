// Next-token choice from fp32 logits, one block per row.
//
// Reference behaviour: ArgmaxKernel (src/backends/cuda/ops/layers.cu:413-452,
// ties go to the lower index) and SampleKernel (layers.cu:1051-1303): greedy when
// temperature <= 0; otherwise p_i ~ exp(logit_i / t - max), a probability cutoff
// found by bisection for top-k (the k-th largest) and for top-p (the smallest
// head of the distribution whose mass reaches top_p), the min-p floor
// min_p * p_max in closed form, one uniform from a counter-based generator keyed
// by the row's seed, and an inverse-CDF walk in index order over the kept
// tokens.  The host twin is src/engine/host_sampling.cc:50-111.
//
// The uniform comes from splitmix64(seed) (top 24 bits), so the host can compute
// the same number without a device.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ float uniform_from_seed(unsigned long long seed) {
  unsigned long long z = seed + 0x9e3779b97f4a7c15ULL;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float m = -INFINITY;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, scratch[w]);
  return m;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const int* __restrict__ top_k,
              const float* __restrict__ min_p, const unsigned long long* __restrict__ seeds,
              int* __restrict__ out) {
  __shared__ float scratch[32];
  __shared__ int scratch_i[32];
  __shared__ float csum[SAMPLE_THREADS];
  __shared__ int s_chunk;
  __shared__ float s_base;
  IX_PDL_WAIT();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const float t = temperature ? temperature[r] : 0.f;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  if (!(t > 0.f)) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
      const float v = row[i];
      if (v > best || bi == 0x7fffffff) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) {
        best = ob; bi = oi;
      }
    }
    if (lane == 0) { scratch[warp] = best; scratch_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float b = scratch[0];
      int idx = scratch_i[0];
      for (int w = 1; w < SAMPLE_THREADS / 32; ++w) {
        const float ob = scratch[w];
        const int oi = scratch_i[w];
        if (oi != 0x7fffffff && (idx == 0x7fffffff || ob > b || (ob == b && oi < idx))) {
          b = ob; idx = oi;
        }
      }
      out[r] = idx == 0x7fffffff ? 0 : idx;
    }
    return;
  }

  const float inv_t = 1.0f / t;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, __fmul_rn(row[i], inv_t));
  mx = block_max(mx, scratch);
  float part = 0.f;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) part += expf(__fmul_rn(row[i], inv_t) - mx);
  const float total = block_sum(part, scratch);

  // probability cutoff in units where p_max = 1
  float cut = 0.f;
  const float mp = min_p ? min_p[r] : 0.f;
  if (mp > 0.f) cut = fminf(mp, 1.0f);
  const int tk = top_k ? top_k[r] : 0;
  if (tk > 0 && tk < V) {
    float lo = 0.f, hi = 1.f;
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f;
      for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS)
        cnt += expf(__fmul_rn(row[i], inv_t) - mx) >= mid ? 1.f : 0.f;
      cnt = block_sum(cnt, scratch);
      if (cnt >= (float)tk) lo = mid; else hi = mid;
    }
    cut = fmaxf(cut, lo);
  }
  const float tp = top_p ? top_p[r] : 1.f;
  if (tp < 1.f) {
    float lo = cut, hi = 1.f;
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo + hi);
      float mass = 0.f;
      for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
        const float p = expf(__fmul_rn(row[i], inv_t) - mx);
        mass += p >= mid ? p : 0.f;
      }
      mass = block_sum(mass, scratch);
      if (mass >= tp * total) lo = mid; else hi = mid;
    }
    cut = lo;
  }

  // inverse CDF in index order over the kept tokens; thread i owns a contiguous chunk
  const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int c0 = threadIdx.x * chunk;
  const int c1 = min(V, c0 + chunk);
  float mine = 0.f;
  for (int i = c0; i < c1; ++i) {
    const float p = expf(__fmul_rn(row[i], inv_t) - mx);
    if (p >= cut) mine += p;
  }
  csum[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int i = 0; i < SAMPLE_THREADS; ++i) run += csum[i];
    const float target = uniform_from_seed(seeds ? seeds[r] : 0ULL) * run;
    float acc = 0.f;
    int pick = -1, last = 0;
    float base = 0.f, last_base = 0.f;
    for (int i = 0; i < SAMPLE_THREADS; ++i) {
      const float c = csum[i];
      if (c > 0.f) {
        last = i; last_base = acc;
        if (acc + c >= target) { pick = i; base = acc; break; }
      }
      acc += c;
    }
    if (pick < 0) { pick = last; base = last_base; }
    s_chunk = pick;
    s_base = base;
    csum[0] = target;
  }
  __syncthreads();
  if ((int)threadIdx.x == s_chunk) {
    const float target = csum[0];
    float run = s_base;
    int chosen = -1, last = c0;
    for (int i = c0; i < c1; ++i) {
      const float p = expf(__fmul_rn(row[i], inv_t) - mx);
      if (p >= cut) {
        run += p;
        last = i;
        if (run >= target) { chosen = i; break; }
      }
    }
    out[r] = chosen >= 0 ? chosen : last;
  }
}

IX_API int ix_sample(const float* logits, int R, int V, const float* temperature,
                     const float* top_p, const int* top_k, const float* min_p,
                     const unsigned long long* seeds, int* out, cudaStream_t stream) {
  if (R <= 0) return IX_OK;
  if (V <= 0) return IX_ERR_SIZE;
  ix_launch(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, logits, V, temperature,
            top_p, top_k, min_p, seeds, out);
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// Penalties and masks on the logits before a token is chosen, in place.
//
// Reference behaviour (src/engine/host_sampling.cc:21-48; the device twin is
// ApplyPenaltiesKernel, src/backends/cuda/ops/layers.cu:1310-1347): for every distinct token a
// row has generated so far (at most `hist_cap` of them, with how often), the logit is
// divided by the repetition penalty when positive and multiplied by it otherwise, then
// lowered by the presence penalty and by the frequency penalty times the count; after
// that the row's masked tokens (stop tokens while fewer than `min_tokens` have been
// generated) are set to -inf.  Ids below zero are padding.  One block per row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
apply_penalties_kernel(float* __restrict__ logits, int V, const int* __restrict__ hist_ids,
                       const int* __restrict__ hist_counts, int hist_cap,
                       const float* __restrict__ penalties, const int* __restrict__ mask_ids,
                       int mask_cap) {
  IX_PDL_WAIT();
  const int r = blockIdx.x;
  float* row = logits + (size_t)r * V;
  if (hist_ids) {
    const float presence = penalties[3 * r], frequency = penalties[3 * r + 1],
                repetition = penalties[3 * r + 2];
    if (presence != 0.f || frequency != 0.f || repetition != 1.f) {
      for (int j = threadIdx.x; j < hist_cap; j += blockDim.x) {
        const int id = hist_ids[(size_t)r * hist_cap + j];
        if (id < 0 || id >= V) continue;
        float v = row[id];                 // the ids of a row are distinct
        if (repetition != 1.f) v = v > 0.f ? v / repetition : v * repetition;
        v -= presence;
        v -= frequency * (float)hist_counts[(size_t)r * hist_cap + j];
        row[id] = v;
      }
    }
  }
  __syncthreads();
  if (mask_ids) {
    for (int j = threadIdx.x; j < mask_cap; j += blockDim.x) {
      const int id = mask_ids[(size_t)r * mask_cap + j];
      if (id >= 0 && id < V) row[id] = -INFINITY;
    }
  }
}

// logits [R, V] fp32, changed in place; hist_ids / hist_counts [R, hist_cap] int32 with
// penalties [R, 3] (presence, frequency, repetition), or all three null; mask_ids
// [R, mask_cap] int32 or null.
IX_API int ix_apply_penalties(float* logits, int R, int V, const int* hist_ids,
                              const int* hist_counts, int hist_cap, const float* penalties,
                              const int* mask_ids, int mask_cap, cudaStream_t stream) {
  if (R <= 0) return IX_OK;
  if (V <= 0 || !logits) return IX_ERR_SIZE;
  if ((hist_ids != nullptr) != (hist_counts != nullptr) ||
      (hist_ids != nullptr) != (penalties != nullptr))
    return IX_ERR_SIZE;
  if ((hist_ids && hist_cap <= 0) || (mask_ids && mask_cap <= 0)) return IX_ERR_SIZE;
  if (!hist_ids && !mask_ids) return IX_OK;
  ix_launch(apply_penalties_kernel, dim3(R), dim3(256), 0, stream, logits, V, hist_ids,
            hist_counts, hist_cap, penalties, mask_ids, mask_cap);
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// Log-probabilities of the chosen token and of the most probable alternatives.
//
// Reference behaviour (src/engine/host_sampling.cc:114-146, ComputeLogprobsKernel in
// src/backends/cuda/ops/layers.cu:1351-1460): over the row as it was
// sampled from (after penalties and masks, before temperature),
// log Z = log(sum exp(x - max)) + max with the sum in fp64; the chosen token's
// log-probability is x[chosen] - log Z; the alternatives are the `k` largest logits,
// ties to the lower id, most probable first.  One block per row; the k-th alternative
// is the largest element that comes after the (k-1)-th in that order, so no list of
// taken ids is kept.  A row whose k is negative is skipped.
// ---------------------------------------------------------------------------
#define LOGPROB_THREADS 1024
#define LOGPROB_MAX_TOP 20

__global__ void __launch_bounds__(LOGPROB_THREADS)
token_logprobs_kernel(const float* __restrict__ logits, int V, const int* __restrict__ chosen,
                      const int* __restrict__ want_k, int top_cap,
                      float* __restrict__ chosen_lp, int* __restrict__ top_ids,
                      float* __restrict__ top_lps) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ double s_sum[32];
  __shared__ float s_best;
  __shared__ int s_best_i;
  IX_PDL_WAIT();
  const int r = blockIdx.x;
  const int k = want_k ? want_k[r] : 0;
  if (k < 0) return;
  const float* row = logits + (size_t)r * V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += LOGPROB_THREADS) mx = fmaxf(mx, row[i]);
  mx = block_max(mx, s_val);
  double sum = 0.0;
  for (int i = threadIdx.x; i < V; i += LOGPROB_THREADS) sum += (double)expf(row[i] - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncthreads();
  if (lane == 0) s_sum[warp] = sum;
  __syncthreads();
  double total = 0.0;
  for (int w = 0; w < LOGPROB_THREADS / 32; ++w) total += s_sum[w];
  const float log_z = (float)log(total) + mx;
  if (threadIdx.x == 0) {
    const int c = chosen[r];
    chosen_lp[r] = (c >= 0 && c < V) ? row[c] - log_z : -INFINITY;
  }
  // the alternatives, one pass over the row each
  float prev = INFINITY;
  int prev_i = -1;
  const int n = min(k, top_cap);
  for (int j = 0; j < top_cap; ++j) {
    if (j >= n) {
      if (threadIdx.x == 0) {
        top_ids[(size_t)r * top_cap + j] = -1;
        top_lps[(size_t)r * top_cap + j] = 0.f;
      }
      continue;
    }
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += LOGPROB_THREADS) {
      const float v = row[i];
      // after (prev, prev_i) in the order: value descending, then id ascending
      const bool after = v < prev || (v == prev && i > prev_i);
      if (after && (v > best || (v == best && i < bi))) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    __syncthreads();
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float b = s_val[0];
      int bidx = s_idx[0];
      for (int w = 1; w < LOGPROB_THREADS / 32; ++w)
        if (s_val[w] > b || (s_val[w] == b && s_idx[w] < bidx)) { b = s_val[w]; bidx = s_idx[w]; }
      s_best = b;
      s_best_i = bidx;
      const bool found = bidx != 0x7fffffff;
      top_ids[(size_t)r * top_cap + j] = found ? bidx : -1;
      top_lps[(size_t)r * top_cap + j] = found ? b - log_z : 0.f;
    }
    __syncthreads();
    prev = s_best;
    prev_i = s_best_i;
    if (prev_i == 0x7fffffff) prev = -INFINITY;   // nothing left: the rest stay empty
  }
}

IX_API int ix_logprobs_max_top() { return LOGPROB_MAX_TOP; }

// logits [R, V] fp32; chosen [R] int32; want_k [R] int32 (negative: skip the row) or null
// (chosen token only, every row); chosen_lp [R] fp32; top_ids / top_lps [R, top_cap],
// -1 / 0 where a row asked for fewer.
IX_API int ix_token_logprobs(const float* logits, int R, int V, const int* chosen,
                             const int* want_k, int top_cap, float* chosen_lp, int* top_ids,
                             float* top_lps, cudaStream_t stream) {
  if (R <= 0) return IX_OK;
  if (V <= 0 || !logits || !chosen || !chosen_lp) return IX_ERR_SIZE;
  if (top_cap < 0 || top_cap > LOGPROB_MAX_TOP || (top_cap > 0 && (!top_ids || !top_lps)))
    return IX_ERR_SIZE;
  ix_launch(token_logprobs_kernel, dim3(R), dim3(LOGPROB_THREADS), 0, stream, logits, V, chosen,
            want_k, top_cap, chosen_lp, top_ids, top_lps);
  return ix_launch_status();
}
