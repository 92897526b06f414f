// Row-wise kernels: embedding gather, residual add + RMSNorm, SiLU*mul, and the
// MoE combine with the sigmoid-gated shared expert.
//
// Reference behaviour: EmbeddingKernel (src/backends/cuda/ops/layers.cu:465-481),
// RmsNormKernel (layers.cu:50-76) with AddKernel (layers.cu:542-548) folded in,
// SiluMulFusedKernel (layers.cu:512-529), CombineRowsKernel and
// AddSharedExpertKernel (src/backends/cuda/ops/moe.cu:237-255,275-287).
// The residual stream is kept in 32-bit here, so the residual sum never rounds.
#include "common.cuh"

// ---------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :] widened to fp32 (the residual stream)
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int H, int V) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;  // host validates; never read out of range
  const TW* row = table + (size_t)id * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

IX_API int ix_embed(const void* table, int table_dtype, const int* ids, int T, int H, int V,
                    float* out, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || V <= 0) return IX_ERR_SIZE;
  const int threads = H >= 1024 ? 256 : 128;
  IX_DISPATCH_DTYPE(table_dtype, TW,
                    (embed_kernel<TW><<<T, threads, 0, stream>>>((const TW*)table, ids, out, H, V)));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// residual add + RMSNorm.
//   v = resid[src] + delta[src]        (delta optional)
//   resid[src] = v                     (when write_resid)
//   out[r] = v * (1/sqrt(mean(v^2)+eps)) * gain
// src = rows[r] when a gather list is given, else r.  One block per row; the sum
// of squares is reduced in an order fixed by H and the block size only.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                                   const float* __restrict__ gain, const int* __restrict__ rows,
                                   TA* __restrict__ out, int H, float eps, int write_resid) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* x = resid + src * H;
  const TA* d = delta ? delta + src * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = x[i];
    if (d) v += to_f32(d[i]);
    if (write_resid) x[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TA* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = x[i];
    if (d && !write_resid) v += to_f32(d[i]);
    o[i] = from_f32<TA>(v * inv * gain[i]);
  }
}

IX_API int ix_add_rmsnorm(float* resid, const void* delta, const float* gain, const int* rows,
                          void* out, int act_dtype, int R, int H, float eps, int write_resid,
                          cudaStream_t stream) {
  if (R <= 0) return IX_OK;
  if (H <= 0) return IX_ERR_SIZE;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    (add_rmsnorm_kernel<TA><<<R, threads, 0, stream>>>(
                        resid, (const TA*)delta, gain, rows, (TA*)out, H, eps, write_resid)));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// out[t, j] = silu(gu[t, j]) * gu[t, I + j],  silu(g) = g / (1 + exp(-g))
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void silu_mul_kernel(const TA* __restrict__ gu, TA* __restrict__ out, long long total,
                                int I) {
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / I;
    const int j = (int)(idx - t * I);
    const float g = to_f32(gu[t * 2 * I + j]);
    const float u = to_f32(gu[t * 2 * I + I + j]);
    out[idx] = from_f32<TA>(g / (1.0f + expf(-g)) * u);
  }
}

IX_API int ix_silu_mul(const void* gu, void* out, int act_dtype, int T, int I,
                       cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (I <= 0) return IX_ERR_SIZE;
  const long long total = (long long)T * I;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    (silu_mul_kernel<TA><<<(int)blocks, 256, 0, stream>>>((const TA*)gu, (TA*)out,
                                                                          total, I)));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// MoE combine: out[t] = sum_slot w[t,slot] * y[dest[t*k+slot]]   (slot order)
//                     + sigmoid(shared_logit[t]) * shared[t]      (optional;
//                       ungated when shared_logit is null)
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ y, const int* __restrict__ dest,
                                   const float* __restrict__ w, const TA* __restrict__ shared,
                                   const float* __restrict__ shared_logit, TA* __restrict__ out,
                                   int H, int k) {
  const int t = blockIdx.x;
  float sg = 1.0f;
  if (shared && shared_logit) sg = 1.0f / (1.0f + expf(-shared_logit[t]));
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < k; ++s) {
      const int row = dest[t * k + s];
      acc += w[t * k + s] * to_f32(y[(size_t)row * H + i]);
    }
    if (shared) acc += sg * to_f32(shared[(size_t)t * H + i]);
    out[(size_t)t * H + i] = from_f32<TA>(acc);
  }
}

IX_API int ix_moe_combine(const void* y, const int* dest, const float* w, const void* shared,
                          const float* shared_logit, void* out, int act_dtype, int T, int H, int k,
                          cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || k <= 0) return IX_ERR_SIZE;
  const int threads = H >= 1024 ? 256 : 128;
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    (moe_combine_kernel<TA><<<T, threads, 0, stream>>>(
                        (const TA*)y, dest, w, (const TA*)shared, shared_logit, (TA*)out, H, k)));
  return ix_launch_status();
}
