// Row-wise kernels: embedding gather, residual add + RMSNorm, SiLU*mul, and the
// MoE combine with the sigmoid-gated shared expert.
//
// Reference behaviour: EmbeddingKernel (src/backends/cuda/ops/layers.cu:465-481),
// RmsNormKernel (layers.cu:50-76) with AddKernel (layers.cu:542-548) folded in,
// SiluMulFusedKernel (layers.cu:512-529), CombineRowsKernel and
// AddSharedExpertKernel (src/backends/cuda/ops/moe.cu:237-255,275-287).
// The residual stream is kept in 32-bit here, so the residual sum never rounds.
#include "common.cuh"
#include "elementwise_vec.cuh"

IX_API int ix_dependent_launch_flag(int set_to) {
  static int flag = 0;
  if (set_to >= 0) flag = set_to ? 1 : 0;
  return flag;
}

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

__global__ void embed_bf16_vec_kernel(const uint4* __restrict__ table, const int* __restrict__ ids,
                                      float4* __restrict__ out, int chunks, int V) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;
  const uint4* row = table + (size_t)id * chunks;
  float4* o = out + (size_t)t * chunks * 2;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    float f[8];
    bf8_to_f32(row[c], f);
    o[2 * c] = make_float4(f[0], f[1], f[2], f[3]);
    o[2 * c + 1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

IX_API int ix_embed(const void* table, int table_dtype, const int* ids, int T, int H, int V,
                    float* out, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || V <= 0) return IX_ERR_SIZE;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == IX_BF16 && H % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
    ix_launch(embed_bf16_vec_kernel, dim3(T), dim3(threads), 0, stream, (const uint4*)table, ids,
              (float4*)out, H / 8, V);
    return ix_launch_status();
  }
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

// bf16 activations, H a multiple of 8: each thread keeps up to NI chunks of 8 values in
// registers, so the row is read once.  Same sum order as the scalar kernel is not
// needed for equality between batches (a row is always reduced by one block the same way).
template <int NI>
__global__ void add_rmsnorm_bf16_vec_kernel(float* __restrict__ resid, const bf16* __restrict__ delta,
                                            const float* __restrict__ gain,
                                            const int* __restrict__ rows, bf16* __restrict__ out,
                                            int H, float eps, int write_resid) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float4* x = reinterpret_cast<float4*>(resid + src * H);
  const uint4* d = delta ? reinterpret_cast<const uint4*>(delta + src * H) : nullptr;
  const int chunks = H >> 3;
  float v[NI][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      const float4 a = x[2 * c], b = x[2 * c + 1];
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
      v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
      if (d) {
        float f[8];
        bf8_to_f32(d[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += f[j];
      }
      if (write_resid && d) {
        x[2 * c] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
        x[2 * c + 1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  uint4* o = reinterpret_cast<uint4*>(out + (size_t)r * H);
  const float4* gw = reinterpret_cast<const float4*>(gain);
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      const float4 ga = gw[2 * c], gb = gw[2 * c + 1];
      float f[8];
      f[0] = v[i][0] * inv * ga.x; f[1] = v[i][1] * inv * ga.y;
      f[2] = v[i][2] * inv * ga.z; f[3] = v[i][3] * inv * ga.w;
      f[4] = v[i][4] * inv * gb.x; f[5] = v[i][5] * inv * gb.y;
      f[6] = v[i][6] * inv * gb.z; f[7] = v[i][7] * inv * gb.w;
      o[c] = f32_to_bf8(f);
    }
  }
}

IX_API int ix_add_rmsnorm(float* resid, const void* delta, const float* gain, const int* rows,
                          void* out, int act_dtype, int R, int H, float eps, int write_resid,
                          cudaStream_t stream) {
  if (R <= 0) return IX_OK;
  if (H <= 0) return IX_ERR_SIZE;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  if (act_dtype == IX_BF16 && H % 8 == 0 &&
      (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)gain | (uintptr_t)out) & 15) == 0) {
    const int chunks = H / 8;
    const int vt = chunks >= 256 ? 256 : (chunks >= 128 ? 128 : 64);
    const int ni = (chunks + vt - 1) / vt;
    if (ni <= 4) {
      if (ni == 1)
        ix_launch(add_rmsnorm_bf16_vec_kernel<1>, dim3(R), dim3(vt), 0, stream, resid,
                  (const bf16*)delta, gain, rows, (bf16*)out, H, eps, write_resid);
      else if (ni == 2)
        ix_launch(add_rmsnorm_bf16_vec_kernel<2>, dim3(R), dim3(vt), 0, stream, resid,
                  (const bf16*)delta, gain, rows, (bf16*)out, H, eps, write_resid);
      else
        ix_launch(add_rmsnorm_bf16_vec_kernel<4>, dim3(R), dim3(vt), 0, stream, resid,
                  (const bf16*)delta, gain, rows, (bf16*)out, H, eps, write_resid);
      return ix_launch_status();
    }
  }
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

// bf16 rows of 8-element chunks.  Two chunks a pass (four loads in flight), 32-bit index
// arithmetic, and the fast exponential and reciprocal: the exact ones make this kernel
// wait on instruction issue instead of on memory (their error is far below a bf16 ulp).
__global__ void __launch_bounds__(256)
silu_mul_bf16_vec_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out,
                         unsigned total_chunks, unsigned chunks_per_row) {
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < total_chunks; i0 += 2 * stride) {
    const unsigned i1 = i0 + stride;
    const bool two = i1 < total_chunks;
    const unsigned t0 = i0 / chunks_per_row, t1 = two ? i1 / chunks_per_row : t0;
    const size_t a0 = (size_t)t0 * chunks_per_row + i0;          // t * 2 * cpr + c
    const size_t a1 = two ? (size_t)t1 * chunks_per_row + i1 : a0;
    const uint4 g0 = gu[a0], u0 = gu[a0 + chunks_per_row];
    const uint4 g1 = gu[a1], u1 = gu[a1 + chunks_per_row];
    float g[8], u[8], o[8];
    bf8_to_f32(g0, g);
    bf8_to_f32(u0, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __fdividef(g[j], 1.0f + __expf(-g[j])) * u[j];
    out[i0] = f32_to_bf8(o);
    if (two) {
      bf8_to_f32(g1, g);
      bf8_to_f32(u1, u);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __fdividef(g[j], 1.0f + __expf(-g[j])) * u[j];
      out[i1] = f32_to_bf8(o);
    }
  }
}

IX_API int ix_silu_mul(const void* gu, void* out, int act_dtype, int T, int I,
                       cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (I <= 0) return IX_ERR_SIZE;
  const long long total = (long long)T * I;
  if (act_dtype == IX_BF16 && I % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0 &&
      total / 8 < (1LL << 30)) {
    const long long chunks = total / 8;
    long long vb = (chunks + 511) / 512;
    if (vb > 148 * 8) vb = 148 * 8;
    silu_mul_bf16_vec_kernel<<<(int)vb, 256, 0, stream>>>((const uint4*)gu, (uint4*)out,
                                                          (unsigned)chunks, (unsigned)(I / 8));
    return ix_launch_status();
  }
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

__global__ void moe_combine_bf16_vec_kernel(const uint4* __restrict__ y, const int* __restrict__ dest,
                                            const float* __restrict__ w,
                                            const uint4* __restrict__ shared,
                                            const float* __restrict__ shared_logit,
                                            uint4* __restrict__ out, int chunks, int k) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  float sg = 1.0f;
  if (shared && shared_logit) sg = 1.0f / (1.0f + expf(-shared_logit[t]));
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      const int row = dest[t * k + s];
      const float ws = w[t * k + s];
      float f[8];
      bf8_to_f32(y[(size_t)row * chunks + c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += ws * f[j];
    }
    if (shared) {
      float f[8];
      bf8_to_f32(shared[(size_t)t * chunks + c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += sg * f[j];
    }
    out[(size_t)t * chunks + c] = f32_to_bf8(acc);
  }
}

// ---------------------------------------------------------------------------
// The combine above folded into the residual add + RMSNorm that consumes it: the
// row of routed and shared contributions is formed in registers and never written.
// ---------------------------------------------------------------------------
template <int NI>
__global__ void combine_add_rmsnorm_bf16_vec_kernel(
    float* __restrict__ resid, const uint4* __restrict__ y, const int* __restrict__ dest,
    const float* __restrict__ w, const uint4* __restrict__ shared,
    const float* __restrict__ shared_logit, const float* __restrict__ gain,
    bf16* __restrict__ out, int H, int k, float eps) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int chunks = H >> 3;
  float4* x = reinterpret_cast<float4*>(resid + (size_t)t * H);
  float sg = 1.0f;
  if (shared && shared_logit) sg = 1.0f / (1.0f + expf(-shared_logit[t]));
  float v[NI][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int s = 0; s < k; ++s) {
        const int row = dest[t * k + s];
        const float ws = w[t * k + s];
        float f[8];
        bf8_to_f32(y[(size_t)row * chunks + c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += ws * f[j];
      }
      if (shared) {
        float f[8];
        bf8_to_f32(shared[(size_t)t * chunks + c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += sg * f[j];
      }
      const float4 a = x[2 * c], b = x[2 * c + 1];
      v[i][0] = a.x + acc[0]; v[i][1] = a.y + acc[1]; v[i][2] = a.z + acc[2];
      v[i][3] = a.w + acc[3]; v[i][4] = b.x + acc[4]; v[i][5] = b.y + acc[5];
      v[i][6] = b.z + acc[6]; v[i][7] = b.w + acc[7];
      x[2 * c] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
      x[2 * c + 1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  uint4* o = reinterpret_cast<uint4*>(out + (size_t)t * H);
  const float4* gw = reinterpret_cast<const float4*>(gain);
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      const float4 ga = gw[2 * c], gb = gw[2 * c + 1];
      float f[8];
      f[0] = v[i][0] * inv * ga.x; f[1] = v[i][1] * inv * ga.y;
      f[2] = v[i][2] * inv * ga.z; f[3] = v[i][3] * inv * ga.w;
      f[4] = v[i][4] * inv * gb.x; f[5] = v[i][5] * inv * gb.y;
      f[6] = v[i][6] * inv * gb.z; f[7] = v[i][7] * inv * gb.w;
      o[c] = f32_to_bf8(f);
    }
  }
}

// resid[t] += combine(t); out[t] = RMSNorm(resid[t]) * gain.  bf16, H a multiple of 8 up
// to 8192; anything else is refused and the caller runs the two kernels.
IX_API int ix_combine_add_rmsnorm(float* resid, const void* y, const int* dest, const float* w,
                                  const void* shared, const float* shared_logit,
                                  const float* gain, void* out, int T, int H, int k, float eps,
                                  cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || k <= 0) return IX_ERR_SIZE;
  if (H % 8 != 0) return IX_ERR_UNSUPPORTED;
  if ((((uintptr_t)resid | (uintptr_t)y | (uintptr_t)shared | (uintptr_t)gain | (uintptr_t)out) &
       15) != 0)
    return IX_ERR_ALIGN;
  const int chunks = H / 8;
  const int vt = chunks >= 256 ? 256 : (chunks >= 128 ? 128 : 64);
  const int ni = (chunks + vt - 1) / vt;
  if (ni > 4) return IX_ERR_UNSUPPORTED;
#define IX_CAR(NI)                                                                           \
  ix_launch(combine_add_rmsnorm_bf16_vec_kernel<NI>, dim3(T), dim3(vt), 0, stream, resid,     \
            (const uint4*)y, dest, w, (const uint4*)shared, shared_logit, gain, (bf16*)out, H, k, \
            eps)
  if (ni == 1) IX_CAR(1);
  else if (ni == 2) IX_CAR(2);
  else IX_CAR(4);
#undef IX_CAR
  return ix_launch_status();
}

IX_API int ix_moe_combine(const void* y, const int* dest, const float* w, const void* shared,
                          const float* shared_logit, void* out, int act_dtype, int T, int H, int k,
                          cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || k <= 0) return IX_ERR_SIZE;
  const int threads = H >= 1024 ? 256 : 128;
  if (act_dtype == IX_BF16 && H % 8 == 0 &&
      (((uintptr_t)y | (uintptr_t)shared | (uintptr_t)out) & 15) == 0) {
    ix_launch(moe_combine_bf16_vec_kernel, dim3(T), dim3(H >= 2048 ? 256 : 128), 0, stream,
              (const uint4*)y, dest, w, (const uint4*)shared, shared_logit, (uint4*)out, H / 8, k);
    return ix_launch_status();
  }
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    (moe_combine_kernel<TA><<<T, threads, 0, stream>>>(
                        (const TA*)y, dest, w, (const TA*)shared, shared_logit, (TA*)out, H, k)));
  return ix_launch_status();
}
