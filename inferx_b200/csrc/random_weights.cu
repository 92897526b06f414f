// Seeded random weights drawn on the device: one launch per tensor.
//
// out[i] = float(shift + std * z_i), z_i standard normal and a function of (key, i) only:
// the splitmix64 finaliser of the counter key + (i + 1) * golden gives 64 bits, of which
// the top 16 choose a cell of the inverse normal distribution function (a table of 65537
// quantiles computed on the host) and the next 32 a place inside the cell by linear
// interpolation.  The integer arithmetic wraps, and every double operation is a single
// IEEE operation rounded to nearest (no fused multiply-add), so the result is the same
// bits as the same steps done with torch on the CPU (weights/loader.py: counter_normal),
// which is what lets a plain CPU implementation draw the model the engine drew.  The
// reference engine has no random-weights mode; its tests synthesise deterministic
// tensors on the host (tests/kernel/deepseek_v2_model_test.cc:91-116).
#include "common.cuh"

__global__ void __launch_bounds__(256)
counter_normal_kernel(unsigned long long key, long long n, const double* __restrict__ table,
                      double std, double shift, int add_shift, float* __restrict__ out) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    unsigned long long z = key + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z ^= z >> 31;
    const unsigned cell = (unsigned)(z >> 48);
    const double frac = __dmul_rn((double)((z >> 16) & 0xFFFFFFFFULL), 1.0 / 4294967296.0);
    const double a = table[cell], b = table[cell + 1];
    double v = __dadd_rn(a, __dmul_rn(__dsub_rn(b, a), frac));
    v = __dmul_rn(v, std);
    if (add_shift) v = __dadd_rn(v, shift);
    out[i] = __double2float_rn(v);
  }
}

// table: 65537 doubles on the device; out: n floats.
IX_API int ix_counter_normal(unsigned long long key, long long n, const double* table, double std,
                             double shift, int add_shift, float* out, cudaStream_t stream) {
  if (n <= 0) return IX_OK;
  if (!table || !out) return IX_ERR_SIZE;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;
  counter_normal_kernel<<<(unsigned)blocks, 256, 0, stream>>>(key, n, table, std, shift,
                                                              add_shift, out);
  return ix_launch_status();
}
