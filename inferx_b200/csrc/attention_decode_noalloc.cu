// The allocation-free face of the split-KV decode attention: same kernels, with
// the partial results kept in an array that lives inside the library.  What it
// is for, its limit and its rules are in inferx_b200_noalloc.h.
#include <stdio.h>

#include <mutex>

#include "common.cuh"
#include "inferx_b200_noalloc.h"

// The ordinary entry points this one is built on (attention_decode.cu).
extern "C" int ix_attn_decode_splits(int S, int heads, int kvh, int max_kv_len);
extern "C" int ix_paged_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                                         const int* block_table, const int* kv_len, float* part_o,
                                         float* part_ml, void* out, int act_dtype, int S,
                                         int heads, int kvh, int hd, int page_size,
                                         int max_blocks, int window, float scale, int splits,
                                         cudaStream_t stream);

// Partial outputs first, then the (max, sum) pairs.  In host code this name only
// stands for the symbol; the address kernels can use comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_decode_scratch[IX_NOALLOC_SCRATCH_FLOATS];

#define IX_NOALLOC_MAX_DEVICES 64
static float* g_scratch_addr[IX_NOALLOC_MAX_DEVICES];
static std::mutex g_scratch_mutex;

// Device address of the array on the current device; looked up once per device.
static int scratch_for_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= IX_NOALLOC_MAX_DEVICES) return IX_ERR_SIZE;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  *ptr = g_scratch_addr[dev];
  return IX_OK;
}

IX_API int ix_paged_attention_decode_noalloc(const void* q, const void* k_cache,
                                             const void* v_cache, const int* block_table,
                                             const int* kv_len, void* out, int act_dtype, int S,
                                             int heads, int kv_heads, int head_dim, int page_size,
                                             int max_blocks, int window, float scale,
                                             int max_kv_len, cudaStream_t stream) {
  if (S <= 0) return IX_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || head_dim <= 0 || max_kv_len <= 0)
    return IX_ERR_SIZE;
  const int splits = ix_attn_decode_splits(S, heads, kv_heads, max_kv_len);
  const unsigned long long rows = (unsigned long long)S * heads * splits;
  const unsigned long long need = rows * ((unsigned long long)head_dim + 2ull);
  if (splits > 1 && need > IX_NOALLOC_SCRATCH_FLOATS) {
    fprintf(stderr,
            "ix_paged_attention_decode_noalloc: %d sequences x %d heads x %d splits x "
            "(head_dim %d + 2) = %llu floats of partial results exceed the built-in scratch of "
            "%u floats; use ix_paged_attention_decode with your own buffers, or a smaller batch\n",
            S, heads, splits, head_dim, need, (unsigned)IX_NOALLOC_SCRATCH_FLOATS);
    return IX_ERR_SCRATCH_TOO_SMALL;
  }
  float* base = nullptr;
  const int rc = scratch_for_current_device(&base);
  if (rc != IX_OK) return rc;
  float* part_o = base;
  float* part_ml = base + rows * (unsigned long long)head_dim;
  return ix_paged_attention_decode(q, k_cache, v_cache, block_table, kv_len, part_o, part_ml, out,
                                   act_dtype, S, heads, kv_heads, head_dim, page_size, max_blocks,
                                   window, scale, splits, stream);
}
