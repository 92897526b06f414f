// Shared declarations for the sm_100a kernel library.
//
// Every entry point is a plain C function taking raw device pointers, sizes and
// the CUDA stream to launch on; it returns 0, a positive cudaError_t, or a
// negative IX_ERR_* code for arguments the kernel refuses.  Nothing here
// allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#include <tuple>
#include <utility>

#define IX_API extern "C" __attribute__((visibility("default")))

enum { IX_F32 = 0, IX_BF16 = 1 };

enum {
  IX_OK = 0,
  IX_ERR_DTYPE = -1,       // element type code not known
  IX_ERR_SIZE = -2,        // a size the kernel does not take
  IX_ERR_ALIGN = -3,       // pointer or stride not aligned as required
  IX_ERR_SMEM = -4,        // shared memory need exceeds the device limit
  IX_ERR_UNSUPPORTED = -5  // combination not built
};

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block in a fixed order: shuffle tree inside each warp, then the
// per-warp partials are added by every thread in ascending warp order.
// `scratch` holds at least 32 floats.  All threads get the same value.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel that starts with IX_PDL_WAIT() may be
// launched with ix_launch(): it is then allowed onto the SMs while its predecessor
// in the stream is still draining (its blocks sit at the wait until the predecessor
// has completed and its writes are visible), which hides launch latency, block
// scheduling and the kernel's own prologue.  IX_PDL_WAIT() must come before the
// first access to global memory; a kernel launched the ordinary way passes through
// it at once.  INFERX_PDL=0 in the environment turns the attribute off.
// ---------------------------------------------------------------------------
#define IX_PDL_WAIT()                                             \
  do {                                                            \
    asm volatile("griddepcontrol.wait;" ::: "memory");            \
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); \
  } while (0)

// Whether launches carry the attribute: set per step by the caller (it pays for
// steps of a few tokens, where kernels are short; with many tokens early-resident
// dependents get in the way of other streams), and INFERX_PDL=0 forces it off.
extern "C" int ix_dependent_launch_flag(int set_to);   // -1 reads; defined in elementwise.cu

static inline bool ix_pdl_enabled() {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("INFERX_PDL");
    env = (e && e[0] == '0') ? 0 : 1;
  }
  return env == 1 && ix_dependent_launch_flag(-1) == 1;
}

template <typename... P, typename... A, size_t... I>
static inline cudaError_t ix_launch_impl(void (*kern)(P...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, std::index_sequence<I...>, A... a) {
  std::tuple<P...> params{static_cast<P>(a)...};
  void* ptrs[] = {(void*)&std::get<I>(params)...};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ix_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelExC(&cfg, (const void*)kern, ptrs);
}

// Launch a kernel whose first statement is IX_PDL_WAIT().
template <typename... P, typename... A>
static inline void ix_launch(void (*kern)(P...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, A... a) {
  static_assert(sizeof...(P) == sizeof...(A), "argument count differs from the kernel's");
  ix_launch_impl(kern, grid, block, smem, stream, std::index_sequence_for<P...>{}, a...);
}

static inline int ix_launch_status() {
  cudaError_t e = cudaGetLastError();
  return (int)e;
}

#define IX_DISPATCH_DTYPE(code, T, ...)            \
  do {                                             \
    if ((code) == IX_F32) {                        \
      typedef float T;                             \
      __VA_ARGS__;                                 \
    } else if ((code) == IX_BF16) {                \
      typedef bf16 T;                              \
      __VA_ARGS__;                                 \
    } else {                                       \
      return IX_ERR_DTYPE;                         \
    }                                              \
  } while (0)
