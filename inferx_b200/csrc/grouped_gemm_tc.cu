// Grouped (per-expert) matrix product on the 5th-generation tensor cores:
// TMA-fed, tcgen05.mma with the accumulator in tensor memory.
//
//   out[r, j] = sum_k a[r, k] * w[e(r), j, k]                      (plain)
//   out[r, j] = silu(a . wg[e, j]) * (a . wu[e, j])                 (DUAL: SwiGLU)
//
// `a` holds the activation rows already grouped by expert (rows of expert e are
// offsets[e] .. offsets[e+1]); `w` is [E, rows_per_expert, K] with K contiguous.
// This is the prompt-sized counterpart of the reference's scalar
// GroupedGemmBf16Kernel<16> + SiluMulFused (src/backends/cuda/ops/moe.cu:324-392,
// 647-705; src/backends/cuda/ops/layers.cu:512-529), whose own notes name a
// tensor-core grouped GEMM as the upgrade (include/inferx/ops/moe.h:125-126).
//
// One block computes a 128 x 128 output tile of one expert (two accumulators when
// DUAL: gate and up).  Warp 0 streams 128 x 64 tiles of A and W into a ring of
// shared-memory stages with cp.async.bulk.tensor (128-byte swizzle); warp 1
// issues tcgen05.mma (M 128, N 128, K 16 per instruction, bf16 in, fp32
// accumulate in TMEM) and releases stages with tcgen05.commit; warps 2-5 read the
// finished accumulator with tcgen05.ld, apply the epilogue and store bf16 rows
// that belong to the expert.  Rows of the tile beyond the expert's range, columns
// beyond N and the K tail are computed on whatever TMA delivered (neighbouring
// rows or zero fill) and never stored.
//
// Every wait on an mbarrier is bounded: after the limit the waiter records a code
// in `status`, raises an abort flag that ends the other roles, and the block still
// frees its tensor memory before it returns.
//
// Requires bf16, K a multiple of 8 (16-byte row pitch for TMA), 16-byte aligned
// bases.  Anything else is refused with IX_ERR_UNSUPPORTED.
#include "common.cuh"
#include "tma_common.cuh"

#define TC_BM 128
#define TC_BN 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_TILE_BYTES (TC_BM * TC_BK * 2)   // 16 KB: one 128 x 64 bf16 tile
// two blocks per SM (96 KB of stages each), so that one block's epilogue and set-up
// overlap the other's MMA work
#define TC_STAGES_DUAL 2
#define TC_STAGES_PLAIN 3

enum { TC_ERR_PRODUCER = 1, TC_ERR_MMA = 2, TC_ERR_EPILOGUE = 3 };

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long adesc,
                                       unsigned long long bdesc, unsigned idesc, unsigned accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_ld32(unsigned taddr, float* v) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024
// bytes apart (stride byte offset), version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ unsigned long long umma_desc(const void* smem_tile) {
  const unsigned addr = smem_u32(smem_tile);
  return (unsigned long long)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) |
         (1ull << 46) | (2ull << 61);
}
// kind::f16, D fp32, A and B bf16, both K-major, N = 128, M = 128
#define TC_IDESC ((1u << 4) | (1u << 7) | (1u << 10) | ((TC_BN >> 3) << 17) | ((TC_BM >> 4) << 24))

// ---------------------------------------------------------------------------
template <bool DUAL>
__global__ void __launch_bounds__(TC_THREADS)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                       const __grid_constant__ CUtensorMap map_w,
                       const int* __restrict__ offsets, bf16* __restrict__ out, int N, int K,
                       int E, int w_rows_per_expert, int* __restrict__ status) {
  constexpr int STAGES = DUAL ? TC_STAGES_DUAL : TC_STAGES_PLAIN;
  constexpr int STAGE_BYTES = TC_TILE_BYTES * (DUAL ? 3 : 2);
  constexpr unsigned TMEM_COLS = DUAL ? 256 : 128;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles =
      reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long full_bar[STAGES];
  __shared__ __align__(8) unsigned long long empty_bar[STAGES];
  __shared__ __align__(8) unsigned long long accum_bar;
  __shared__ unsigned tmem_holder;
  __shared__ int abort_flag;

  // which expert and which 128-row tile of it
  int e = 0, m0 = 0, m_end = 0;
  {
    int tile = blockIdx.y;
    bool found = false;
    for (int ee = 0; ee < E; ++ee) {
      const int lo = offsets[ee], hi = offsets[ee + 1];
      const int tiles_e = (hi - lo + TC_BM - 1) / TC_BM;
      if (tile < tiles_e) {
        e = ee; m0 = lo + tile * TC_BM; m_end = hi; found = true;
        break;
      }
      tile -= tiles_e;
    }
    if (!found) return;   // before any barrier or allocation: the whole block leaves
  }
  const int n0 = blockIdx.x * TC_BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_holder;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int armed = 0;
      bool ok = true;
      for (int kt = 0; kt < k_tiles && ok; ++kt) {
        const int s = kt % STAGES;
        ok = mbar_wait(&empty_bar[s], ((kt / STAGES) & 1) ^ 1, abortp);
        if (!ok) break;
        unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(st, &map_a, kt * TC_BK, m0, &full_bar[s]);
        tma_load_2d(st + TC_TILE_BYTES, &map_w, kt * TC_BK, e * w_rows_per_expert + n0,
                    &full_bar[s]);
        if (DUAL)
          tma_load_2d(st + 2 * TC_TILE_BYTES, &map_w, kt * TC_BK,
                      e * w_rows_per_expert + N + n0, &full_bar[s]);
        armed = kt + 1;
      }
      if (!ok) {
        if (!*abortp) { atomicExch(status, TC_ERR_PRODUCER); *abortp = 1; }
        // let copies already issued land before the block's shared memory goes away
        for (int kt = max(0, armed - STAGES); kt < armed; ++kt)
          mbar_drain(&full_bar[kt % STAGES], (kt / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kt = 0; kt < k_tiles && ok; ++kt) {
        const int s = kt % STAGES;
        ok = mbar_wait(&full_bar[s], (kt / STAGES) & 1, abortp);
        if (!ok) break;
        tc_fence_after();
        unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
        const unsigned long long ad = umma_desc(st);
        const unsigned long long bd = umma_desc(st + TC_TILE_BYTES);
        const unsigned long long ud = umma_desc(st + 2 * TC_TILE_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
          const unsigned accum = (kt > 0 || k4 > 0) ? 1u : 0u;
          // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
          tc_mma(tmem_base, ad + 2 * k4, bd + 2 * k4, TC_IDESC, accum);
          if (DUAL) tc_mma(tmem_base + TC_BN, ad + 2 * k4, ud + 2 * k4, TC_IDESC, accum);
        }
        tc_commit(&empty_bar[s]);   // frees the stage once these MMAs have read it
      }
      if (ok) tc_commit(&accum_bar);
      else if (!*abortp) { atomicExch(status, TC_ERR_MMA); *abortp = 1; }
    }
  } else {
    const bool ok = mbar_wait(&accum_bar, 0, abortp);
    if (!ok) {
      if (lane == 0 && !*abortp) { atomicExch(status, TC_ERR_EPILOGUE); *abortp = 1; }
    } else {
      tc_fence_after();
      const int quarter = warp & 3;              // TMEM lanes this warp may read
      const int row = quarter * 32 + lane;
      const int r = m0 + row;
      const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
      for (int c0 = 0; c0 < TC_BN; c0 += 32) {
        float g[32], u[DUAL ? 32 : 1];
        tc_ld32(taddr + c0, g);
        if (DUAL) tc_ld32(taddr + TC_BN + c0, u);
        if (r < m_end) {
          bf16* dst = out + (size_t)r * N + n0 + c0;
          if (n0 + c0 + 32 <= N && (N % 8) == 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              unsigned pk[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float a = g[i + 2 * j], b = g[i + 2 * j + 1];
                if (DUAL) {
                  a = a / (1.0f + __expf(-a)) * u[i + 2 * j];
                  b = b / (1.0f + __expf(-b)) * u[i + 2 * j + 1];
                }
                __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
                pk[j] = *reinterpret_cast<unsigned*>(&v);
              }
              *reinterpret_cast<uint4*>(dst + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          } else {
            for (int i = 0; i < 32; ++i) {
              if (n0 + c0 + i < N) {
                float a = g[i];
                if (DUAL) a = a / (1.0f + __expf(-a)) * u[i];
                dst[i] = __float2bfloat16_rn(a);
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// gather: dst[i, :] = src[rows[i], :]  (16-byte copies; the reference's
// GatherRowsKernel, src/backends/cuda/ops/moe.cu:223-231)
// ---------------------------------------------------------------------------
__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ rows,
                                   uint4* __restrict__ dst, int chunks) {
  const size_t r = blockIdx.x;
  const size_t s = rows[r];
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) dst[r * chunks + c] = src[s * chunks + c];
}

IX_API int ix_gather_rows(const void* src, const int* rows, void* dst, int n_rows, int row_bytes,
                          cudaStream_t stream) {
  if (n_rows <= 0) return IX_OK;
  if (row_bytes <= 0 || row_bytes % 16 != 0) return IX_ERR_UNSUPPORTED;
  if (((uintptr_t)src | (uintptr_t)dst) & 15) return IX_ERR_ALIGN;
  gather_rows_kernel<<<n_rows, 128, 0, stream>>>((const uint4*)src, rows, (uint4*)dst,
                                                 row_bytes / 16);
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// 2-D bf16 tensor [rows, cols] with cols contiguous; boxes of 128 rows x 64 columns.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols) {
  return ix_tensor_map_bf16_2d(map, base, rows, cols, TC_BK, TC_BM);
}

// a: [A_rows, K] bf16 grouped rows; w: [E, (dual ? 2N : N), K] bf16; out: [A_rows, N] bf16.
// status: one int in device memory, zero before the first call; a bounded wait that
// ran out leaves a nonzero code there.
IX_API int ix_grouped_gemm_tc(const void* a, const int* offsets, const void* w, void* out,
                              int dual, int A_rows, int N, int K, int E, int* status,
                              cudaStream_t stream) {
  if (A_rows <= 0) return IX_OK;
  if (N <= 0 || K <= 0 || E <= 0 || status == nullptr) return IX_ERR_SIZE;
  if (K % 8 != 0) return IX_ERR_UNSUPPORTED;
  if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)out) & 15) return IX_ERR_ALIGN;
  const long long w_rows = dual ? 2LL * N : N;
  if ((long long)E * w_rows > 0x7fffffffLL) return IX_ERR_SIZE;
  CUtensorMap map_a, map_w;
  int rc = make_map(&map_a, a, A_rows, K);
  if (rc != IX_OK) return rc;
  rc = make_map(&map_w, w, (long long)E * w_rows, K);
  if (rc != IX_OK) return rc;
  const int m_tiles = (A_rows + TC_BM - 1) / TC_BM + E;   // every expert can add a partial tile
  if (m_tiles > 65535) return IX_ERR_SIZE;
  dim3 grid((N + TC_BN - 1) / TC_BN, m_tiles);
  if (dual) {
    const int smem = TC_STAGES_DUAL * TC_TILE_BYTES * 3 + 1024;
    auto kern = grouped_gemm_tc_kernel<true>;
    cudaError_t e2 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e2 != cudaSuccess) return (int)e2;
    kern<<<grid, TC_THREADS, smem, stream>>>(map_a, map_w, offsets, (bf16*)out, N, K, E,
                                             (int)w_rows, status);
  } else {
    const int smem = TC_STAGES_PLAIN * TC_TILE_BYTES * 2 + 1024;
    auto kern = grouped_gemm_tc_kernel<false>;
    cudaError_t e2 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e2 != cudaSuccess) return (int)e2;
    kern<<<grid, TC_THREADS, smem, stream>>>(map_a, map_w, offsets, (bf16*)out, N, K, E,
                                             (int)w_rows, status);
  }
  return ix_launch_status();
}
