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
// The weights are the M side of the MMA and the tokens the N side.  An expert's row
// count is ragged (a few hundred at most for a prompt portion of a few thousand
// tokens) and M is fixed at 128 while N may be any multiple of 16 up to 256, so
// this way round no tensor-core work is spent on padding, and - what matters more,
// since at these sizes the product is bound by reading the experts' weights - each
// 128-row tile of an expert's weights is read once for up to 256 of its tokens.
//
// The unit of work is, for one expert, 128 output features (gate and up rows when
// DUAL: two accumulators) for a tile of up to BT (128 to 256) of the expert's tokens;
// an expert with more rows is cut into equal tiles.
// The kernel is persistent: one block per SM takes work items round robin, ordered so
// that the feature tiles of one token tile run at the same time on neighbouring SMs
// (they share the token rows through L2).  Warp 0 streams the tiles (weights 128 x
// 64, tokens in boxes of 32 x 64) into a ring of shared-memory stages with
// cp.async.bulk.tensor (128-byte swizzle) and runs ahead into the next work item;
// warp 1 issues tcgen05.mma (M 128, N the tile's token count rounded up to 16, K 16
// per instruction, bf16 in, fp32 accumulate in TMEM) and releases stages with
// tcgen05.commit; warps 2-5 read the finished accumulator with tcgen05.ld (a thread
// holds one feature for 32 tokens), apply the epilogue and store bf16.  Where tensor
// memory has room for two accumulator sets (plain form; SwiGLU form at 128 tokens), the
// epilogue of one item overlaps the MMAs of the next; where it has not, the epilogue is
// short enough (branch-free, a microsecond or two a tile) that the wider tile still pays.  Token rows of the last box beyond the tile, feature rows beyond N and
// the K tail are computed on whatever TMA delivered (neighbouring rows or zero fill)
// and never stored.
//
// Every wait on an mbarrier is bounded: after the limit the waiter records a code
// in `status`, raises an abort flag that ends the other roles, and the block still
// frees its tensor memory before it returns.
//
// Requires bf16, K a multiple of 8 (16-byte row pitch for TMA), 16-byte aligned
// bases.  Anything else is refused with IX_ERR_UNSUPPORTED.
#include "common.cuh"
#include "tma_common.cuh"
#include "tcgen05_common.cuh"

#define TC_BF 128        // output features per work item (the MMA's M)
#define TC_BOX_T 32      // token rows per TMA box
#define TC_BK 64
#define TC_THREADS 192
#define TC_W_BYTES (TC_BF * TC_BK * 2)   // 16 KB: one 128 x 64 bf16 weight tile
#define TC_SMEM_STAGES (208 * 1024)      // shared memory given to the ring of stages
#define TC_MAX_EXPERTS 1024              // the per-expert tile prefix lives in shared memory

enum { TC_ERR_PRODUCER = 1, TC_ERR_MMA = 2, TC_ERR_EPILOGUE = 3 };

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
// kind::f16, D fp32, A and B bf16, both K-major, M = 128, N = n (a multiple of 16)
__device__ __forceinline__ unsigned tc_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(TC_BF >> 4) << 24);
}

// Tiles of an expert with `rows` rows: as few as hold BT each, of equal size (a
// multiple of 16).
template <int BT> __host__ __device__ __forceinline__ int tc_tiles_of(int rows) {
  return (rows + BT - 1) / BT;
}
__device__ __forceinline__ int tc_tile_rows(int rows, int tiles) {
  return ((rows + tiles - 1) / tiles + 15) & ~15;
}

struct TcItem {
  int e, m0, n_valid, f0;
};

// Work item `w` of the launch: token tile w / f_tiles (found by bisection in the
// prefix of tiles per expert), feature tile w % f_tiles.
template <int BT>
__device__ __forceinline__ TcItem tc_item(int w, int f_tiles, const int* tile_start,
                                          const int* __restrict__ offsets, int E,
                                          int f_item = TC_BF) {
  const int tt = w / f_tiles;
  int lo = 0, hi = E;                       // largest e with tile_start[e] <= tt
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_start[mid] <= tt) lo = mid; else hi = mid;
  }
  TcItem it;
  it.e = lo;
  const int r0 = offsets[lo], rows = offsets[lo + 1] - r0;
  const int tiles_e = tc_tiles_of<BT>(rows);
  const int per = tc_tile_rows(rows, tiles_e);
  it.m0 = r0 + (tt - tile_start[lo]) * per;
  it.n_valid = max(0, min(r0 + rows - it.m0, per));
  it.f0 = (w - tt * f_tiles) * f_item;
  return it;
}

// ---------------------------------------------------------------------------
// MODE 0: one weight tile an item; 1: gate and up tiles, SwiGLU epilogue; 2: two
// neighbouring feature tiles, both stored.
template <int MODE, int BT>
__global__ void __launch_bounds__(TC_THREADS, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                       const __grid_constant__ CUtensorMap map_w,
                       const int* __restrict__ offsets, bf16* __restrict__ out, int N, int K,
                       int E, int w_rows_per_expert, int* __restrict__ status) {
  constexpr bool DUAL = MODE != 0;      // two weight tiles and two accumulators an item
  constexpr bool SWIGLU = MODE == 1;
  constexpr int F_ITEM = MODE == 2 ? 2 * TC_BF : TC_BF;   // output features of an item
  constexpr int A_BYTES = BT * TC_BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + TC_W_BYTES * (DUAL ? 2 : 1);
  constexpr int STAGES = TC_SMEM_STAGES / STAGE_BYTES;
  constexpr int ACC_COLS = BT * (DUAL ? 2 : 1);          // one accumulator set
  constexpr int NBUF = ACC_COLS * 2 <= 512 ? 2 : 1;
  // tcgen05.alloc takes a power of two of at least 32 columns
  constexpr unsigned TMEM_NEED = ACC_COLS * NBUF;
  constexpr unsigned TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128
                                 : TMEM_NEED <= 256 ? 256 : 512;
  static_assert(TMEM_NEED <= 512, "tensor memory has 512 columns");
  static_assert(STAGES >= 2 && STAGES <= 8, "ring depth");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles =
      reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long full_bar[STAGES];
  __shared__ __align__(8) unsigned long long empty_bar[STAGES];
  __shared__ __align__(8) unsigned long long acc_full[NBUF];
  __shared__ __align__(8) unsigned long long acc_empty[NBUF];
  __shared__ unsigned tmem_holder;
  __shared__ int abort_flag;
  __shared__ int tile_start[TC_MAX_EXPERTS + 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + TC_BK - 1) / TC_BK;
  const int f_tiles = (N + F_ITEM - 1) / F_ITEM;

  // prefix of token tiles per expert (warp 2, 32 experts at a time)
  if (warp == 2) {
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int t = e < E ? tc_tiles_of<BT>(offsets[e + 1] - offsets[e]) : 0;
      int incl = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (e < E) tile_start[e] = carry + incl - t;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) tile_start[E] = carry;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);          // one arrival per epilogue warp
    }
    abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async();
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
  const int n_items = tile_start[E] * f_tiles;

  if (warp == 0) {
    if (lane == 0) {
      int fill = 0;            // k-tiles issued so far, over all items
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        const TcItem it = tc_item<BT>(w, f_tiles, tile_start, offsets, E, F_ITEM);
        if (it.n_valid <= 0) continue;
        const int boxes = (((it.n_valid + 15) & ~15) + TC_BOX_T - 1) / TC_BOX_T;
        const unsigned stage_tx =
            (unsigned)(TC_W_BYTES * (DUAL ? 2 : 1) + boxes * TC_BOX_T * TC_BK * 2);
        for (int kt = 0; kt < k_tiles; ++kt, ++fill) {
          const int s = fill % STAGES;
          ok = mbar_wait(&empty_bar[s], ((fill / STAGES) & 1) ^ 1, abortp);
          if (!ok) break;
          unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], stage_tx);
          tma_load_2d(st + A_BYTES, &map_w, kt * TC_BK, it.e * w_rows_per_expert + it.f0,
                      &full_bar[s]);
          if (DUAL)   // the up rows of the same features, or the next 128 features
            tma_load_2d(st + A_BYTES + TC_W_BYTES, &map_w, kt * TC_BK,
                        it.e * w_rows_per_expert + (SWIGLU ? N : TC_BF) + it.f0, &full_bar[s]);
          for (int b = 0; b < boxes; ++b)
            tma_load_2d(st + b * (TC_BOX_T * TC_BK * 2), &map_a, kt * TC_BK,
                        it.m0 + b * TC_BOX_T, &full_bar[s]);
        }
      }
      if (!ok) {
        if (!*abortp) { atomicExch(status, TC_ERR_PRODUCER); *abortp = 1; }
        // let copies already issued land before the block's shared memory goes away
        for (int f = max(0, fill - STAGES); f < fill; ++f)
          mbar_drain(&full_bar[f % STAGES], (f / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int drain = 0, n_done = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        const TcItem it = tc_item<BT>(w, f_tiles, tile_start, offsets, E, F_ITEM);
        if (it.n_valid <= 0) continue;
        const unsigned idesc = tc_idesc((it.n_valid + 15) & ~15);
        const int buf = n_done % NBUF;
        // the epilogue must have read this accumulator set's previous contents
        ok = mbar_wait(&acc_empty[buf], ((n_done / NBUF) & 1) ^ 1, abortp);
        if (!ok) break;
        tc_fence_after();
        const unsigned acc = tmem_base + buf * ACC_COLS;
        for (int kt = 0; kt < k_tiles; ++kt, ++drain) {
          const int s = drain % STAGES;
          ok = mbar_wait(&full_bar[s], (drain / STAGES) & 1, abortp);
          if (!ok) break;
          tc_fence_after();
          unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          const unsigned long long td = umma_desc(st);                          // tokens: N side
          const unsigned long long gd = umma_desc(st + A_BYTES);                // weights: M side
          const unsigned long long ud = umma_desc(st + A_BYTES + TC_W_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
            const unsigned accum = (kt > 0 || k4 > 0) ? 1u : 0u;
            // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
            tc_mma(acc, gd + 2 * k4, td + 2 * k4, idesc, accum);
            if (DUAL) tc_mma(acc + BT, ud + 2 * k4, td + 2 * k4, idesc, accum);
          }
          tc_commit(&empty_bar[s]);   // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        tc_commit(&acc_full[buf]);
        ++n_done;
      }
      if (!ok && !*abortp) { atomicExch(status, TC_ERR_MMA); *abortp = 1; }
    }
  } else {
    const int quarter = warp & 3;              // TMEM lanes this warp may read
    int n_done = 0;
    for (int w = blockIdx.x; w < n_items; w += gridDim.x) {
      const TcItem it = tc_item<BT>(w, f_tiles, tile_start, offsets, E, F_ITEM);
      if (it.n_valid <= 0) continue;
      const int buf = n_done % NBUF;
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (n_done / NBUF) & 1, abortp))) {
        if (lane == 0 && !*abortp) { atomicExch(status, TC_ERR_EPILOGUE); *abortp = 1; }
        break;
      }
      tc_fence_after();
      const int f = it.f0 + quarter * 32 + lane;    // this thread's output feature
      const bool f_ok = f < N;
      const unsigned taddr = tmem_base + buf * ACC_COLS + ((unsigned)(quarter * 32) << 16);
      for (int c0 = 0; c0 < it.n_valid; c0 += 32) {
        float g[32], u[DUAL ? 32 : 1];
        tc_ld32(taddr + c0, g);
        if (DUAL) tc_ld32(taddr + BT + c0, u);
        if (c0 + 32 >= it.n_valid) {
          // everything this warp needs is in registers: hand the accumulator back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        // All 32 values are computed without a branch (columns past the tile hold
        // whatever the MMA made of the rows TMA delivered; they are not stored), so the
        // exponentials and reciprocals of different columns overlap; a branch per column
        // would serialise their latencies.  The fast reciprocal's error is far below a
        // bf16 ulp.
        bf16 r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float a = g[i];
          if (SWIGLU) a = __fdividef(a, 1.0f + __expf(-a)) * u[i];
          r[i] = __float2bfloat16_rn(a);
        }
        // a warp's 32 threads hold 32 neighbouring features of one token: 64-byte stores
        bf16* dst = out + (size_t)(it.m0 + c0) * N + f;
        const int n_here = f_ok ? it.n_valid - c0 : 0;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < n_here) dst[(size_t)i * N] = r[i];
        if (MODE == 2) {        // the second tile's features, 128 further on
          const int n_second = f + TC_BF < N ? it.n_valid - c0 : 0;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < n_second) dst[(size_t)i * N + TC_BF] = __float2bfloat16_rn(u[i]);
        }
      }
      ++n_done;
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
// a: [A_rows, K] bf16 grouped rows; w: [E, (dual ? 2N : N), K] bf16; out: [A_rows, N] bf16.
// status: one int in device memory, zero before the first call; a bounded wait that
// ran out leaves a nonzero code there.
template <int MODE, int BT>
static int launch_tc(const void* a, const int* offsets, const void* w, void* out, int A_rows,
                     int N, int K, int E, long long w_rows, int* status, cudaStream_t stream) {
  CUtensorMap map_a, map_w;
  int rc = ix_tensor_map_bf16_2d(&map_a, a, A_rows, K, TC_BK, TC_BOX_T);
  if (rc != IX_OK) return rc;
  rc = ix_tensor_map_bf16_2d(&map_w, w, (long long)E * w_rows, K, TC_BK, TC_BF);
  if (rc != IX_OK) return rc;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms <= 0)
      sms = 148;
  }
  // every expert can add a partial token tile
  constexpr int F_ITEM = MODE == 2 ? 2 * TC_BF : TC_BF;
  const long long items =
      ((long long)tc_tiles_of<BT>(A_rows) + E) * ((N + F_ITEM - 1) / F_ITEM);
  const int grid = (int)(items < sms ? items : sms);
  const int smem = TC_SMEM_STAGES + 1024;
  auto kern = grouped_gemm_tc_kernel<MODE, BT>;
  cudaError_t e2 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e2 != cudaSuccess) return (int)e2;
  kern<<<grid, TC_THREADS, smem, stream>>>(map_a, map_w, offsets, (bf16*)out, N, K, E,
                                           (int)w_rows, status);
  return ix_launch_status();
}

IX_API int ix_grouped_gemm_tc(const void* a, const int* offsets, const void* w, void* out,
                              int dual, int A_rows, int N, int K, int E, int* status,
                              cudaStream_t stream) {
  if (A_rows <= 0) return IX_OK;
  if (N <= 0 || K <= 0 || E <= 0 || status == nullptr) return IX_ERR_SIZE;
  if (K % 8 != 0 || E > TC_MAX_EXPERTS) return IX_ERR_UNSUPPORTED;
  if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)out) & 15) return IX_ERR_ALIGN;
  const long long w_rows = dual ? 2LL * N : N;
  if ((long long)E * w_rows > 0x7fffffffLL) return IX_ERR_SIZE;
  // Width of the token tile: the mean rows of an expert plus 15 % for imbalance, cut
  // into as few tiles as 256 rows allow, and then the narrowest of 128 / 160 / 192 / 256
  // that holds such a tile.  The narrower the tile, the smaller its stage and the more
  // stages the ring holds; what the kernel achieves follows the bytes in flight, not the
  // tensor pipe (measured at 60 experts of 1408 x 2048: SwiGLU form, 136 rows an expert:
  // 150 / 153 / 154 us at 160 / 128 / 256; 273 rows: 223 / 237 / 243 us; plain form, 136
  // rows: 76 / 98 / 79 us; 102 rows: 69 us at 128 against 71-74 us).
  const double rows = 1.15 * (double)A_rows / (double)E;
  const int cuts = rows <= 256.0 ? 1 : (int)((rows + 255.0) / 256.0);
  const double per = rows / cuts;
  const int bt = per <= 128.0 ? 128 : per <= 160.0 ? 160 : per <= 192.0 ? 192 : 256;
#define IX_TC(D)                                                                              \
  do {                                                                                        \
    if (bt == 128) return launch_tc<D, 128>(a, offsets, w, out, A_rows, N, K, E, w_rows, status, stream); \
    if (bt == 160) return launch_tc<D, 160>(a, offsets, w, out, A_rows, N, K, E, w_rows, status, stream); \
    if (bt == 192) return launch_tc<D, 192>(a, offsets, w, out, A_rows, N, K, E, w_rows, status, stream); \
    return launch_tc<D, 256>(a, offsets, w, out, A_rows, N, K, E, w_rows, status, stream);   \
  } while (0)
  if (dual) IX_TC(1);
  // plain: two feature tiles an item when the features fill them (measured at 60 experts
  // of 2048 x 1408 against one tile an item: 77 us either way at 2,048 tokens, where 480
  // items on 148 blocks balance worse than 960; 109 against 131 us at 4,096 tokens and
  // 202 against 241 us at 8,192, where the token tile is read half as often)
  if (N >= 2 * TC_BF) IX_TC(2);
  IX_TC(0);
#undef IX_TC
}
