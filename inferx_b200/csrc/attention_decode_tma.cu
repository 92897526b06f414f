// Decode attention over the paged cache with the keys and values brought in by TMA.
//
// Same arithmetic, split layout and scratch as attn_decode_mma_kernel (64-key tiles,
// four warps of 16 keys each, mma.sync.m16n8k16 for S = Q K^T and O += P V, online
// softmax per warp, merge through shared memory); what differs is how a tile reaches
// shared memory.  A fifth warp (one lane per page of the tile) issues one
// cp.async.bulk.tensor per page and 64-wide half of the head (box: page_size keys x
// 64 elements, 128-byte swizzle) into a ring of stages guarded by full/empty
// mbarriers, so the four computing warps spend no instructions on addresses or copies
// and never stop at a block-wide barrier inside the loop.
//
// The cache [pages, kv_heads, page_size, head_dim] is seen by the tensor map as a 2-D
// tensor [pages * kv_heads * page_size, head_dim]; a page of one KV head is
// page_size consecutive rows.  Tiles start at multiples of 64 keys, so a page never
// straddles two tiles; pages wholly outside the live range [lo, k1) are not copied
// (their table entry may be -1 once a window has passed them) and their keys are
// masked; shared memory is zeroed once so that what a skipped page leaves behind is
// finite.
//
// Contract with the caller when launches carry the programmatic-serialisation
// attribute: kv_len, the block table and every key and value except the newest of each
// sequence must have been written before the preceding launch in the stream began; the
// preceding launch may write the query and the newest key and value only.  (The engine's
// step does exactly that: lengths and tables arrive with the step's inputs, older keys
// in earlier steps.)  The kernel uses it to request its first tiles before it waits for
// the preceding launch.
//
// Requires bf16, head_dim 64 or 128, page_size a power of two from 8 to 64.  Every
// wait on an mbarrier is bounded; a wait that ran out records a code (11: the copying
// warp, 12: a computing warp) in the caller's status word and the block runs on to its
// end.
#include "common.cuh"
#include "tma_common.cuh"

#define DT_BN 64
#define DT_STAGES 3                       // 101 KB a block: two blocks per SM
#define DT_WARPS 4                        // computing warps
#define DT_THREADS ((DT_WARPS + 1) * 32)  // + the copying warp

__device__ __forceinline__ void dt_ldsm(unsigned* r, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void dt_ldsm_t(unsigned* r, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void dt_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float dt_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Byte offset of 16-byte chunk c (0 .. HD/8-1) of key row r inside a stage: 64-wide
// halves of the head one after the other, each [64 rows][128 bytes] with the chunk
// index XORed by the row's low three bits (what the 128-byte swizzle of TMA writes).
__device__ __forceinline__ int dt_kv_off(int r, int c) {
  return (c >> 3) * (DT_BN * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}
// The query tile [16][HD] keeps the layout of the cp.async kernel.
template <int CH> __device__ __forceinline__ int dt_q_off(int r, int c) {
  return (r * CH + (c ^ (r & 7))) * 16;
}

template <int HD>
__global__ void __launch_bounds__(DT_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const bf16* __restrict__ q,
                       const int* __restrict__ block_table, const int* __restrict__ kv_len,
                       float* __restrict__ part_o, float* __restrict__ part_ml,
                       bf16* __restrict__ out, int heads, int kvh, int page_size, int page_shift,
                       int maxb, int window, float scale_log2e, int splits,
                       int* __restrict__ status) {
  constexpr int CH = HD / 8, KS = HD / 16, DTL = HD / 8, HALVES = HD / 64;
  constexpr int TILE_BYTES = DT_BN * HD * 2;
  extern __shared__ unsigned char dsm_raw[];
  unsigned char* dsm =
      reinterpret_cast<unsigned char*>(((uintptr_t)dsm_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* Ks = dsm;                                   // [STAGES][halves][64][128 B]
  unsigned char* Vs = Ks + DT_STAGES * TILE_BYTES;
  unsigned char* Qs = Vs + DT_STAGES * TILE_BYTES;           // [16][HD]
  __shared__ float sm_m[DT_WARPS][16];
  __shared__ float sm_l[DT_WARPS][16];
  __shared__ __align__(8) unsigned long long full_bar[DT_STAGES];
  __shared__ __align__(8) unsigned long long empty_bar[DT_STAGES];
  __shared__ int abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // set-up that touches no global memory runs before the wait on the predecessor
  if (tid == 0) {
    for (int i = 0; i < DT_STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], DT_WARPS);
    }
    abort_flag = 0;
    mbar_init_fence();
  }
  for (int i = tid; i < 2 * DT_STAGES * TILE_BYTES / 16; i += DT_THREADS)
    reinterpret_cast<uint4*>(Ks)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
  __syncthreads();     // barriers and zeroes are in place before any copy is issued

  // Lengths and block tables arrive with the step's inputs and the pages hold earlier
  // steps' keys: all of that was written long before the predecessor in the stream,
  // which only adds this step's newest key and the query.  So the geometry is worked out
  // and the first tiles (those that end before the newest key) are requested before the
  // wait on the predecessor; their latency then overlaps its tail.
  const int split = blockIdx.x, s = blockIdx.z;
  const int rep = heads / kvh;
  const int row_groups = (rep + 15) / 16;
  const int kh = blockIdx.y / row_groups;
  const int qrow0 = (blockIdx.y % row_groups) * 16;
  const int rows_valid = min(16, rep - qrow0);
  const int h0 = kh * rep + qrow0;
  const int g = lane >> 2, t = lane & 3;

  const int len = kv_len[s];
  const int lo = window > 0 ? max(0, len - window) : 0;     // first live key
  const int base = lo & ~(DT_BN - 1);                       // tiles start on 64-key marks
  const int n = len - base;
  int chunk = (n + splits - 1) / splits;
  chunk = (chunk + DT_BN - 1) / DT_BN * DT_BN;
  const int k0 = base + split * chunk;
  const int k1 = min(len, k0 + chunk);
  const int n_tiles = k1 > k0 ? (k1 - k0 + DT_BN - 1) / DT_BN : 0;

  // ---- copying warp: lane p brings page p of each tile; the page numbers of the next
  // tile are fetched before the wait for a free stage, so that their latency is off
  // the path between "stage free" and "copies issued" ----
  const int* bt = block_table + (size_t)s * maxb;
  const int pages_per_tile = DT_BN >> page_shift;
  const unsigned page_bytes = (unsigned)page_size * HD * 2;
  auto page_live = [&](int it) {     // does this lane's page of tile `it` hold live keys?
    const int kp = k0 + it * DT_BN + (lane << page_shift);
    return lane < pages_per_tile && it < n_tiles && kp + page_size > lo && kp < k1;
  };
  auto page_id = [&](int it) {
    return page_live(it) ? bt[((k0 + it * DT_BN) >> page_shift) + lane] : -1;
  };
  auto issue_tile = [&](int it, int pid) {
    const int stage = it % DT_STAGES;
    const bool live = page_live(it);
    const unsigned n_live = __popc(__ballot_sync(0xffffffffu, live));
    if (lane == 0) mbar_expect_tx(&full_bar[stage], 2u * page_bytes * n_live);
    __syncwarp();
    if (live) {
      const int row = (pid * kvh + kh) << page_shift;
      unsigned char* kd = Ks + stage * TILE_BYTES;
      unsigned char* vd = Vs + stage * TILE_BYTES;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        const int off = h * (DT_BN * 128) + (lane << page_shift) * 128;
        tma_load_2d(kd + off, &map_k, h * 64, row, &full_bar[stage]);
        tma_load_2d(vd + off, &map_v, h * 64, row, &full_bar[stage]);
      }
    }
  };
  int issued = 0, pid_next = -1;
  if (warp == DT_WARPS) {
    pid_next = page_id(0);
    while (issued < n_tiles && issued < DT_STAGES && k0 + (issued + 1) * DT_BN <= len - 1) {
      const int pid = pid_next;
      pid_next = page_id(issued + 1);
      issue_tile(issued, pid);
      ++issued;
    }
  }
  IX_PDL_WAIT();

  for (int idx = tid; idx < 16 * CH; idx += DT_THREADS) {
    const int r = idx / CH, c = idx - r * CH;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows_valid)
      v = *reinterpret_cast<const uint4*>(q + ((size_t)s * heads + h0 + r) * HD + c * 8);
    *reinterpret_cast<uint4*>(Qs + dt_q_off<CH>(r, c)) = v;
  }
  __syncthreads();

  float o[DTL][4];
#pragma unroll
  for (int j = 0; j < DTL; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  if (warp == DT_WARPS) {
    for (int it = issued; it < n_tiles; ++it) {
      const int stage = it % DT_STAGES;
      const int pid = pid_next;
      pid_next = page_id(it + 1);
      if (it >= DT_STAGES &&
          !__all_sync(0xffffffffu,
                      mbar_wait(&empty_bar[stage], ((it / DT_STAGES) - 1) & 1, &abort_flag))) {
        if (lane == 0) {
          atomicExch(status, 11);
          abort_flag = 1;
        }
        break;
      }
      issue_tile(it, pid);
    }
  } else {
    // ---- computing warps ----
    unsigned qf[KS][4];
#pragma unroll
    for (int kk = 0; kk < KS; ++kk)
      dt_ldsm(qf[kk], Qs + dt_q_off<CH>((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));
    for (int it = 0; it < n_tiles; ++it) {
      const int stage = it % DT_STAGES;
      if (!__all_sync(0xffffffffu,
                      mbar_wait(&full_bar[stage], (it / DT_STAGES) & 1, &abort_flag))) {
        if (lane == 0) {
          atomicExch(status, 12);
          abort_flag = 1;
        }
        break;
      }
      const unsigned char* kt = Ks + stage * TILE_BYTES;
      const unsigned char* vt = Vs + stage * TILE_BYTES;
      const int kw = k0 + it * DT_BN + warp * 16;      // first key of this warp's 16
      if (kw < k1 && kw + 16 > lo) {
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) sc[j][c] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
          unsigned b[4];
          dt_ldsm(b, kt + dt_kv_off(warp * 16 + (lane >> 4) * 8 + (lane & 7),
                                    kk * 2 + ((lane >> 3) & 1)));
          dt_mma(sc[0], qf[kk], b[0], b[1]);
          dt_mma(sc[1], qf[kk], b[2], b[3]);
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int kp = kw + j * 8 + 2 * t + (c & 1);
            const float v = (kp < k1 && kp >= lo) ? sc[j][c] * scale_log2e : -INFINITY;
            sc[j][c] = v;
            mx[c >> 1] = fmaxf(mx[c >> 1], v);
          }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
          const float m_new = fmaxf(m_run[r], mx[r]);
          m_use[r] = m_new == -INFINITY ? 0.f : m_new;
          corr[r] = dt_exp2(m_run[r] - m_use[r]);
          m_run[r] = m_new;
          l_run[r] *= corr[r];
        }
#pragma unroll
        for (int j = 0; j < DTL; ++j) {
          o[j][0] *= corr[0]; o[j][1] *= corr[0];
          o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
        unsigned pf[4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float p0 = dt_exp2(sc[j][0] - m_use[0]);
          const float p1 = dt_exp2(sc[j][1] - m_use[0]);
          const float p2 = dt_exp2(sc[j][2] - m_use[1]);
          const float p3 = dt_exp2(sc[j][3] - m_use[1]);
          l_run[0] += p0 + p1;
          l_run[1] += p2 + p3;
          __nv_bfloat162 lo2 = __floats2bfloat162_rn(p0, p1), hi2 = __floats2bfloat162_rn(p2, p3);
          pf[j * 2 + 0] = *reinterpret_cast<unsigned*>(&lo2);
          pf[j * 2 + 1] = *reinterpret_cast<unsigned*>(&hi2);
        }
#pragma unroll
        for (int jd = 0; jd < DTL; jd += 2) {
          unsigned b[4];
          dt_ldsm_t(b, vt + dt_kv_off(warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7),
                                      jd + (lane >> 4)));
          dt_mma(o[jd], pf, b[0], b[1]);
          dt_mma(o[jd + 1], pf, b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }
  }
  __syncthreads();
  if (abort_flag) {
    // let copies in flight land before shared memory is given up; the output of this
    // block is not meaningful and the status word says so
    if (tid == 0)
      for (int i = 0; i < DT_STAGES; ++i) {
        mbar_drain(&full_bar[i], 0);
        mbar_drain(&full_bar[i], 1);
      }
    __syncthreads();
  }

  // merge the four warps (each saw different keys); stage memory is free now
  float* sm_o = reinterpret_cast<float*>(Ks);     // [DT_WARPS][16][HD]
  if (warp < DT_WARPS) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    if (t == 0) {
      sm_m[warp][g] = m_run[0];     sm_l[warp][g] = l_run[0];
      sm_m[warp][g + 8] = m_run[1]; sm_l[warp][g + 8] = l_run[1];
    }
#pragma unroll
    for (int j = 0; j < DTL; ++j) {
      const int d = j * 8 + 2 * t;
      sm_o[(warp * 16 + g) * HD + d] = o[j][0];
      sm_o[(warp * 16 + g) * HD + d + 1] = o[j][1];
      sm_o[(warp * 16 + g + 8) * HD + d] = o[j][2];
      sm_o[(warp * 16 + g + 8) * HD + d + 1] = o[j][3];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < rows_valid * HD; idx += DT_THREADS) {
    const int r = idx / HD, d = idx - r * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) M = fmaxf(M, sm_m[w][r]);
    float ov = 0.f, L = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DT_WARPS; ++w) {
        const float cw = dt_exp2(sm_m[w][r] - M);   // exp2(-inf) = 0 for idle warps
        ov += sm_o[(w * 16 + r) * HD + d] * cw;
        L += sm_l[w][r] * cw;
      }
    }
    const size_t hrow = (size_t)s * heads + h0 + r;
    if (splits == 1) {
      out[hrow * HD + d] = __float2bfloat16_rn(L > 0.f ? ov / L : 0.f);
    } else {
      part_o[(hrow * splits + split) * HD + d] = ov;
      if (d == 0) {
        part_ml[(hrow * splits + split) * 2] = M;
        part_ml[(hrow * splits + split) * 2 + 1] = L;
      }
    }
  }
}

template <int HD>
static int launch_tma(const void* q, const void* kc, const void* vc, long long cache_rows,
                      const int* bt, const int* kv_len, float* part_o, float* part_ml, void* out,
                      int S, int heads, int kvh, int page_size, int page_shift, int maxb,
                      int window, float scale, int splits, int* status, cudaStream_t stream) {
  CUtensorMap map_k, map_v;
  int rc = ix_tensor_map_bf16_2d(&map_k, kc, cache_rows, HD, 64, page_size);
  if (rc != IX_OK) return rc;
  rc = ix_tensor_map_bf16_2d(&map_v, vc, cache_rows, HD, 64, page_size);
  if (rc != IX_OK) return rc;
  const int rep = heads / kvh;
  const float sl2 = scale * 1.4426950408889634f;
  const int smem = 2 * DT_STAGES * DT_BN * HD * 2 + 16 * HD * 2 + 1024;
  dim3 grid(splits, kvh * ((rep + 15) / 16), S);
  auto kern = attn_decode_tma_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  ix_launch(kern, grid, dim3(DT_THREADS), smem, stream, map_k, map_v, (const bf16*)q, bt, kv_len,
            part_o, part_ml, (bf16*)out, heads, kvh, page_size, page_shift, maxb, window, sl2,
            splits, status);
  return ix_launch_status();
}

// Whether the TMA form takes these sizes.
extern "C" int ix_attn_decode_tma_applies(int hd, int page_size) {
  return (hd == 64 || hd == 128) && (page_size == 8 || page_size == 16 || page_size == 32 ||
                                     page_size == 64);
}

// The split pass alone (partials into part_o / part_ml, or `out` when splits == 1);
// the caller launches the merge.  num_pages: pages in the cache tensors; status: one
// int in device memory, zero before the first call.
extern "C" int ix_attn_decode_tma_partials(const void* q, const void* kc, const void* vc,
                                           int num_pages, const int* bt, const int* kv_len,
                                           float* part_o, float* part_ml, void* out, int S,
                                           int heads, int kvh, int hd, int page_size, int maxb,
                                           int window, float scale, int splits, int* status,
                                           cudaStream_t stream) {
  if (!ix_attn_decode_tma_applies(hd, page_size) || num_pages <= 0) return IX_ERR_UNSUPPORTED;
  if (status == nullptr) return IX_ERR_SIZE;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const long long cache_rows = (long long)num_pages * kvh * page_size;
  if (cache_rows > 0x7fffffffLL) return IX_ERR_SIZE;
  if (hd == 128)
    return launch_tma<128>(q, kc, vc, cache_rows, bt, kv_len, part_o, part_ml, out, S, heads, kvh,
                           page_size, page_shift, maxb, window, scale, splits, status, stream);
  return launch_tma<64>(q, kc, vc, cache_rows, bt, kv_len, part_o, part_ml, out, S, heads, kvh,
                        page_size, page_shift, maxb, window, scale, splits, status, stream);
}
