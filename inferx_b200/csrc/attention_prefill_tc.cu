// Paged causal attention for prompt portions on the 5th-generation tensor cores:
// S = Q K^T and O += P V by tcgen05.mma with S and O in tensor memory, K and V pages
// brought in by TMA.  Same semantics as attn_prefill_kernel (ragged batch, tiles
// aligned to absolute positions, causal and window mask by position, softmax in fp32
// with exp2 on scores pre-scaled by log2 e, P rounded to bf16 before P V; the
// reference's FlashInfer prefill, src/backends/cuda/ops/flashinfer_prefill.cu:294-343).
//
// One block owns 128 consecutive queries of one sequence and one head (a query is a
// lane of tensor memory) and walks its keys in tiles of 64.  Roles:
//   warp 0     copies: Q once, then per tile one cp.async.bulk.tensor per page and
//              64-wide half of the head for K and for V (one lane per page), into
//              two-stage rings with their own full/empty mbarriers;
//   warp 1     one thread issues the MMAs: S_{j+1} = Q K_{j+1}^T (M 128, N 64) ahead
//              of O += P_j V_j (M 128, N head_dim, V read as an MN-major operand
//              straight from its [key][dim] tile), so the tensor pipe works on the
//              next scores while the softmax warps are busy with the current ones;
//   warps 2-5  softmax: a thread holds one query row; it reads the row of S with
//              tcgen05.ld, masks, keeps the running max and sum, writes P as bf16
//              back into the columns of tensor memory that S came from (P V takes
//              its A operand from there), and at the end scales O by 1 / sum and
//              stores it.
// The running max is updated lazily: O (in tensor memory) is rescaled only when some
// row's max grew by more than 2^8 since the last rescale, the exponent in between is
// taken against the older max, which changes nothing in exact arithmetic and keeps
// P within bf16's range.
//
// Two blocks fit on an SM (96 KB of shared memory and 256 columns of tensor memory
// each), so one block's softmax overlaps the other's MMAs.  A step with few (query
// tile, head) items over a long context (a prompt portion late in its sequence) has its
// keys cut into runs, one block each (blockIdx.z), that leave their unnormalised O,
// reference max and sum for a small merge kernel.  Every mbarrier wait is
// bounded; a wait that ran out records a code (21: copies, 22: MMA, 23: softmax) in
// the caller's status word and the block runs to its end (its output is then not
// meaningful).
//
// Requires bf16, head_dim 64 or 128, page_size a power of two from 8 to 64.
#include "common.cuh"
#include "tma_common.cuh"
#include "tcgen05_common.cuh"

#define FA_BM 128
#define FA_BN 64
#define FA_THREADS 192
#define FA_RESCALE_STEP 8.0f   // log2 units

enum { FA_ERR_COPY = 21, FA_ERR_MMA = 22, FA_ERR_SOFTMAX = 23, FA_ERR_ALIGN = 24 };

struct FaBars {
  unsigned long long q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready,
      o_done;
  unsigned tmem_holder;
  int abort_flag;
};

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two fp32 operations per instruction (packed f32x2) and a three-input maximum: the
// softmax warps are bound by instruction issue, so the per-score work is kept to a
// max, a fused multiply-add, an exp2, an add and half a pack.
__device__ __forceinline__ void fa_fma2(float& r0, float& r1, float x0, float x1, float s,
                                        float c) {
  asm("{ .reg .b64 va, vs, vc, vd;\n\t"
      "mov.b64 va, {%2, %3};\n\t"
      "mov.b64 vs, {%4, %4};\n\t"
      "mov.b64 vc, {%5, %5};\n\t"
      "fma.rn.f32x2 vd, va, vs, vc;\n\t"
      "mov.b64 {%0, %1}, vd; }"
      : "=f"(r0), "=f"(r1)
      : "f"(x0), "f"(x1), "f"(s), "f"(c));
}
__device__ __forceinline__ void fa_add2(float& a0, float& a1, float b0, float b1) {
  asm("{ .reg .b64 va, vb, vd;\n\t"
      "mov.b64 va, {%0, %1};\n\t"
      "mov.b64 vb, {%2, %3};\n\t"
      "add.rn.f32x2 vd, va, vb;\n\t"
      "mov.b64 {%0, %1}, vd; }"
      : "+f"(a0), "+f"(a1)
      : "f"(b0), "f"(b1));
}
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
  float m;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(a), "f"(b), "f"(c));
  return m;
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v,
                       const int* __restrict__ block_table, const int* __restrict__ cu_q,
                       const int* __restrict__ q_pos0, bf16* __restrict__ out, int S, int heads,
                       int kvh, int page_size, int page_shift, int maxb, int window,
                       float scale_log2e, int* __restrict__ status, int nsplit,
                       float* __restrict__ part_o, float* __restrict__ part_ml) {
  constexpr int HALVES = HD / 64;
  constexpr int Q_BYTES = FA_BM * HD * 2;
  constexpr int Q_HALF = FA_BM * 128;
  constexpr int KV_TILE = FA_BN * HD * 2;
  constexpr int KV_HALF = FA_BN * 128;
  constexpr unsigned TMEM_COLS = 256;
  // O: columns [0, HD); then two S buffers of 64 columns; P_j overwrites the first 32
  // columns of S_j's buffer
  constexpr unsigned S_COL = HD;
  // kind::f16, D fp32, A and B bf16; S: both K-major, N = 64; P V: B is MN-major, N = HD
  constexpr unsigned IDESC_S =
      (1u << 4) | (1u << 7) | (1u << 10) | ((FA_BN >> 3) << 17) | ((FA_BM >> 4) << 24);
  constexpr unsigned IDESC_PV =
      (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((HD >> 3) << 17) | ((FA_BM >> 4) << 24);

  extern __shared__ unsigned char smem[];       // the block has no static shared memory,
  unsigned char* Qs = smem;                     // so this starts on a 1024-byte mark
  unsigned char* Ks = Qs + Q_BYTES;             // [2][halves][64 keys][128 B]
  unsigned char* Vs = Ks + 2 * KV_TILE;
  FaBars* bars = reinterpret_cast<FaBars*>(Vs + 2 * KV_TILE);

  // which sequence and which 128-query tile of it; heavy tiles first (see the
  // mma.sync kernel)
  int s = 0, tile = gridDim.y - 1 - blockIdx.y;
  {
    bool found = false;
    for (int ss = 0; ss < S; ++ss) {
      const int n = cu_q[ss + 1] - cu_q[ss];
      const int tiles = (n + FA_BM - 1) / FA_BM;
      if (tile < tiles) { s = ss; found = true; break; }
      tile -= tiles;
    }
    if (!found) return;
  }
  const int h = blockIdx.x;
  const int kh = h / (heads / kvh);
  const int tok0 = cu_q[s];
  const int nq = cu_q[s + 1] - tok0;
  const int q0 = tile * FA_BM;
  const int rows_valid = min(FA_BM, nq - q0);
  const int pos0 = q_pos0[s] + q0;               // position of the tile's first query
  const int pmax = pos0 + rows_valid - 1;
  const int kv_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kv_hi = pmax + 1;
  // the tile's keys, cut into nsplit runs of whole 64-key tiles (blockIdx.z takes one)
  const int kt_first = kv_lo & ~(FA_BN - 1);
  const int n_all = (kv_hi - kt_first + FA_BN - 1) / FA_BN;
  const int per_split = (n_all + nsplit - 1) / nsplit;
  const int kt0 = kt_first + (int)blockIdx.z * per_split * FA_BN;
  const int n_tiles = max(0, min(per_split, n_all - (int)blockIdx.z * per_split));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  if ((smem_u32(smem) & 1023u) != 0) {           // the swizzle needs it; never seen
    if (tid == 0) atomicExch(status, FA_ERR_ALIGN);
    return;
  }
  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
    }
    mbar_init(&bars->p_ready, 4);               // one arrival per softmax warp
    mbar_init(&bars->o_done, 1);
    bars->abort_flag = 0;
    mbar_init_fence();
  }
  // pages that hold no live key are not copied; what they would leave in a stage must
  // be finite
  for (int i = tid; i < 4 * KV_TILE / 16; i += FA_THREADS)
    reinterpret_cast<uint4*>(Ks)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&bars->tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = bars->tmem_holder;
  volatile int* abortp = &bars->abort_flag;

  if (warp == 0) {
    // ---- copies ----
    const int* bt = block_table + (size_t)s * maxb;
    const int pages_per_tile = FA_BN >> page_shift;
    const unsigned page_bytes = (unsigned)page_size * HD * 2;
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, Q_BYTES);
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf)
        tma_load_2d(Qs + hf * Q_HALF, &map_q, h * HD + hf * 64, tok0 + q0, &bars->q_full);
    }
    auto page_live = [&](int j) {
      const int kp = kt0 + j * FA_BN + (lane << page_shift);
      return lane < pages_per_tile && j < n_tiles && kp + page_size > kv_lo && kp < kv_hi;
    };
    auto page_id = [&](int j) {
      return page_live(j) ? bt[((kt0 + j * FA_BN) >> page_shift) + lane] : -1;
    };
    int pid_next = page_id(0);
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
      const int pid = pid_next;
      pid_next = page_id(j + 1);
      const bool live = page_live(j);
      const unsigned n_live = __popc(__ballot_sync(0xffffffffu, live));
      const int row = (pid * kvh + kh) << page_shift;
      const int dst = (lane << page_shift) * 128;
      ok = __all_sync(0xffffffffu,
                      mbar_wait(&bars->k_empty[st], ((j >> 1) & 1) ^ 1, abortp));
      if (!ok) break;
      if (lane == 0) mbar_expect_tx(&bars->k_full[st], page_bytes * n_live);
      __syncwarp();
      if (live) {
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf)
          tma_load_2d(Ks + st * KV_TILE + hf * KV_HALF + dst, &map_k, hf * 64, row,
                      &bars->k_full[st]);
      }
      ok = __all_sync(0xffffffffu,
                      mbar_wait(&bars->v_empty[st], ((j >> 1) & 1) ^ 1, abortp));
      if (!ok) break;
      if (lane == 0) mbar_expect_tx(&bars->v_full[st], page_bytes * n_live);
      __syncwarp();
      if (live) {
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf)
          tma_load_2d(Vs + st * KV_TILE + hf * KV_HALF + dst, &map_v, hf * 64, row,
                      &bars->v_full[st]);
      }
    }
    if (!ok && lane == 0 && !*abortp) { atomicExch(status, FA_ERR_COPY); *abortp = 1; }
  } else if (warp == 1) {
    // ---- MMA issue ----
    if (lane == 0) {
      bool ok = mbar_wait(&bars->q_full, 0, abortp);
      auto issue_s = [&](int j) {      // S_j = Q K_j^T into S buffer j & 1
        const int st = j & 1;
        if (!mbar_wait(&bars->k_full[st], (j >> 1) & 1, abortp)) return false;
        // the buffer's last reader, P_{j-2} V_{j-2}, was issued before this: the tensor
        // pipe keeps the order
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const unsigned long long qd = umma_desc(Qs + (kk >> 2) * Q_HALF) + 2 * (kk & 3);
          const unsigned long long kd =
              umma_desc(Ks + st * KV_TILE + (kk >> 2) * KV_HALF) + 2 * (kk & 3);
          tc_mma(tmem_base + S_COL + st * FA_BN, qd, kd, IDESC_S, kk > 0 ? 1u : 0u);
        }
        tc_commit(&bars->k_empty[st]);
        tc_commit(&bars->s_full[st]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        const int st = j & 1;
        ok = mbar_wait(&bars->p_ready, j & 1, abortp) &&
             mbar_wait(&bars->v_full[st], (j >> 1) & 1, abortp);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k4 = 0; k4 < FA_BN / 16; ++k4) {
          // 16 keys further along K: 8 columns of packed P, two 8-key groups (2048
          // bytes) down V's tile
          const unsigned long long vd = umma_desc_mn(Vs + st * KV_TILE, KV_HALF, 1024) + 128 * k4;
          tc_mma_ts(tmem_base, tmem_base + S_COL + st * FA_BN + 8 * k4, vd, IDESC_PV,
                    (j > 0 || k4 > 0) ? 1u : 0u);
        }
        tc_commit(&bars->v_empty[st]);
        tc_commit(&bars->o_done);
      }
      if (!ok && !*abortp) { atomicExch(status, FA_ERR_MMA); *abortp = 1; }
    }
  } else {
    // ---- softmax ----
    const int quarter = warp & 3;                  // TMEM lanes this warp may touch
    const int row = quarter * 32 + lane;
    const int pos = pos0 + row;
    const int lo_r = window > 0 ? pos - window + 1 : 0;
    const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[st], (j >> 1) & 1, abortp));
      if (!ok) break;
      tc_fence_after();
      float sc[FA_BN];
      tc_ld32(lane_addr + S_COL + st * FA_BN, sc);
      tc_ld32(lane_addr + S_COL + st * FA_BN + 32, sc + 32);
      const int kbase = kt0 + j * FA_BN;
      const bool need_mask = (kbase + FA_BN - 1 > pos0) || kbase < kv_lo ||
                             (window > 0 && kbase < pmax - window + 1);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < FA_BN; ++i) {
          const int kp = kbase + i;
          if (kp > pos || kp < lo_r) sc[i] = -INFINITY;
        }
      }
      // of the raw scores (the scale is positive); two chains, so that one max does not
      // wait for the one before it
      float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
      for (int i = 0; i < FA_BN; i += 4) {
        mxa = fa_max3(mxa, sc[i], sc[i + 1]);
        mxb = fa_max3(mxb, sc[i + 2], sc[i + 3]);
      }
      const float mx = fmaxf(mxa, mxb);
      const float m_new = fmaxf(m_ref, mx * scale_log2e);
      // rescale when this row's max has outgrown the reference by more than the step
      // (or when the row sees its first key); the decision is the warp's
      const bool grow = m_new > m_ref + FA_RESCALE_STEP || (m_ref == -INFINITY && m_new > m_ref);
      const bool rescale = __any_sync(0xffffffffu, grow);
      float corr = 1.f;
      if (rescale) {
        corr = m_new == -INFINITY ? 1.f : fa_exp2(m_ref - m_new);
        m_ref = m_new;
        l_run *= corr;
      }
      const float nbase = m_ref == -INFINITY ? 0.f : -m_ref;
      float pk[FA_BN / 2];          // bf16 pairs, as the bit patterns tcgen05.st takes
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
      for (int i = 0; i < FA_BN; i += 4) {
        float a0, a1, a2, a3;
        fa_fma2(a0, a1, sc[i], sc[i + 1], scale_log2e, nbase);   // -inf stays -inf
        fa_fma2(a2, a3, sc[i + 2], sc[i + 3], scale_log2e, nbase);
        const float p0 = fa_exp2(a0), p1 = fa_exp2(a1), p2 = fa_exp2(a2), p3 = fa_exp2(a3);
        fa_add2(sum0, sum1, p0, p1);
        fa_add2(sum2, sum3, p2, p3);
        __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1), v2 = __floats2bfloat162_rn(p2, p3);
        pk[i >> 1] = __uint_as_float(*reinterpret_cast<unsigned*>(&v));
        pk[(i >> 1) + 1] = __uint_as_float(*reinterpret_cast<unsigned*>(&v2));
      }
      const float sum = (sum0 + sum1) + (sum2 + sum3);
      l_run += sum;
      if (j > 0) {
        // O may be touched once the previous P V has completed.  Every phase of this
        // barrier is waited for, in order, also when nothing is rescaled: a parity
        // wait that skipped a phase would take an older completion for the one it wants.
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_done, (j - 1) & 1, abortp));
        if (!ok) break;
        if (rescale) {
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 32) {
            float o[32];
            tc_ld32(lane_addr + c0, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= corr;
            tc_st32(lane_addr + c0, o);
          }
        }
      }
      tc_st32(lane_addr + S_COL + st * FA_BN, pk);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready);
    }
    if (ok && n_tiles > 0)
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_done, (n_tiles - 1) & 1, abortp));
    if (!ok) {
      if (lane == 0 && !*abortp) { atomicExch(status, FA_ERR_SOFTMAX); *abortp = 1; }
    } else if (nsplit > 1) {
      // this run's share: O and the sum as they stand against the reference max, for
      // the merge kernel (a run without keys for a row leaves max = -inf, which the
      // merge skips)
      if (n_tiles > 0) tc_fence_after();
      const size_t hrow = (size_t)(tok0 + q0 + row) * heads + h;
      float* po = part_o + (hrow * nsplit + blockIdx.z) * HD;
      const bool live = n_tiles > 0 && l_run > 0.f;
      if (n_tiles > 0) {
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          float o[32];
          tc_ld32(lane_addr + c0, o);            // every lane takes part in the load
          if (row < rows_valid && live) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(po + c0 + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
          }
        }
      }
      if (row < rows_valid) {
        part_ml[(hrow * nsplit + blockIdx.z) * 2] = live ? m_ref : -INFINITY;
        part_ml[(hrow * nsplit + blockIdx.z) * 2 + 1] = live ? l_run : 0.f;
      }
    } else if (n_tiles > 0) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      bf16* dst = out + ((size_t)(tok0 + q0 + row) * heads + h) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float o[32];
        tc_ld32(lane_addr + c0, o);            // every lane takes part in the load
        if (row < rows_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            unsigned w4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              __nv_bfloat162 v = __floats2bfloat162_rn(o[i + 2 * u] * inv, o[i + 2 * u + 1] * inv);
              w4[u] = *reinterpret_cast<unsigned*>(&v);
            }
            *reinterpret_cast<uint4*>(dst + c0 + i) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abortp && tid == 0) {
    // let copies in flight land before shared memory is given up
    mbar_drain(&bars->q_full, 0);
    for (int i = 0; i < 2; ++i) {
      mbar_drain(&bars->k_full[i], 0);
      mbar_drain(&bars->k_full[i], 1);
      mbar_drain(&bars->v_full[i], 0);
      mbar_drain(&bars->v_full[i], 1);
    }
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// Merge of the runs' shares: out = sum_j o_j 2^(m_j - M) / sum_j l_j 2^(m_j - M), one
// block per (query, head).
__global__ void attn_prefill_tc_merge_kernel(const float* __restrict__ part_o,
                                             const float* __restrict__ part_ml,
                                             bf16* __restrict__ out, int hd, int nsplit) {
  const size_t hrow = blockIdx.x;
  const float* ml = part_ml + hrow * nsplit * 2;
  float M = -INFINITY;
  for (int j = 0; j < nsplit; ++j) M = fmaxf(M, ml[2 * j]);
  float L = 0.f;
  for (int j = 0; j < nsplit; ++j)
    if (ml[2 * j] != -INFINITY) L += ml[2 * j + 1] * fa_exp2(ml[2 * j] - M);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int j = 0; j < nsplit; ++j)
      if (ml[2 * j] != -INFINITY)
        o += part_o[(hrow * nsplit + j) * hd + d] * fa_exp2(ml[2 * j] - M);
    out[hrow * hd + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
  }
}

template <int HD>
static int launch_prefill_tc(const void* q, const void* kc, const void* vc, long long cache_rows,
                             const int* bt, const int* cu_q, const int* q_pos0, void* out, int T,
                             int S, int heads, int kvh, int page_size, int page_shift, int maxb,
                             int window, float scale, int* status, int nsplit, float* part_o,
                             float* part_ml, cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_v;
  int rc = ix_tensor_map_bf16_2d(&map_q, q, T, (long long)heads * HD, 64, FA_BM);
  if (rc != IX_OK) return rc;
  rc = ix_tensor_map_bf16_2d(&map_k, kc, cache_rows, HD, 64, page_size);
  if (rc != IX_OK) return rc;
  rc = ix_tensor_map_bf16_2d(&map_v, vc, cache_rows, HD, 64, page_size);
  if (rc != IX_OK) return rc;
  const int smem = FA_BM * HD * 2 + 4 * FA_BN * HD * 2 + (int)sizeof(FaBars);
  auto kern = attn_prefill_tc_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles = (T + FA_BM - 1) / FA_BM + S;   // every sequence can add one partial tile
  if (tiles > 65535) return IX_ERR_SIZE;
  dim3 grid(heads, tiles, nsplit);
  kern<<<grid, FA_THREADS, smem, stream>>>(map_q, map_k, map_v, bt, cu_q, q_pos0, (bf16*)out, S,
                                           heads, kvh, page_size, page_shift, maxb, window,
                                           scale * 1.4426950408889634f, status, nsplit, part_o,
                                           part_ml);
  rc = ix_launch_status();
  if (rc != IX_OK || nsplit == 1) return rc;
  attn_prefill_tc_merge_kernel<<<T * heads, HD >= 128 ? 128 : 64, 0, stream>>>(
      part_o, part_ml, (bf16*)out, HD, nsplit);
  return ix_launch_status();
}

// Runs to cut every query tile's keys into: only when the step has so few (query tile,
// head) items that they leave SMs idle (a short prompt portion over a long context),
// and never runs shorter than 2,048 keys (the merge is a launch and a pass over fp32
// partial outputs of its own; measured at 16 heads of 128: 512 queries over 8,192 keys
// 129 -> 55 us, over 32,768 keys 506 -> 160 us, 128 queries over 8,192 keys 123 -> 31 us
// with more and shorter runs).  `keys` bounds the longest context of the step.
IX_API int ix_attn_prefill_tc_splits(int T, int S, int heads, int keys, int window) {
  if (T <= 0 || S <= 0 || heads <= 0 || keys <= 0) return 1;
  const long long items = (long long)heads * ((T + FA_BM - 1) / FA_BM + S - 1);
  long long k = keys;
  if (window > 0 && k > (long long)window + FA_BM + FA_BN) k = window + FA_BM + FA_BN;
  const long long by_items = (2 * 148) / (items > 0 ? items : 1);
  const long long by_keys = k / (32 * FA_BN);
  long long n = by_items < by_keys ? by_items : by_keys;
  if (n > 16) n = 16;
  return n < 1 ? 1 : (int)n;
}

// q: [T, heads, hd] bf16; caches [num_pages, kvh, page_size, hd] bf16; status: one int
// in device memory, zero before the first call.  splits > 1: part_o [T, heads, splits,
// hd] and part_ml [T, heads, splits, 2] fp32 scratch.
IX_API int ix_paged_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache,
                                         int num_pages, const int* block_table, const int* cu_q,
                                         const int* q_pos0, void* out, int T, int S, int heads,
                                         int kvh, int hd, int page_size, int max_blocks,
                                         int window, float scale, int splits, float* part_o,
                                         float* part_ml, int* status, cudaStream_t stream) {
  if (T <= 0 || S <= 0) return IX_OK;
  if (heads <= 0 || kvh <= 0 || heads % kvh != 0 || max_blocks <= 0 || window < 0 ||
      num_pages <= 0 || status == nullptr)
    return IX_ERR_SIZE;
  if (heads > 65535) return IX_ERR_SIZE;
  if (splits < 1 || splits > 64 || (splits > 1 && (!part_o || !part_ml))) return IX_ERR_SIZE;
  if (!(hd == 64 || hd == 128) ||
      !(page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64))
    return IX_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out |
       (uintptr_t)part_o) & 15)
    return IX_ERR_ALIGN;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const long long cache_rows = (long long)num_pages * kvh * page_size;
  if (cache_rows > 0x7fffffffLL) return IX_ERR_SIZE;
  if (hd == 128)
    return launch_prefill_tc<128>(q, k_cache, v_cache, cache_rows, block_table, cu_q, q_pos0, out,
                                  T, S, heads, kvh, page_size, page_shift, max_blocks, window,
                                  scale, status, splits, part_o, part_ml, stream);
  return launch_prefill_tc<64>(q, k_cache, v_cache, cache_rows, block_table, cu_q, q_pos0, out, T,
                               S, heads, kvh, page_size, page_shift, max_blocks, window, scale,
                               status, splits, part_o, part_ml, stream);
}
