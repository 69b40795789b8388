// FlashAttention forward for sm_100a (B200), head dim 64, bf16 in / fp32 accumulate / bf16 out.
//
// One CTA owns 256 consecutive query rows of one (batch, head): two 128-row Q tiles ("stages")
// that share every K/V tile the CTA streams through shared memory.
//
//   warp 9 (1 thread)   TMA producer: Q tiles once, then K_j, V_j into a ring of 16 KB slots,
//                       128-byte swizzle, completion on mbarriers (no multicast).
//   warp 8 (1 thread)   tcgen05 issuer: S_s = Q_s K_j^T (M128 N128 K64, both operands in shared
//                       memory) and O_s += P_s V_j (M128 N64 K128, P read from tensor memory,
//                       V MN-major from shared memory); tcgen05.commit signals the mbarriers.
//   warps 0-3 / 4-7     softmax warpgroup for stage 0 / 1: one thread per query row.  Reads its S
//                       row from TMEM, keeps the running max and sum, writes P (bf16) back over S
//                       in TMEM, rescales O in TMEM when the running max grew by more than 2^8,
//                       and finally writes O / l and the log-sum-exp.
//
// TMEM columns (fp32, 128 lanes): S0 [0,128)  S1 [128,256)  O0 [256,320)  O1 [320,384);
// P_s (bf16 pairs) overlays the first 64 columns of S_s.
//
// Every mbarrier wait is bounded: a wait that exceeds kWaitLimitNs records a code in the status
// word, raises the CTA's abort flag, and every role drains and leaves through the normal exit
// (TMEM is freed).  Nothing traps and nothing spins without a limit.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <math_constants.h>

#include "ptx_sm100.cuh"
#include "tmem_ops_gen.cuh"

namespace fa {

constexpr int kBlockM = 128;           // query rows per tile
constexpr int kBlockN = 128;           // key/value rows per tile
constexpr int kHeadDim = 64;           // fixed, as in the reference (common_types.hpp:33)
constexpr int kTileBytes = kBlockN * kHeadDim * 2;
constexpr int kKVSlots = 6;            // ring: K0 V0 K1 V1 ...
constexpr int kMmaWarp = 8;
constexpr int kLoadWarp = 9;
constexpr int kNumThreads = 320;
constexpr uint32_t kTmemCols = 512;
__host__ __device__ constexpr uint32_t tmem_col_s(int s) { return s ? 128u : 0u; }    // S_s / P_s
__host__ __device__ constexpr uint32_t tmem_col_o(int s) { return s ? 320u : 256u; }  // O_s
constexpr float kRescaleThresholdLog2 = 8.0f;
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait

// watchdog codes (status word 0); low byte tells which wait ran out
constexpr uint32_t kWatchdogBase = 0x10000u;
enum WaitId : uint32_t {
  kWaitQFull = 1, kWaitKVFull = 2, kWaitKVEmpty = 3, kWaitSFull = 4, kWaitPFull = 5,
  kWaitOFull = 6, kWaitDrain = 7
};

struct __align__(1024) SharedStorage {
  uint8_t q[2][kTileBytes];
  uint8_t kv[kKVSlots][kTileBytes];
  uint64_t q_full[2];
  uint64_t kv_full[kKVSlots];
  uint64_t kv_empty[kKVSlots];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_full[2];
  uint32_t tmem_base;
  uint32_t abort;
};
constexpr int kSmemBytes = sizeof(SharedStorage) + 1024;  // + slack to align the base to 1024

struct FwdParams {
  __nv_bfloat16* o;
  float* lse;                 // may be null
  long long o_sb, o_sh, o_sn; // element strides of O: batch, head, row
  int B, H, N;
  int n_pairs;                // ceil(N / 256): CTAs per (batch, head)
  int causal;
  float scale_log2;           // softmax_scale * log2(e)
  unsigned int* status;       // [4] watchdog words in global memory
};

struct Watch {
  volatile uint32_t* abort;
  unsigned int* status;
};

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const Watch& w,
                                         uint32_t id, uint64_t limit_ns = kWaitLimitNs,
                                         bool heed_abort = true) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t polls = 1; polls < (1u << 26); ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 63u) == 0u) {
      if (heed_abort && *w.abort) return false;
      if (globaltimer_ns() - t0 > limit_ns) break;
    }
  }
  *w.abort = 1;
  if (atomicCAS(w.status, 0u, kWatchdogBase | id) == 0u) {
    w.status[1] = blockIdx.x;
    w.status[2] = threadIdx.x;
    w.status[3] = parity;
  }
  return false;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kNumThreads, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  SharedStorage& sm =
      *reinterpret_cast<SharedStorage*>(smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which rows does this CTA own?  Heaviest (latest) causal row blocks are launched first.
  const int pair_slot = blockIdx.x % p.n_pairs;
  const int bh = blockIdx.x / p.n_pairs;
  const int pr = p.causal ? (p.n_pairs - 1 - pair_slot) : pair_slot;
  const int b = bh / p.H;
  const int h = bh % p.H;
  const int nkv = (p.N + kBlockN - 1) / kBlockN;
  int q_row[2], n_tiles[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    q_row[s] = pr * 2 * kBlockM + s * kBlockM;
    n_tiles[s] = q_row[s] < p.N ? (p.causal ? min(nkv, 2 * pr + s + 1) : nkv) : 0;
  }
  const int nmax = max(n_tiles[0], n_tiles[1]);

  // ---- one-time setup
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&sm.q_full[s]), 1);
      mbar_init(smem_u32(&sm.s_full[s]), 1);
      mbar_init(smem_u32(&sm.p_full[s]), kBlockM);
      mbar_init(smem_u32(&sm.o_full[s]), 1);
    }
    for (int i = 0; i < kKVSlots; ++i) {
      mbar_init(smem_u32(&sm.kv_full[i]), 1);
      mbar_init(smem_u32(&sm.kv_empty[i]), 1);
    }
    sm.abort = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sm.tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  const Watch watch{&sm.abort, p.status};

  if (warp == kLoadWarp) {
    // =================================================================== TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      bool ok = true;
      int it = 0;
      auto load_kv = [&](const CUtensorMap* map, int j) {
        const int slot = it % kKVSlots;
        const int use = it / kKVSlots;
        if (use > 0 && ok)
          ok = wait_bar(smem_u32(&sm.kv_empty[slot]), (use - 1) & 1, watch, kWaitKVEmpty);
        if (ok) {
          const uint32_t bar = smem_u32(&sm.kv_full[slot]);
          mbar_arrive_expect_tx(bar, kTileBytes);
          tma_load_4d(smem_u32(sm.kv[slot]), map, bar, 0, j * kBlockN, h, b);
          ++it;
        }
      };
      auto load_q = [&](int s) {
        const uint32_t bar = smem_u32(&sm.q_full[s]);
        mbar_arrive_expect_tx(bar, kTileBytes);
        tma_load_4d(smem_u32(sm.q[s]), &tmap_q, bar, 0, q_row[s], h, b);
      };
      load_q(0);
      load_kv(&tmap_k, 0);
      if (n_tiles[1] > 0) load_q(1);
      load_kv(&tmap_v, 0);
      for (int j = 1; j < nmax && ok; ++j) {
        load_kv(&tmap_k, j);
        load_kv(&tmap_v, j);
      }
      if (sm.abort) {
        // leave no copy of ours in flight: wait (bounded) for every load still armed
        for (int i = max(0, it - kKVSlots); i < it; ++i)
          wait_bar(smem_u32(&sm.kv_full[i % kKVSlots]), (i / kKVSlots) & 1, watch, kWaitDrain,
                   20ull * 1000 * 1000, false);
        wait_bar(smem_u32(&sm.q_full[0]), 0, watch, kWaitDrain, 20ull * 1000 * 1000, false);
        if (n_tiles[1] > 0)
          wait_bar(smem_u32(&sm.q_full[1]), 0, watch, kWaitDrain, 20ull * 1000 * 1000, false);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // =================================================================== tcgen05 issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kBlockM, kBlockN, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(kBlockM, kHeadDim, true);
      const uint64_t desc_q[2] = {make_sw128_desc(smem_u32(sm.q[0])),
                                  make_sw128_desc(smem_u32(sm.q[1]))};
      auto issue_s = [&](int s, int slot) {
        const uint64_t dk = make_sw128_desc(smem_u32(sm.kv[slot]));
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)  // +32 bytes along the row per K=16 step
          umma_ss(tmem_base + tmem_col_s(s), desc_q[s] + 2 * kk, dk + 2 * kk, idesc_s, kk > 0);
      };
      auto issue_pv = [&](int s, int slot, bool first) {
        const uint64_t dv = make_sw128_desc(smem_u32(sm.kv[slot]));
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk)  // 16 V rows = 2048 bytes; 16 P values = 8 columns
          umma_ts(tmem_base + tmem_col_o(s), tmem_base + tmem_col_s(s) + 8 * kk, dv + 128 * kk, idesc_o,
                  (!first) || kk > 0);
      };
      auto slot_of = [](int it) { return it % kKVSlots; };
      auto par_of = [](int it) { return (uint32_t)((it / kKVSlots) & 1); };

      bool ok = wait_bar(smem_u32(&sm.q_full[0]), 0, watch, kWaitQFull) &&
                wait_bar(smem_u32(&sm.kv_full[0]), 0, watch, kWaitKVFull);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        tc_commit(smem_u32(&sm.s_full[0]));
      }
      if (ok && n_tiles[1] > 0) {
        ok = wait_bar(smem_u32(&sm.q_full[1]), 0, watch, kWaitQFull);
        if (ok) {
          tc_fence_after();
          issue_s(1, 0);
          tc_commit(smem_u32(&sm.s_full[1]));
        }
      }
      if (ok) tc_commit(smem_u32(&sm.kv_empty[0]));

      for (int j = 0; j < nmax && ok; ++j) {
        const int itv = 2 * j + 1, itk = 2 * j + 2;
        const bool has_next = j + 1 < nmax;
        ok = wait_bar(smem_u32(&sm.kv_full[slot_of(itv)]), par_of(itv), watch, kWaitKVFull);
        if (ok && has_next)
          ok = wait_bar(smem_u32(&sm.kv_full[slot_of(itk)]), par_of(itk), watch, kWaitKVFull);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (ok && j < n_tiles[s]) {
            ok = wait_bar(smem_u32(&sm.p_full[s]), j & 1, watch, kWaitPFull);
            if (ok) {
              tc_fence_after();
              issue_pv(s, slot_of(itv), j == 0);
              tc_commit(smem_u32(&sm.o_full[s]));
              if (j + 1 < n_tiles[s]) {
                issue_s(s, slot_of(itk));
                tc_commit(smem_u32(&sm.s_full[s]));
              }
            }
          }
        }
        if (!ok) break;
        tc_commit(smem_u32(&sm.kv_empty[slot_of(itv)]));
        if (has_next) tc_commit(smem_u32(&sm.kv_empty[slot_of(itk)]));
      }
    }
    __syncwarp();
  } else {
    // =================================================================== softmax warpgroups
    const int s = warp >> 2;                 // which Q tile
    const int r = threadIdx.x & (kBlockM - 1);  // row inside the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + lane_base + tmem_col_s(s);
    const uint32_t t_o = tmem_base + lane_base + tmem_col_o(s);
    const int ns = n_tiles[s];
    const float c = p.scale_log2;
    const uint32_t bar_s = smem_u32(&sm.s_full[s]);
    const uint32_t bar_p = smem_u32(&sm.p_full[s]);
    const uint32_t bar_o = smem_u32(&sm.o_full[s]);
    constexpr uint32_t kNegInf = 0xff800000u;

    float m_ref = -CUDART_INF_F;  // max the exponentials are currently taken against (raw scores)
    float l = 0.f;                // running sum of exp2((s - m_ref) * c)
    bool ok = true;

    for (int j = 0; j < ns; ++j) {
      ok = __all_sync(0xffffffffu, wait_bar(bar_s, j & 1, watch, kWaitSFull));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[kBlockN];
      tmem_ld_x128(t_s, sv);

      const int col0 = j * kBlockN;
      if (p.causal) {
        if (col0 == q_row[s]) {  // the diagonal tile: column k is visible to row r iff k <= r
#pragma unroll
          for (int k = 0; k < kBlockN; ++k)
            if (k > r) sv[k] = kNegInf;
        }
      } else if (col0 + kBlockN > p.N) {  // ragged last tile: TMA zero-fill gives score 0, not -inf
        const int lim = p.N - col0;
#pragma unroll
        for (int k = 0; k < kBlockN; ++k)
          if (k >= lim) sv[k] = kNegInf;
      }

      float mx0 = fmax3(__uint_as_float(sv[0]), __uint_as_float(sv[1]), __uint_as_float(sv[2]));
      float mx1 = fmax3(__uint_as_float(sv[3]), __uint_as_float(sv[4]), __uint_as_float(sv[5]));
#pragma unroll
      for (int k = 6; k + 3 < kBlockN; k += 4) {
        mx0 = fmax3(mx0, __uint_as_float(sv[k]), __uint_as_float(sv[k + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sv[k + 2]), __uint_as_float(sv[k + 3]));
      }
      // 6 + 4*30 = 126 consumed; two left
      const float m_new = fmaxf(m_ref, fmax3(fmaxf(mx0, mx1), __uint_as_float(sv[126]),
                                             __uint_as_float(sv[127])));

      if (j == 0) {
        m_ref = m_new;
      } else {
        // Rescale lazily: while the max grew by less than 2^8 keep the old reference; P stays
        // below 256 and the final O / l is exact because O, l and P share one reference.
        const bool need = (m_new - m_ref) * c > kRescaleThresholdLog2;
        if (__any_sync(0xffffffffu, need)) {
          const float f = need ? ex2_approx((m_ref - m_new) * c) : 1.0f;
          ok = __all_sync(0xffffffffu, wait_bar(bar_o, (j - 1) & 1, watch, kWaitOFull));
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t ov[32];
            tmem_ld_x32(t_o + 32 * half, ov);
#pragma unroll
            for (int k = 0; k < 32; ++k) ov[k] = __float_as_uint(__uint_as_float(ov[k]) * f);
            tmem_st_x32(t_o + 32 * half, ov);
          }
          tmem_wait_st();
          l *= f;
          if (need) m_ref = m_new;
        }
      }

      const float neg_mc = -m_ref * c;
      uint32_t pk[kBlockN / 2];
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int k = 0; k < kBlockN; k += 4) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(sv[k + 0]), c, neg_mc));
        const float p1 = ex2_approx(fmaf(__uint_as_float(sv[k + 1]), c, neg_mc));
        const float p2 = ex2_approx(fmaf(__uint_as_float(sv[k + 2]), c, neg_mc));
        const float p3 = ex2_approx(fmaf(__uint_as_float(sv[k + 3]), c, neg_mc));
        l0 += p0; l1 += p1; l2 += p2; l3 += p3;
        pk[k / 2 + 0] = pack_bf16(p0, p1);
        pk[k / 2 + 1] = pack_bf16(p2, p3);
      }
      l += (l0 + l1) + (l2 + l3);
      tmem_st_x64(t_s, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p);
    }

    // ---- epilogue: O / l -> bf16, LSE
    if (ok && ns > 0) {
      ok = __all_sync(0xffffffffu, wait_bar(bar_o, (ns - 1) & 1, watch, kWaitOFull));
      if (ok) {
        tc_fence_after();
        const int row = q_row[s] + r;
        const float inv_l = 1.0f / l;
        __nv_bfloat16* orow = p.o + (long long)b * p.o_sb + (long long)h * p.o_sh +
                              (long long)row * p.o_sn;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t ov[32];
          tmem_ld_x32(t_o + 32 * half, ov);
          if (row < p.N) {
#pragma unroll
            for (int k = 0; k < 32; k += 8) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(ov[k + 0]) * inv_l, __uint_as_float(ov[k + 1]) * inv_l);
              w.y = pack_bf16(__uint_as_float(ov[k + 2]) * inv_l, __uint_as_float(ov[k + 3]) * inv_l);
              w.z = pack_bf16(__uint_as_float(ov[k + 4]) * inv_l, __uint_as_float(ov[k + 5]) * inv_l);
              w.w = pack_bf16(__uint_as_float(ov[k + 6]) * inv_l, __uint_as_float(ov[k + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + 32 * half + k) = w;
            }
          }
        }
        if (p.lse != nullptr && row < p.N) {
          // ln(sum_j exp(scale * s_j)) = ln2 * (m_ref * c + log2(l))
          p.lse[((long long)b * p.H + h) * p.N + row] =
              0.6931471805599453f * (m_ref * c + log2f(l));
        }
      }
    }
  }

  // ---- teardown: every TMEM access above is complete (loads waited, MMAs observed via o_full)
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fa
