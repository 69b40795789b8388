// FlashAttention forward for sm_100a (B200), head dim 64, bf16 in / fp32 accumulate / bf16 out.
//
// One CTA owns 256 consecutive query rows of one (batch, head): two 128-row Q tiles ("stages")
// that share every K/V tile the CTA streams through shared memory.
//
//   warp 10             TMA producer: Q tiles once, then K_j, V_j into a ring of 16 KB slots,
//                       128-byte swizzle, completion on mbarriers (no multicast).
//   warp 8 / warp 9     tcgen05 issuer for stage 0 / 1: S_s = Q_s K_j^T (M128 N128 K64, both
//                       operands in shared memory) and O_s += P_s V_j (M128 N64 K128, P read from
//                       tensor memory, V MN-major from shared memory).  Control flow is
//                       warp-uniform; one elected lane issues, tcgen05.commit signals mbarriers.
//   warps 0-3 / 4-7     softmax warpgroup for stage 0 / 1: one thread per query row.  Pulls its S
//                       row from TMEM into registers and releases S at once, so the issuer can
//                       start S for the next K tile while this one is exponentiated; keeps the
//                       running max and sum; writes P (bf16) to its own TMEM columns; rescales O
//                       in TMEM only when the running max grew by more than 2^8; finally writes
//                       O / l and the log-sum-exp.
//
// TMEM columns (32-bit, 128 lanes), all 512 in use:
//   S0 [0,128)  S1 [128,256)  P0 [256,320)  P1 [320,384)  O0 [384,448)  O1 [448,512)
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
constexpr int kHalfN = kBlockN / 2;    // S columns per softmax thread
constexpr int kNumSoftmaxWarps = 16;   // warps 0-7: stage 0 (columns 0-63, 64-127); warps 8-15: stage 1
constexpr int kMmaWarp0 = 16;          // warps 16, 17: tcgen05 issuers of stage 0, 1
constexpr int kLoadWarp = 18;          // warp 19 idles (setmaxnreg needs whole warpgroups)
constexpr int kNumThreads = 640;
// setmaxnreg.inc can only take registers that this CTA's own setmaxnreg.dec released (it blocks,
// without a time limit, until they exist), so the budget after the exchange must not exceed what
// the CTA was launched with: 640 threads x 96 registers.
constexpr int kLaunchRegs = 96;
constexpr int kSoftmaxRegs = 112;
constexpr int kOtherRegs = 32;
static_assert(kNumSoftmaxWarps * 32 * kSoftmaxRegs + (kNumThreads - kNumSoftmaxWarps * 32) * kOtherRegs <=
                  kNumThreads * kLaunchRegs,
              "setmaxnreg budget exceeds the launch allocation: the kernel would hang");
constexpr uint32_t kTmemCols = 512;
__host__ __device__ constexpr uint32_t tmem_col_s(int s) { return 128u * s; }
__host__ __device__ constexpr uint32_t tmem_col_p(int s) { return 256u + 64u * s; }
__host__ __device__ constexpr uint32_t tmem_col_o(int s) { return 384u + 64u * s; }
constexpr float kRescaleThresholdLog2 = 8.0f;
constexpr float kRoundBiasLog2 = 0.0028150156f;   // log2(1 + 2^-9)
// Which of every 8 consecutive exponentials are evaluated by the FMA-pipe polynomial instead of
// the MUFU ex2 unit (bit i set: element with k % 8 == i).  The two pipes run side by side.
#ifndef FA_POLY_MASK
#define FA_POLY_MASK 0x00
#endif
constexpr uint32_t kPolyMask = FA_POLY_MASK;
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait

// watchdog codes (status word 0); low byte tells which wait ran out
constexpr uint32_t kWatchdogBase = 0x10000u;
enum WaitId : uint32_t {
  kWaitQFull = 1, kWaitKVFull = 2, kWaitKVEmpty = 3, kWaitSFull = 4, kWaitPFull = 5,
  kWaitOFull = 6, kWaitDrain = 7, kWaitSFree = 8, kWaitExchange = 9, kWaitExpTurn = 10
};

struct __align__(1024) SharedStorage {
  uint8_t q[2][kTileBytes];
  uint8_t kv[kKVSlots][kTileBytes];
  uint64_t q_full[2];
  uint64_t kv_full[kKVSlots];
  uint64_t kv_empty[kKVSlots];   // one release per active stage issuer
  uint64_t s_full[2];            // S_s written by the tensor core
  uint64_t s_free[2];            // S_s copied to registers by all four softmax warps
  uint64_t p_full[2];            // P_s written to TMEM by all four softmax warps
  uint64_t o_full[2];            // O_s += P_s V_j finished (P_s reusable, O_s stable)
  uint64_t x_ready[2];           // both halves of every row of stage s have posted to xchg
  uint64_t exp_turn[2];          // stage s may run its exponentials (the other stage finished its own)
  float xchg[2][2][2 * kBlockM]; // [stage][parity][half * 128 + row]: half-row max (or sum)
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

// Optional timeline trace (compile with -DFA_TRACE): the CTA named by g_fa_trace_block stores
// clock64() stamps of its role hand-offs; read back with fa_b200_trace_read().  Not compiled
// into the product library.
#ifdef FA_TRACE
constexpr int kTraceSlots = 8192;
__device__ unsigned long long g_fa_trace[kTraceSlots];
__device__ int g_fa_trace_block = 0;
// layout: role r (0,1 = softmax stage 0/1, first half; 2,3 = issuer stage 0/1), iteration j (< 64), event e (< 16)
#define FA_TRACE_EVENT(role, j, e)                                                   \
  do {                                                                               \
    if (blockIdx.x == g_fa_trace_block && (j) < 64)                                  \
      g_fa_trace[((role) * 64 + (j)) * 16 + (e)] = clock64();                        \
  } while (0)
#else
#define FA_TRACE_EVENT(role, j, e) do {} while (0)
#endif

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
// The same for a whole converged warp: every lane polls, the verdict is made uniform.
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity, const Watch& w,
                                              uint32_t id) {
  return __all_sync(0xffffffffu, wait_bar(bar, parity, w, id));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Two floats -> packed bf16 pair by truncation (one byte-permute on the integer pipe; the bf16
// convert instruction shares the MUFU pipe with ex2, which is the kernel's bottleneck).
__device__ __forceinline__ uint32_t pack_bf16_trunc(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}

// 2^x on the FMA pipe: split x into a rounded integer part (added to the exponent field) and a
// fraction in [-0.5, 0.5] fed to a degree-3 minimax polynomial (max relative error 7.5e-5, well
// below the 2^-9 of the bf16 value it becomes).  x is clamped at -126, so 2^-inf comes out as
// 2^-126 instead of 0.
__device__ __forceinline__ float exp2_poly(float x) {
  constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: x + kMagic holds round(x) in its low bits
  x = fmaxf(x, -126.0f);
  const float t = x + kMagic;
  const float xf = x - (t - kMagic);
  float pl = fmaf(0.0551716685f, xf, 0.2426111251f);
  pl = fmaf(pl, xf, 0.6932609677f);
  pl = fmaf(pl, xf, 0.9999280572f);
  return __uint_as_float(__float_as_uint(pl) + (__float_as_uint(t) << 23));
}
// `use_poly` is a compile-time constant at every call site once the loops are unrolled.
__device__ __forceinline__ float exp2_sel(bool use_poly, float x) {
  return use_poly ? exp2_poly(x) : ex2_approx(x);
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
      mbar_init(smem_u32(&sm.s_free[s]), 8);
      mbar_init(smem_u32(&sm.p_full[s]), 8);
      mbar_init(smem_u32(&sm.o_full[s]), 1);
      mbar_init(smem_u32(&sm.x_ready[s]), 8);
      mbar_init(smem_u32(&sm.exp_turn[s]), 8);
    }
    for (int i = 0; i < kKVSlots; ++i) {
      mbar_init(smem_u32(&sm.kv_full[i]), 1);
      mbar_init(smem_u32(&sm.kv_empty[i]), n_tiles[1] > 0 ? 2 : 1);  // one release per active stage
    }
    sm.abort = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp0) {
    tmem_alloc(smem_u32(&sm.tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  const Watch watch{&sm.abort, p.status};

  auto slot_of = [](int it) { return it % kKVSlots; };
  auto par_of = [](int it) { return static_cast<uint32_t>((it / kKVSlots) & 1); };

  // Register budget: the four softmax warpgroups take 112 registers per thread, the warpgroup
  // that holds the issuers and the producer gives up what it does not need.  Each setmaxnreg is
  // executed by all four warps of its warpgroup from one place.
  if (warp >= kNumSoftmaxWarps) {
  reg_dealloc<kOtherRegs>();
  if (warp == kLoadWarp) {
    // =================================================================== TMA producer
    // ring order: K_0 V_0 K_1 V_1 ...  (K_j is load 2j, V_j is load 2j+1)
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
    }
    bool ok = true;
    int it = 0;
    auto load_kv = [&](const CUtensorMap* map, int j) {
      const int slot = slot_of(it);
      const int use = it / kKVSlots;
      if (use > 0 && ok)
        ok = wait_bar_warp(smem_u32(&sm.kv_empty[slot]), (use - 1) & 1, watch, kWaitKVEmpty);
      if (ok) {
        if (elect_one()) {
          const uint32_t bar = smem_u32(&sm.kv_full[slot]);
          mbar_arrive_expect_tx(bar, kTileBytes);
          tma_load_4d(smem_u32(sm.kv[slot]), map, bar, 0, j * kBlockN, h, b);
        }
        ++it;
      }
    };
    auto load_q = [&](int s) {
      if (elect_one()) {
        const uint32_t bar = smem_u32(&sm.q_full[s]);
        mbar_arrive_expect_tx(bar, kTileBytes);
        tma_load_4d(smem_u32(sm.q[s]), &tmap_q, bar, 0, q_row[s], h, b);
      }
    };
    load_q(0);
    load_kv(&tmap_k, 0);
    if (n_tiles[1] > 0) load_q(1);
    load_kv(&tmap_v, 0);
    for (int j = 1; j < nmax && ok; ++j) {
      load_kv(&tmap_k, j);
      load_kv(&tmap_v, j);
    }
    if (sm.abort && lane == 0) {
      // leave no copy of ours in flight: wait (bounded) for every load still armed
      for (int i = max(0, it - kKVSlots); i < it; ++i)
        wait_bar(smem_u32(&sm.kv_full[slot_of(i)]), par_of(i), watch, kWaitDrain,
                 20ull * 1000 * 1000, false);
      wait_bar(smem_u32(&sm.q_full[0]), 0, watch, kWaitDrain, 20ull * 1000 * 1000, false);
      if (n_tiles[1] > 0)
        wait_bar(smem_u32(&sm.q_full[1]), 0, watch, kWaitDrain, 20ull * 1000 * 1000, false);
    }
    __syncwarp();
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // =================================================================== tcgen05 issuer, stage s
    const int s = warp - kMmaWarp0;
    const int ns = n_tiles[s];
    constexpr uint32_t idesc_s = make_idesc_bf16(kBlockM, kBlockN, false);
    constexpr uint32_t idesc_o = make_idesc_bf16(kBlockM, kHeadDim, true);
    const uint64_t desc_q = make_sw128_desc(smem_u32(sm.q[s]));
    const uint32_t t_s = tmem_base + tmem_col_s(s);
    const uint32_t t_p = tmem_base + tmem_col_p(s);
    const uint32_t t_o = tmem_base + tmem_col_o(s);
    const uint32_t bar_s_full = smem_u32(&sm.s_full[s]);
    const uint32_t bar_o_full = smem_u32(&sm.o_full[s]);

    // S_s = Q_s K^T from ring slot `slot`, then release that slot (for this stage)
    auto issue_s = [&](int slot) {
      if (elect_one()) {
        const uint64_t dk = make_sw128_desc(smem_u32(sm.kv[slot]));
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)  // +32 bytes along the row per K=16 step
          umma_ss(t_s, desc_q + 2 * kk, dk + 2 * kk, idesc_s, kk > 0);
        tc_commit(bar_s_full);
        tc_commit(smem_u32(&sm.kv_empty[slot]));
      }
      __syncwarp();
    };
    auto issue_pv = [&](int slot, bool first) {
      if (elect_one()) {
        const uint64_t dv = make_sw128_desc(smem_u32(sm.kv[slot]));
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk)  // 16 V rows = 2048 bytes; 16 P values = 8 columns
          umma_ts(t_o, t_p + 8 * kk, dv + 128 * kk, idesc_o, (!first) || kk > 0);
        tc_commit(bar_o_full);
        tc_commit(smem_u32(&sm.kv_empty[slot]));
      }
      __syncwarp();
    };
    // A tile only the other stage needs.  Released with a commit, not a plain arrive, so that it
    // cannot overtake this thread's earlier (asynchronous) commit on the same slot.
    auto release_unused = [&](int slot) {
      if (elect_one()) tc_commit(smem_u32(&sm.kv_empty[slot]));
      __syncwarp();
    };

    bool ok = true;
    if (ns > 0) {
      ok = wait_bar_warp(smem_u32(&sm.q_full[s]), 0, watch, kWaitQFull) &&
           wait_bar_warp(smem_u32(&sm.kv_full[0]), 0, watch, kWaitKVFull);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
    }
    for (int j = 0; j < nmax && ok && ns > 0; ++j) {
      const int itv = 2 * j + 1, itk = 2 * j + 2;
      // ---- S for the next K tile, as soon as the softmax warps hold S(j) in registers
      if (j + 1 < nmax) {
        if (j + 1 < ns) {
          FA_TRACE_EVENT(2 + s, j, 0);
          ok = wait_bar_warp(smem_u32(&sm.kv_full[slot_of(itk)]), par_of(itk), watch, kWaitKVFull) &&
               wait_bar_warp(smem_u32(&sm.s_free[s]), j & 1, watch, kWaitSFree);
          if (!ok) break;
          FA_TRACE_EVENT(2 + s, j, 1);
          tc_fence_after();
          issue_s(slot_of(itk));
          FA_TRACE_EVENT(2 + s, j, 2);
        } else {
          release_unused(slot_of(itk));
        }
      }
      // ---- O += P V for this tile
      if (j < ns) {
        FA_TRACE_EVENT(2 + s, j, 3);
        ok = wait_bar_warp(smem_u32(&sm.kv_full[slot_of(itv)]), par_of(itv), watch, kWaitKVFull) &&
             wait_bar_warp(smem_u32(&sm.p_full[s]), j & 1, watch, kWaitPFull);
        if (!ok) break;
        FA_TRACE_EVENT(2 + s, j, 4);
        tc_fence_after();
        issue_pv(slot_of(itv), j == 0);
        FA_TRACE_EVENT(2 + s, j, 5);
      } else {
        release_unused(slot_of(itv));
      }
    }
  }
  } else {
    // =================================================================== softmax warpgroups
    reg_alloc<kSoftmaxRegs>();
    // Stage s is served by two warpgroups; each thread owns HALF a query row (64 of the 128
    // columns of S).  Four softmax warps per SM sub-partition keep the pipes fed while others
    // sit in TMEM-load, barrier or store latency.
    const int s = warp >> 3;                    // which Q tile
    const int hf = (warp >> 2) & 1;             // which column half
    const int r = (warp & 3) * 32 + lane;       // row inside the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + lane_base + tmem_col_s(s) + 64 * hf;
    const uint32_t t_p = tmem_base + lane_base + tmem_col_p(s) + 32 * hf;
    const uint32_t t_o = tmem_base + lane_base + tmem_col_o(s) + 32 * hf;
    const int ns = n_tiles[s];
    const float c = p.scale_log2;
    const uint32_t bar_s_full = smem_u32(&sm.s_full[s]);
    const uint32_t bar_s_free = smem_u32(&sm.s_free[s]);
    const uint32_t bar_p = smem_u32(&sm.p_full[s]);
    const uint32_t bar_o = smem_u32(&sm.o_full[s]);
    const uint32_t bar_x = smem_u32(&sm.x_ready[s]);
    // The exponentials are bound by the MUFU unit; everything around them (TMEM loads, the max
    // exchange, barrier waits, TMEM stores) is latency.  Left alone, the two stages fall into
    // step and the MUFU idles during the latency phases of both.  They therefore take turns --
    // stage 0 tile j, stage 1 tile j, stage 0 tile j+1, ... -- so that one stage's latency
    // phases run under the other stage's exponentials.
#ifndef FA_NO_TURNS
    const bool take_turns = n_tiles[0] > 0 && n_tiles[1] > 0;
#else
    const bool take_turns = false;
#endif
    const uint32_t bar_my_turn = smem_u32(&sm.exp_turn[s]);
    const uint32_t bar_other_turn = smem_u32(&sm.exp_turn[s ^ 1]);
    constexpr uint32_t kNegInf = 0xff800000u;
#ifdef FA_TRACE
    const bool tracer = r == 0 && hf == 0;
#endif

    float m_ref = -CUDART_INF_F;  // max the exponentials are currently taken against (raw scores)
    float l = 0.f;                // this half's running sum of exp2((s - m_ref) * c)
    bool ok = true;

    for (int j = 0; j < ns; ++j) {
#ifdef FA_TRACE
      if (tracer) FA_TRACE_EVENT(s, j, 0);
#endif
      ok = wait_bar_warp(bar_s_full, j & 1, watch, kWaitSFull);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[kHalfN];
      tmem_ld_x64(t_s, sv);
      // S is in registers: let the issuer overwrite it with the next tile's scores
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_s_free);

      const int col0 = j * kBlockN + kHalfN * hf;   // first key index of this half-tile
      if (p.causal) {
        if (j * kBlockN == q_row[s]) {  // the diagonal tile: key col0+k is visible to row r iff <= r
          const int lim = r - kHalfN * hf;
#pragma unroll
          for (int k = 0; k < kHalfN; ++k)
            if (k > lim) sv[k] = kNegInf;
        }
      } else if (col0 + kHalfN > p.N) {  // ragged last tile: TMA zero-fill gives score 0, not -inf
        const int lim = p.N - col0;
#pragma unroll
        for (int k = 0; k < kHalfN; ++k)
          if (k >= lim) sv[k] = kNegInf;
      }

      float mx[2];
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {   // two independent chains of 32
        const int o = 32 * ch;
        float m = fmax3(__uint_as_float(sv[o]), __uint_as_float(sv[o + 1]), __uint_as_float(sv[o + 2]));
#pragma unroll
        for (int k = 3; k + 1 < 32; k += 2)
          m = fmax3(m, __uint_as_float(sv[o + k]), __uint_as_float(sv[o + k + 1]));
        mx[ch] = fmaxf(m, __uint_as_float(sv[o + 31]));
      }
      // exchange the half-row maxima with the thread that owns the other half of this row
      float* xbuf = sm.xchg[s][j & 1];
      xbuf[hf * kBlockM + r] = fmaxf(mx[0], mx[1]);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_x);
      ok = wait_bar_warp(bar_x, j & 1, watch, kWaitExchange);
      if (!ok) break;
      const float m_new = fmax3(fmaxf(mx[0], mx[1]), xbuf[(hf ^ 1) * kBlockM + r], m_ref);

      if (j == 0) {
        m_ref = m_new;
      } else {
        // O += P V of the previous tile must be finished before P is overwritten or O is touched
        ok = wait_bar_warp(bar_o, (j - 1) & 1, watch, kWaitOFull);
        if (!ok) break;
        // Rescale lazily: while the max grew by less than 2^8 keep the old reference; P stays
        // below 256 and the final O / l is exact because O, l and P share one reference.
        // m_new is identical in both halves of a row, so both take the same decision; each
        // half rescales its own 32 columns of O.
        const bool need = (m_new - m_ref) * c > kRescaleThresholdLog2;
        if (__any_sync(0xffffffffu, need)) {
          const float f = need ? ex2_approx((m_ref - m_new) * c) : 1.0f;
          tc_fence_after();
          uint32_t ov[32];
          tmem_ld_x32(t_o, ov);
#pragma unroll
          for (int k = 0; k < 32; ++k) ov[k] = __float_as_uint(__uint_as_float(ov[k]) * f);
          tmem_st_x32(t_o, ov);
          l *= f;
          if (need) m_ref = m_new;
        }
      }

      if (take_turns && (s == 1 ? j < n_tiles[0] : j > 0)) {
        // stage 1 tile j follows stage 0 tile j; stage 0 tile j follows stage 1 tile j-1.  Each
        // posted phase is waited for before the next can be posted (a tile stage 0 does not have
        // is simply not waited for), so no waiter ever lags two phases behind its barrier.
        ok = wait_bar_warp(bar_my_turn, (s == 1 ? j : j - 1) & 1, watch, kWaitExpTurn);
        if (!ok) break;
      }
#ifdef FA_TRACE
      if (tracer) FA_TRACE_EVENT(s, j, 1);
#endif
      const float neg_mc = -m_ref * c;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {   // 32 scores -> 16 packed registers -> one TMEM store
        uint32_t pk[16];
#pragma unroll
        for (int k = 0; k < 32; k += 4) {
          const int o = 32 * ch + k;
          const float p0 = exp2_sel(((kPolyMask >> ((k + 0) & 7)) & 1u) != 0u, fmaf(__uint_as_float(sv[o + 0]), c, neg_mc));
          const float p1 = exp2_sel(((kPolyMask >> ((k + 1) & 7)) & 1u) != 0u, fmaf(__uint_as_float(sv[o + 1]), c, neg_mc));
          const float p2 = exp2_sel(((kPolyMask >> ((k + 2) & 7)) & 1u) != 0u, fmaf(__uint_as_float(sv[o + 2]), c, neg_mc));
          const float p3 = exp2_sel(((kPolyMask >> ((k + 3) & 7)) & 1u) != 0u, fmaf(__uint_as_float(sv[o + 3]), c, neg_mc));
          l0 += p0; l1 += p1; l2 += p2; l3 += p3;
          pk[k / 2 + 0] = pack_bf16(p0, p1);
          pk[k / 2 + 1] = pack_bf16(p2, p3);
        }
        tmem_st_x16(t_p + 16 * ch, pk);
      }
      l += (l0 + l1) + (l2 + l3);
#ifdef FA_TRACE
      if (tracer) FA_TRACE_EVENT(s, j, 2);
#endif
      if (take_turns) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_other_turn);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
    }

    // ---- epilogue: O / l -> bf16, LSE
    if (ok && ns > 0) {
      // total row sum = this half's + the other half's (one more round of the exchange barrier)
      float* xbuf = sm.xchg[s][ns & 1];
      xbuf[hf * kBlockM + r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_x);
      ok = wait_bar_warp(bar_x, ns & 1, watch, kWaitExchange) &&
           wait_bar_warp(bar_o, (ns - 1) & 1, watch, kWaitOFull);
      if (ok) {
        l += xbuf[(hf ^ 1) * kBlockM + r];
        tc_fence_after();
        const int row = q_row[s] + r;
        const float inv_l = 1.0f / l;
        __nv_bfloat16* orow = p.o + (long long)b * p.o_sb + (long long)h * p.o_sh +
                              (long long)row * p.o_sn + 32 * hf;
        uint32_t ov[32];
        tmem_ld_x32(t_o, ov);
        if (row < p.N) {
#pragma unroll
          for (int k = 0; k < 32; k += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(ov[k + 0]) * inv_l, __uint_as_float(ov[k + 1]) * inv_l);
            w.y = pack_bf16(__uint_as_float(ov[k + 2]) * inv_l, __uint_as_float(ov[k + 3]) * inv_l);
            w.z = pack_bf16(__uint_as_float(ov[k + 4]) * inv_l, __uint_as_float(ov[k + 5]) * inv_l);
            w.w = pack_bf16(__uint_as_float(ov[k + 6]) * inv_l, __uint_as_float(ov[k + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + k) = w;
          }
          if (p.lse != nullptr && hf == 0) {
            // ln(sum_j exp(scale * s_j)) = ln2 * (m_ref * c + log2(l))
            p.lse[((long long)b * p.H + h) * p.N + row] = 0.6931471805599453f * (m_ref * c + log2f(l));
          }
        }
      }
    }
  }

  // ---- teardown: every TMEM access above is complete (loads waited, MMAs observed via o_full)
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fa
