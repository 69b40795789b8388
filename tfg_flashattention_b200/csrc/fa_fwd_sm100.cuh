// FlashAttention forward for sm_100a (B200), head dim 64, bf16 in / fp32 accumulate / bf16 out.
//
// A work item is one 128-row query tile of one (batch, head); the CTA streams that head's K/V
// tiles through shared memory.  Two CTAs are resident per SM (each takes 256 of the 512 TMEM
// columns, under half the shared memory and half the registers), so one CTA's latency-bound
// phases run under the other CTA's tensor-core and MUFU work.  The grid is either one CTA per
// item or persistent (2 x SM count CTAs striding through a load-balanced item list); in the
// persistent case every role runs ahead across item boundaries: the producer loads the next
// item's Q/K/V, the issuer starts its first S, and the softmax warps run an item's epilogue in
// the middle of the next item's first tile, when the last O += P V has long completed.
//
//   warpgroup 1, warp 5   TMA producer: Q, then K_j, V_j into a ring of 16 KB slots, 128-byte
//                         swizzle, completion on mbarriers (no multicast).
//   warpgroup 1, warp 4   tcgen05 issuer: S = Q K_j^T (M128 N128 K64, both operands in shared
//                         memory) and O += P V_j (M128 N64 K128, P read from tensor memory, V
//                         MN-major from shared memory).  Control flow is warp-uniform; one
//                         elected lane issues, tcgen05.commit signals the mbarriers.
//                         (warps 6, 7 idle: setmaxnreg works on whole warpgroups.)
//   warpgroup 0           softmax, one thread per query row.  Pulls its S row from TMEM into
//                         registers and releases S at once, so the issuer can start S for the
//                         next K tile while this one is exponentiated; keeps the running max and
//                         sum (scaling and sums as packed f32x2 operations; 2 of every 8
//                         exponentials as a cubic on the FMA pipe, the rest on the MUFU: d = 64
//                         is exponential-bound before it is MMA-bound);
//                         writes P (bf16) to its own TMEM columns; rescales O in TMEM only
//                         when the running max grew by more than 2^8; epilogue: O / l -> bf16 ->
//                         swizzled shared-memory tile -> TMA store, and the LSE.
//
// TMEM columns (32-bit, 128 lanes):  S [0,128)  P [128,192)  O [192,256)
//
// Every mbarrier wait is bounded: a wait that exceeds kWaitLimitNs records a code in the status
// word, raises the CTA's abort flag, and every role drains and leaves through the normal exit
// (TMEM is freed).  Nothing traps and nothing spins without a limit.  The one hardware wait
// without a limit, setmaxnreg.inc, is made safe by the static register budget below.
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
constexpr int kKVSlots = 4;            // ring: K0 V0 K1 V1 ..., continuing across work items
constexpr int kNumSoftmaxWarps = 4;
constexpr int kMmaWarp = 4;
constexpr int kLoadWarp = 5;
constexpr int kNumThreads = 256;       // two whole warpgroups
constexpr int kCtasPerSm = 2;
constexpr int kSmCountHint = 148;      // B200; only decorrelates the schedules of co-resident CTAs
// Register budget.  Two 256-thread CTAs per SM start with 128 registers per thread; the softmax
// warpgroup then takes kSoftmaxRegs and the other warpgroup keeps kOtherRegs.  setmaxnreg.inc can
// only take registers that this CTA's own setmaxnreg.dec released and blocks -- with no time limit
// -- until they exist, so the budget after the exchange must fit in the launch allocation.
constexpr int kLaunchRegs = 128;
constexpr int kSoftmaxRegs = 208;
constexpr int kOtherRegs = 48;
static_assert(128 * kSoftmaxRegs + 128 * kOtherRegs <= kNumThreads * kLaunchRegs,
              "setmaxnreg budget exceeds the launch allocation: the kernel would hang");
static_assert(kSoftmaxRegs % 8 == 0 && kOtherRegs % 8 == 0 && kOtherRegs >= 24, "setmaxnreg operands");
constexpr uint32_t kTmemCols = 256;    // two resident CTAs share the SM's 512 columns
constexpr uint32_t kTmemS = 0, kTmemP = 128, kTmemO = 192;
constexpr float kRescaleThresholdLog2 = 8.0f;
constexpr int kItemTable = 256;        // work items per CTA decoded ahead (one per thread at start-up)
static_assert(kItemTable == kNumThreads, "one table entry per thread");
#ifdef FA_WAIT_TEST
// Test build (build.build_wait_test_library): waits give up after 2 ms, and the producer leaves out
// one K tile (see load_kv), so that a test can watch a bounded wait run out and the kernel drain.
constexpr uint64_t kWaitLimitNs = 2ull * 1000ull * 1000ull;
#else
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait
#endif

// watchdog codes (status word 0); low byte tells which wait ran out
constexpr uint32_t kWatchdogBase = 0x10000u;
enum WaitId : uint32_t {
  kWaitQFull = 1, kWaitKVFull = 2, kWaitKVEmpty = 3, kWaitSFull = 4, kWaitPFull = 5,
  kWaitOFull = 6, kWaitDrain = 7, kWaitSFree = 8, kWaitQEmpty = 9, kWaitOFree = 10
};

// Optional timeline trace (compile with -DFA_TRACE; timeline.py builds that variant into a library
// of its own): lane 0 of softmax warps 0 and 3 and of the issuer warp store clock64() stamps of
// their hand-offs for the CTA's first kTraceTilesSm tiles.  The stamps go to shared memory -- a
// store to global memory inside the loop would sit in front of every mbarrier arrive (release
// semantics) and stretch the very phases that are measured -- and the CTA named by
// g_fa_trace_block copies them out when it ends.  The product library is built without it and
// carries none of this.
#ifdef FA_TRACE
constexpr int kTraceRoles = 4, kTraceTiles = 64, kTraceEvents = 16;   // layout of the global copy
constexpr int kTraceRolesSm = 3, kTraceTilesSm = 32, kTraceEventsSm = 10;
constexpr int kTraceSlots = kTraceRoles * kTraceTiles * kTraceEvents;
__device__ unsigned long long g_fa_trace[kTraceSlots];
__device__ int g_fa_trace_block = 0;
#define FA_TRACE_EVENT(role, g, e)                                                     \
  do {                                                                                 \
    if ((role) >= 0 && (threadIdx.x & 31) == 0 && (g) < kTraceTilesSm)                 \
      sm.trace[role][g][e] = clock64();                                                \
  } while (0)
#else
#define FA_TRACE_EVENT(role, g, e) do {} while (0)
#endif

struct __align__(1024) SharedStorage {
  uint8_t q[kTileBytes];
  uint8_t kv[kKVSlots][kTileBytes];
  uint8_t o_stage[kTileBytes];   // bf16 O tile, 128B-swizzled, source of the TMA store
  uint64_t q_full;
  uint64_t q_empty;              // every S of the item that used the Q slot has completed
  uint64_t kv_full[kKVSlots];
  uint64_t kv_empty[kKVSlots];
  uint64_t s_full;               // S written by the tensor core
  uint64_t s_free;               // S copied to registers by all four softmax warps
  uint64_t p_full;               // P written to TMEM by all four softmax warps
  uint64_t o_full;               // O += P V_j finished (P reusable, O stable)
  uint64_t o_free;               // the epilogue has read O: the next item may overwrite it
  uint32_t tmem_base;
  uint32_t abort;                // 0, or the watchdog code of the first wait that gave up
  uint32_t abort_who;            // thread index | parity << 16 of that wait
  float2 owed[kBlockM];          // per row of a finished item: {1 / l, m * c + log2 l} for its epilogue
  int4 items[kItemTable];        // persistent kernel: this CTA's first work items, decoded once:
                                 // {first query row, K/V tiles (0 = no such item), head, batch}
#ifdef FA_TRACE
  unsigned long long trace[kTraceRolesSm][kTraceTilesSm][kTraceEventsSm];
#endif
};
constexpr int kSmemBytes = sizeof(SharedStorage) + 1024;  // + slack to align the base to 1024
static_assert(kCtasPerSm * (kSmemBytes + 1024) <= 227 * 1024, "two CTAs must fit in one SM");

// Division by a run-time constant as multiply-high + shift (the magic pair is computed on the
// host by make_fast_div).  Exact for 0 <= n < 2^31 and 1 <= d < 2^31.  An integer division costs
// the softmax warps over a hundred clocks, and three of them sat on the path between two work
// items.
struct FastDiv {
  uint32_t mul;
  uint32_t shift;
  uint32_t div;
};
__host__ inline FastDiv make_fast_div(uint32_t d) {
  FastDiv f;
  f.div = d;
  if (d == 1) { f.mul = 0; f.shift = 0; return f; }
  uint32_t l = 0;
  while ((1ull << l) < d) ++l;                       // l = ceil(log2 d), 1 <= l <= 31
  const unsigned long long p = 31 + l;
  f.mul = static_cast<uint32_t>(((1ull << p) + d - 1) / d);   // ceil(2^p / d), fits in 32 bits
  f.shift = l - 1;                                   // total shift p - 32
  return f;
}
__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f) {
  return f.div == 1 ? n : (__umulhi(n, f.mul) >> f.shift);
}

struct FwdParams {
  float* lse;                 // may be null
  int B, H, N;
  int n_qtiles;               // ceil(N / 128): work items per (batch, head)
  FastDiv div_qtiles, div_heads;   // divisions by n_qtiles and by H
  int n_items;                // B * H * n_qtiles
  int paired;                 // persistent causal schedule with an even tile count: complementary pairs
  int n_units;                // B * H * n_qtiles / 2 when paired
  FastDiv div_half;           // division by n_qtiles / 2
  int causal;
  float scale_log2;           // softmax_scale * log2(e)
  unsigned int* status;       // [4] watchdog words in global memory
};

struct Watch {
  volatile uint32_t* abort;   // shared memory: 0, or the code of the first wait that gave up
  volatile uint32_t* who;     // shared memory: thread index | parity << 16 of that wait
};

// A bounded wait.  Each failed try_wait suspends the thread for a while in hardware; every 64 of
// them the loop looks at the CTA's abort word and at the clock.  A wait that runs out of time
// leaves its code in shared memory and returns false; the kernel's teardown copies the first
// such code to the status words in global memory.  (Kept this small on purpose: the function is
// inlined at fourteen places, and the tile loop lives off the instruction cache -- the earlier
// form with the status words written at every site cost 1-2 % through its size alone.)
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const Watch& w,
                                         uint32_t id, uint64_t limit_ns = kWaitLimitNs,
                                         bool heed_abort = true) {
  static_assert(kWaitLimitNs < 4000000000ull, "the 32-bit timer difference would wrap");
  uint32_t t0 = 0;   // the low word of the nanosecond timer is enough: limits are below 4 s
#pragma unroll 1
  for (uint32_t polls = 0; polls < (1u << 26); ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 63u) == 63u) {
      if (heed_abort && *w.abort) return false;
      const uint32_t now = globaltimer_lo_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > static_cast<uint32_t>(limit_ns)) break;
    }
  }
  if (*w.abort == 0) {
    *w.who = threadIdx.x | (parity << 16);
    *w.abort = kWatchdogBase | id;
  }
  return false;
}
// The same for a whole converged warp: every lane polls, the answer is made uniform.
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity, const Watch& w,
                                              uint32_t id) {
  return __all_sync(0xffffffffu, wait_bar(bar, parity, w, id));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// kPersistent = true: the grid is 2 x SM count and every role loops over work items (best when
// items are many and short, e.g. N = 1024 causal: 4.5 K/V tiles per item on average).
// kPersistent = false: one CTA per item, no cross-item state in the hot loop (best for long
// sequences and for grids too small to balance statically).
// kCausal selects the masking code at compile time (the non-causal instantiation carries none of
// the diagonal-tile handling).
// kRagged (non-causal only): N is not a multiple of 128, the last K/V tile of every item needs its
// columns past N masked.  The 128 tests for that sit inside the tile loop, and the loop's speed
// depends on its code size, so sequences of whole tiles get an instantiation without them.
template <bool kPersistent, bool kCausal, bool kRagged = false>
__global__ void __launch_bounds__(kNumThreads, kCtasPerSm)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
              const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  SharedStorage& sm =
      *reinterpret_cast<SharedStorage*>(smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nkv = (p.N + kBlockN - 1) / kBlockN;

  // The n-th work item of this CTA -> (batch, head, query tile); false when the CTA is done.
  // A head's tiles are adjacent in the list, so CTAs that run side by side share that head's K/V
  // in L2.  In causal mode tile t costs t+1 K/V tiles.  Three schedules:
  //   one CTA per item      heaviest tile of a head first, the hardware balances dynamically;
  //   persistent, paired    (even tile count) the CTA takes tile nq-1-s and then its complement
  //                         s of the same head: every pair costs nq+1 K/V tiles, so a CTA striding
  //                         through the pairs by gridDim.x gets equal work;
  //   persistent, rotated   (odd tile count, or non-causal) stride through single items, the tile
  //                         order inside a head rotated by the head index.
  struct Item { int b, h, q_row, ns; };
  auto decode_item = [&](int n, Item& w) -> bool {
    int bh, qt;
    if (kPersistent && kCausal && p.paired) {
      const int unit = blockIdx.x + (n >> 1) * gridDim.x;
      if (unit >= p.n_units) return false;
      const int half_q = p.n_qtiles >> 1;
      bh = static_cast<int>(fast_div(unit, p.div_half));
      const int sidx = unit - bh * half_q;
      // CTAs that share an SM (and the grid as a whole) should not all be at the same point of
      // their pair at the same time: half of them take the short tile of each pair first.  Which
      // CTAs share an SM is not known; on a 148-SM B200 CTA i sits with i + 148 or with i ^ 1, and
      // this hash separates both.  (A constant divisor: no division is executed, and nothing is
      // kept in a register through the softmax loop, where one more live value costs spills.)
      const int pair_swap = (blockIdx.x ^ (blockIdx.x / kSmCountHint)) & 1;
      qt = ((n & 1) ^ pair_swap) ? sidx : p.n_qtiles - 1 - sidx;
    } else {
      if (!kPersistent && n > 0) return false;
      const int item = blockIdx.x + n * gridDim.x;
      if (item >= p.n_items) return false;
      bh = static_cast<int>(fast_div(item, p.div_qtiles));
      const int slot = item - bh * p.n_qtiles;
      qt = slot;
      if (kCausal) {
        int rs = slot;
        if (kPersistent) {       // (slot + bh) mod n_qtiles without a second division
          const int bh_mod = bh - static_cast<int>(fast_div(bh, p.div_qtiles)) * p.n_qtiles;
          rs = slot + bh_mod;
          if (rs >= p.n_qtiles) rs -= p.n_qtiles;
        }
        qt = p.n_qtiles - 1 - rs;
      }
    }
    w.b = static_cast<int>(fast_div(bh, p.div_heads));
    w.h = bh - w.b * p.H;
    w.q_row = qt * kBlockM;
    w.ns = kCausal ? min(nkv, qt + 1) : nkv;   // K/V tiles this query tile attends to
    return true;
  };
  // Decoding costs ~170 clocks of dependent integer arithmetic, and every role would pay it on
  // the path between two work items.  A persistent CTA therefore decodes all its items once, one
  // per thread, before the start-up barrier; afterwards an item is one shared-memory load (the
  // same address for the whole warp).  The launcher picks a persistent schedule only where a CTA
  // gets at most kItemTable items.
  auto get_item = [&](int n, Item& w) -> bool {
    if (kPersistent) {
      if (n >= kItemTable) return false;
      const int4 e = sm.items[n];
      w.q_row = e.x; w.ns = e.y; w.h = e.z; w.b = e.w;
      return e.y != 0;
    }
    return decode_item(n, w);
  };

  // ---- one-time setup
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sm.q_full), 1);
    mbar_init(smem_u32(&sm.q_empty), 1);
    mbar_init(smem_u32(&sm.s_full), 1);
    mbar_init(smem_u32(&sm.s_free), kNumSoftmaxWarps);
    mbar_init(smem_u32(&sm.p_full), kNumSoftmaxWarps);
    mbar_init(smem_u32(&sm.o_full), 1);
    mbar_init(smem_u32(&sm.o_free), kNumSoftmaxWarps);
    for (int i = 0; i < kKVSlots; ++i) {
      mbar_init(smem_u32(&sm.kv_full[i]), 1);
      mbar_init(smem_u32(&sm.kv_empty[i]), 1);
    }
    sm.abort = 0;
    sm.abort_who = 0;
    fence_mbar_init();
  }
#ifdef FA_TRACE
  for (int i = threadIdx.x; i < kTraceRolesSm * kTraceTilesSm * kTraceEventsSm; i += kNumThreads)
    (&sm.trace[0][0][0])[i] = 0ull;
#endif
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sm.tmem_base), kTmemCols);
    tmem_relinquish();
  }
  if (kPersistent) {
    Item t;
    const bool has = decode_item(threadIdx.x, t);
    sm.items[threadIdx.x] = has ? make_int4(t.q_row, t.ns, t.h, t.b) : make_int4(0, 0, 0, 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  const Watch watch{&sm.abort, &sm.abort_who};

  auto slot_of = [](int it) { return it % kKVSlots; };
  auto par_of = [](int it) { return static_cast<uint32_t>((it / kKVSlots) & 1); };

  if (warp >= kNumSoftmaxWarps) {
    reg_dealloc<kOtherRegs>();      // executed by all four warps of warpgroup 1
    if (warp == kLoadWarp) {
      // ================================================================= TMA producer
      // K/V ring order: K_0 V_0 K_1 V_1 ... continuing across work items; `it` counts loads.
      // One Q slot is enough to load the next item's Q early: it is free as soon as the current
      // item's LAST S has completed, a whole softmax + PV + epilogue before the item ends.
      if (elect_one()) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
        tma_prefetch_desc(&tmap_o);
      }
      bool ok = true;
      int it = 0, n = 0;
      auto load_kv = [&](const CUtensorMap* map, int row, int h, int b) {
#ifdef FA_WAIT_TEST
        if (it == 2) { ++it; return; }   // the second K tile is never loaded: nothing arms its barrier
#endif
        const int slot = slot_of(it);
        const int use = it / kKVSlots;
        if (use > 0 && ok)
          ok = wait_bar_warp(smem_u32(&sm.kv_empty[slot]), (use - 1) & 1, watch, kWaitKVEmpty);
        if (ok) {
          if (elect_one()) {
            const uint32_t bar = smem_u32(&sm.kv_full[slot]);
            mbar_arrive_expect_tx(bar, kTileBytes);
            tma_load_4d(smem_u32(sm.kv[slot]), map, bar, 0, row, h, b);
          }
          ++it;
        }
      };
      for (; ok; ++n) {
        Item w;
        if (!get_item(n, w)) break;
        if (n > 0) ok = wait_bar_warp(smem_u32(&sm.q_empty), (n - 1) & 1, watch, kWaitQEmpty);
        if (!ok) break;
        if (elect_one()) {
          const uint32_t bar = smem_u32(&sm.q_full);
          mbar_arrive_expect_tx(bar, kTileBytes);
          tma_load_4d(smem_u32(sm.q), &tmap_q, bar, 0, w.q_row, w.h, w.b);
        }
        for (int j = 0; j < w.ns && ok; ++j) {
          load_kv(&tmap_k, j * kBlockN, w.h, w.b);
          load_kv(&tmap_v, j * kBlockN, w.h, w.b);
        }
      }
      if (sm.abort && lane == 0) {
        // leave no copy of ours in flight: wait (bounded) for every load still armed
        for (int i = max(0, it - kKVSlots); i < it; ++i)
          wait_bar(smem_u32(&sm.kv_full[slot_of(i)]), par_of(i), watch, kWaitDrain,
                   20ull * 1000 * 1000, false);
        if (n > 0)
          wait_bar(smem_u32(&sm.q_full), (n - 1) & 1, watch, kWaitDrain, 20ull * 1000 * 1000, false);
      }
      __syncwarp();
    } else if (warp == kMmaWarp) {
      // ================================================================= tcgen05 issuer
      constexpr uint32_t idesc_s = make_idesc_bf16(kBlockM, kBlockN, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(kBlockM, kHeadDim, true);
      const uint64_t desc_q = make_sw128_desc(smem_u32(sm.q));
      const uint32_t t_s = tmem_base + kTmemS;
      const uint32_t t_p = tmem_base + kTmemP;
      const uint32_t t_o = tmem_base + kTmemO;
      const uint32_t bar_s_full = smem_u32(&sm.s_full);
      const uint32_t bar_o_full = smem_u32(&sm.o_full);

      // S = Q K^T from ring slot `slot`; releases that slot, and the Q slot after an item's last S
      auto issue_s = [&](int slot, bool last_of_item) {
        if (elect_one()) {
          const uint64_t dk = make_sw128_desc(smem_u32(sm.kv[slot]));
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)  // +32 bytes along the row per K=16 step
            umma_ss(t_s, desc_q + 2 * kk, dk + 2 * kk, idesc_s, kk > 0);
          tc_commit(bar_s_full);
          tc_commit(smem_u32(&sm.kv_empty[slot]));
          if (last_of_item) tc_commit(smem_u32(&sm.q_empty));
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

      // Running counters: `it` = ring index of the next V to consume, `g` = global index of the
      // tile whose PV comes next, `n` = local item index.
      bool ok = true;
      int it = 1, g = 0, n = 0;
      Item w;
      bool have_item = get_item(0, w);
      if (have_item) {
        ok = wait_bar_warp(smem_u32(&sm.q_full), 0, watch, kWaitQFull) &&
             wait_bar_warp(smem_u32(&sm.kv_full[0]), 0, watch, kWaitKVFull);
        if (ok) {
          tc_fence_after();
          issue_s(0, w.ns == 1);
        }
      }
      for (; have_item && ok; ++n) {
        Item wn = w;
        const bool has_next_item = get_item(n + 1, wn);
        for (int j = 0; j < w.ns && ok; ++j, ++g) {
          const int itv = it;          // V_j of this item
          const int itk = it + 1;      // the next K in ring order: K_{j+1}, or K_0 of the next item
          const bool last = j + 1 == w.ns;
          // ---- S for the next tile, as soon as the softmax warps hold S(g) in registers
          FA_TRACE_EVENT(2, g, 0);
          if (!last || has_next_item) {
            if (last)   // the next item's Q must have landed (its load waited for q_empty)
              ok = wait_bar_warp(smem_u32(&sm.q_full), (n + 1) & 1, watch, kWaitQFull);
            ok = ok &&
                 wait_bar_warp(smem_u32(&sm.kv_full[slot_of(itk)]), par_of(itk), watch, kWaitKVFull);
            FA_TRACE_EVENT(2, g, 1);
            ok = ok && wait_bar_warp(smem_u32(&sm.s_free), g & 1, watch, kWaitSFree);
            if (!ok) break;
            FA_TRACE_EVENT(2, g, 2);
            tc_fence_after();
            issue_s(slot_of(itk), last ? wn.ns == 1 : j + 2 == w.ns);
            FA_TRACE_EVENT(2, g, 3);
          }
          // ---- O += P V for this tile
          ok = wait_bar_warp(smem_u32(&sm.kv_full[slot_of(itv)]), par_of(itv), watch, kWaitKVFull);
          FA_TRACE_EVENT(2, g, 4);
          ok = ok && wait_bar_warp(smem_u32(&sm.p_full), g & 1, watch, kWaitPFull);
          if (ok && j == 0 && n > 0)   // the previous item's epilogue must have read O
            ok = wait_bar_warp(smem_u32(&sm.o_free), (n - 1) & 1, watch, kWaitOFree);
          if (!ok) break;
          FA_TRACE_EVENT(2, g, 5);
          tc_fence_after();
          issue_pv(slot_of(itv), j == 0);
          FA_TRACE_EVENT(2, g, 6);
          it += 2;
        }
        w = wn;
        have_item = has_next_item;
      }
    }
  } else {
    // =================================================================== softmax warps
    reg_alloc<kSoftmaxRegs>();      // executed by all four warps of warpgroup 0
    const int r = threadIdx.x;                  // row inside the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t t_s = tmem_base + lane_base + kTmemS;
    const uint32_t t_p = tmem_base + lane_base + kTmemP;
    const uint32_t t_o = tmem_base + lane_base + kTmemO;
    const float c = p.scale_log2;
    const uint32_t bar_s_full = smem_u32(&sm.s_full);
    const uint32_t bar_s_free = smem_u32(&sm.s_free);
    const uint32_t bar_p = smem_u32(&sm.p_full);
    const uint32_t bar_o = smem_u32(&sm.o_full);
    constexpr uint32_t kNegInf = 0xff800000u;

    bool ok = true;
    int g = 0;   // running tile counter across work items (selects the barrier phases)
    int n = 0;   // local work-item counter
#ifdef FA_TRACE
    const int trole = warp == 0 ? 0 : (warp == 3 ? 1 : -1);
#endif

    // A finished item whose epilogue is still owed.  It is run in the middle of the NEXT item's
    // first tile (after that tile's P is stored, before the issuer is told about it): by then the
    // last O += P V of the finished item has long completed, so nobody sits waiting for it.
    // What the epilogue needs of the finished item waits in shared memory, not in registers that
    // would stay live through the hot loop: each thread parks its row's {1 / l, m * c + log2 l}
    // when the item ends, and the item's coordinates come from the item table again.
    // O / l -> bf16 -> swizzled staging tile -> TMA store; LSE.  Reads O of the owed item.
    auto epilogue = [&](const int owed_n) -> bool {
      Item ow;
      get_item(owed_n, ow);
      const float2 parked = sm.owed[r];
      const uint32_t bar_o_free = smem_u32(&sm.o_free);
      // this thread's row of the staging tile; 16-byte chunk c goes to position c ^ (r & 7)
      // (the 128-byte swizzle the TMA store expects)
      const uint32_t stage_row = smem_u32(sm.o_stage) + r * 128;
      const int owed_q_row = ow.q_row, owed_h = ow.h, owed_b = ow.b;
      tc_fence_after();
      // O / l -> bf16 while loading, 32 columns at a time (keeps the register peak low: the
      // persistent kernel runs this in the middle of a tile)
      const float inv_l = parked.x;
      uint32_t ob[kHeadDim / 2];
      {
        uint32_t ov[kHeadDim];        // one load, one wait: the scores' registers are free by now
        tmem_ld_x64(t_o, ov);
#pragma unroll
        for (int i = 0; i < kHeadDim / 2; ++i)
          ob[i] = pack_bf16(__uint_as_float(ov[2 * i]) * inv_l, __uint_as_float(ov[2 * i + 1]) * inv_l);
      }
      // O is in registers: the issuer may start the next item's accumulation
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_o_free);
      // Each warp stages and stores its own 32 rows, so no other warp is involved: lane 0 issued
      // the previous store from this slab and makes sure it has been read before the slab is
      // rewritten (it was issued a whole work item ago).
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
#pragma unroll
      for (int ck = 0; ck < 8; ++ck) {
        uint4 wv;
        wv.x = ob[4 * ck + 0];
        wv.y = ob[4 * ck + 1];
        wv.z = ob[4 * ck + 2];
        wv.w = ob[4 * ck + 3];
        st_shared_v4(stage_row + ((ck ^ (r & 7)) << 4), wv);
      }
      fence_proxy_async_smem();     // generic-proxy writes -> visible to the TMA engine
      __syncwarp();
      const int slab_row = owed_q_row + 32 * warp;
      if (lane == 0 && slab_row < p.N) {   // rows >= N inside the slab are clipped by the tensor map
        tma_store_4d(&tmap_o, smem_u32(sm.o_stage) + warp * (32 * 128), 0, slab_row, owed_h, owed_b);
        tma_store_commit();
      }
      const int row = owed_q_row + r;
      if (p.lse != nullptr && row < p.N) {
        // ln(sum_j exp(scale * s_j)) = ln2 * (m_ref * c + log2(l))
        p.lse[((long long)owed_b * p.H + owed_h) * p.N + row] =
            0.6931471805599453f * parked.y;
      }
      return true;
    };

    for (; ok; ++n) {
      Item w;
      if (!get_item(n, w)) break;
      float m_ref = -CUDART_INF_F;  // max the exponentials are currently taken against (raw scores)
      float l = 0.f;                // running sum of exp2((s - m_ref) * c)

      for (int j = 0; j < w.ns; ++j, ++g) {
        FA_TRACE_EVENT(trole, g, 0);
        if (j == 0) FA_TRACE_EVENT(trole, g, 9);
        ok = wait_bar_warp(bar_s_full, g & 1, watch, kWaitSFull);
        if (!ok) break;
        FA_TRACE_EVENT(trole, g, 1);
        tc_fence_after();
        uint32_t sv[kBlockN];
        {  // two 64-column loads: a single 128-register instruction does not fit the 128-register
           // launch allocation the assembler plans with, whatever setmaxnreg grants later
          uint32_t (&lo)[64] = *reinterpret_cast<uint32_t (*)[64]>(&sv[0]);
          uint32_t (&hi)[64] = *reinterpret_cast<uint32_t (*)[64]>(&sv[64]);
          tmem_ld_nowait_x64(t_s, lo);
          tmem_ld_nowait_x64(t_s + 64, hi);
          tmem_wait_ld_fence(sv);
        }
        FA_TRACE_EVENT(trole, g, 2);
        // S is in registers: let the issuer overwrite it with the next tile's scores
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s_free);

        const int col0 = j * kBlockN;
        int first_masked_chunk = 4;   // 32-column chunks from here on are invisible to this warp
        if (kCausal) {
          if (col0 == w.q_row) {
            // The diagonal tile: column k is visible to row r iff k <= r.  This warp owns rows
            // 32*warp .. 32*warp+31, so 32-column chunks are decided for the whole warp: chunks
            // below `warp` are fully visible, chunks above are fully masked (handled below without
            // touching the scores: they are left out of the max and exponentiated with an
            // offset of -inf), and only chunk == warp needs a per-element test -- a quarter of
            // the compares and selects of the naive form.
            first_masked_chunk = warp + 1;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              if (ch == warp) {
#pragma unroll
                for (int k = 0; k < 32; ++k)
                  if (k > lane) sv[32 * ch + k] = kNegInf;
              }
            }
          }
        } else if (kRagged && col0 + kBlockN > p.N) {  // ragged last tile: TMA zero-fill gives score 0, not -inf
          const int lim = p.N - col0;
#pragma unroll
          for (int k = 0; k < kBlockN; ++k)
            if (k >= lim) sv[k] = kNegInf;
        }

        float mx[4];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {   // four independent chains of 32
          const int o = 32 * ch;
          float m = fmax3(__uint_as_float(sv[o]), __uint_as_float(sv[o + 1]), __uint_as_float(sv[o + 2]));
#pragma unroll
          for (int k = 3; k + 1 < 32; k += 2)
            m = fmax3(m, __uint_as_float(sv[o + k]), __uint_as_float(sv[o + k + 1]));
          mx[ch] = fmaxf(m, __uint_as_float(sv[o + 31]));
          if (ch >= first_masked_chunk) mx[ch] = -CUDART_INF_F;
        }
        const float m_new = fmaxf(fmax3(mx[0], mx[1], mx[2]), fmaxf(mx[3], m_ref));

        // O += P V of the previous tile (of this or the previous item) must be finished before P
        // is overwritten or O is touched
        FA_TRACE_EVENT(trole, g, 3);
        if (g > 0) {
          ok = wait_bar_warp(bar_o, (g - 1) & 1, watch, kWaitOFull);
          if (!ok) break;
        }
        FA_TRACE_EVENT(trole, g, 4);
        if (j == 0) {
          m_ref = m_new;
        } else {
          // Rescale lazily: while the max grew by less than 2^8 keep the old reference; P stays
          // below 256 and the final O / l is exact because O, l and P share one reference.
          const bool need = (m_new - m_ref) * c > kRescaleThresholdLog2;
          if (__any_sync(0xffffffffu, need)) {
            const float f = need ? ex2_approx((m_ref - m_new) * c) : 1.0f;
            tc_fence_after();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t ov[32];
              tmem_ld_x32(t_o + 32 * half, ov);
#pragma unroll
              for (int k = 0; k < 32; ++k) ov[k] = __float_as_uint(__uint_as_float(ov[k]) * f);
              tmem_st_x32(t_o + 32 * half, ov);
            }
            l *= f;
            if (need) m_ref = m_new;
          }
        }

        const float neg_mc_all = -m_ref * c;
        const uint64_t c2 = pack_f32x2(c, c);
        uint64_t lsum0 = 0ull, lsum1 = 0ull;   // two packed pairs of partial row sums
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {   // 32 scores -> 16 packed registers -> one TMEM store
          uint32_t pk[16];
          const float neg_mc = ch >= first_masked_chunk ? -CUDART_INF_F : neg_mc_all;  // exp2(-inf) = 0
          const uint64_t neg_mc2 = pack_f32x2(neg_mc, neg_mc);
#pragma unroll
          for (int k = 0; k < 32; k += 4) {
            const int o = 32 * ch + k;
            float x0, x1, x2, x3;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[o + 0]), __uint_as_float(sv[o + 1])), c2, neg_mc2), x0, x1);
            const uint64_t xb = fma_f32x2(pack_f32x2(__uint_as_float(sv[o + 2]), __uint_as_float(sv[o + 3])), c2, neg_mc2);
            unpack_f32x2(xb, x2, x3);
            const float p0 = ex2_approx(x0);
            const float p1 = ex2_approx(x1);
            float p2, p3;
            if ((k % 8) == 4) {   // 2 of every 8 on the FMA pipe
              exp2_poly_x2(x2, x3, p2, p3);
            } else {
              p2 = ex2_approx(x2);
              p3 = ex2_approx(x3);
            }
            lsum0 = add_f32x2(lsum0, pack_f32x2(p0, p1));
            lsum1 = add_f32x2(lsum1, pack_f32x2(p2, p3));
            pk[k / 2 + 0] = pack_bf16(p0, p1);
            pk[k / 2 + 1] = pack_bf16(p2, p3);
          }
          tmem_st_x16(t_p + 16 * ch, pk);
        }
        {
          float l0, l1, l2, l3;
          unpack_f32x2(lsum0, l0, l1);
          unpack_f32x2(lsum1, l2, l3);
          l += (l0 + l1) + (l2 + l3);
        }
        FA_TRACE_EVENT(trole, g, 5);
        tmem_wait_st();
        FA_TRACE_EVENT(trole, g, 6);

        FA_TRACE_EVENT(trole, g, 7);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p);
        FA_TRACE_EVENT(trole, g, 8);

        // The epilogue owed to the previous item: its O is final (the o_full wait above covered
        // its last PV).  It runs behind the hand-off of this item's first P: the issuer holds the
        // PV that overwrites O until the epilogue has read it (o_free), and at the end of the
        // tile body the test costs the ordinary tiles no jump over the inlined code.
        if (kPersistent && j == 0 && n > 0) {
          ok = epilogue(n - 1);
          if (!ok) break;
        }
      }
      if (!ok) break;
      // (approximate reciprocal and logarithm: 1 ulp and 2^-22 absolute, far inside the bf16
      // rounding of O and the LSE tolerance, and a few dozen instructions shorter on the path
      // between two work items; l >= 1 always, the row maximum of the first tile contributes 1)
      sm.owed[r] = make_float2(rcp_approx(l), fmaf(m_ref, c, lg2_approx(l)));   // read back by this same thread
    }
    // the last item's epilogue
    if (ok && n > 0) {
      ok = wait_bar_warp(bar_o, (g - 1) & 1, watch, kWaitOFull);
      if (ok) ok = epilogue(n - 1);
    }
    // each warp's last TMA store must have read its slab before shared memory goes away
    if (lane == 0) tma_store_wait_read<0>();
  }

  // ---- teardown: every TMEM access above is complete (loads waited, MMAs observed via o_full)
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && sm.abort != 0) {   // a wait gave up: the first CTA to say so is recorded
    if (atomicCAS(p.status, 0u, sm.abort) == 0u) {
      p.status[1] = blockIdx.x;
      p.status[2] = sm.abort_who & 0xffffu;
      p.status[3] = sm.abort_who >> 16;
    }
  }
#ifdef FA_TRACE
  if (blockIdx.x == g_fa_trace_block) {
    for (int i = threadIdx.x; i < kTraceRolesSm * kTraceTilesSm * kTraceEventsSm; i += kNumThreads) {
      const int role = i / (kTraceTilesSm * kTraceEventsSm);
      const int g = (i / kTraceEventsSm) % kTraceTilesSm;
      const int e = i % kTraceEventsSm;
      g_fa_trace[(role * kTraceTiles + g) * kTraceEvents + e] = sm.trace[role][g][e];
    }
  }
#endif
}

}  // namespace fa
