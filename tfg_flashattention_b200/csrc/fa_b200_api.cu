// Host side of libfa_b200.so: the C ABI declared in include/fa_b200.h.
// Validates arguments, builds the TMA descriptors, launches the sm_100a kernel on the caller's
// stream.  No exceptions, no torch types, no CPU fallback: a device that is not 10.x is an error.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "../../include/fa_b200.h"
#include "add_layernorm_sm100.cuh"
#include "fa_decode_sm100.cuh"
#include "fa_fwd_sm100.cuh"
#include "linear_small_sm100.cuh"

namespace {

constexpr int kMaxDevices = 64;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceState {
  std::once_flag once;
  int init_error = 0;       // value fa_b200_fwd returns if set-up failed
  unsigned int* status = nullptr;  // device address of the watchdog words
  int resident_ctas = 0;           // persistent grid size: CTAs per SM x SM count
  int sm_count = 0;
};

DeviceState g_dev[kMaxDevices];
std::once_flag g_encode_once;
EncodeTiledFn g_encode = nullptr;

// Watchdog words, one set per device that loads the module (a __device__ variable is
// instantiated per device).  Word 0: code, 1: blockIdx.x, 2: threadIdx.x, 3: barrier parity.
__device__ unsigned int g_fa_status[4];

void resolve_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
          cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
}

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  int error = 0;
  explicit DeviceGuard(int dev) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) { error = static_cast<int>(e); return; }
    if (prev != dev) {
      e = cudaSetDevice(dev);
      if (e != cudaSuccess) { error = static_cast<int>(e); return; }
      switched = true;
    }
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

// Runs once per device, with that device current.
void init_device(int dev) {
  DeviceState& st = g_dev[dev];
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) { st.init_error = static_cast<int>(e); return; }
  if (prop.major != 10) { st.init_error = FA_B200_ERR_ARCH; return; }
  // The kernel moves registers between its warpgroups with setmaxnreg; that only works (and
  // otherwise blocks for ever) if the compiler gave the kernel the launch allocation the budget
  // in fa_fwd_sm100.cuh assumes.  Refuse to launch a build where it did not.
  const void* variants[6] = {reinterpret_cast<const void*>(&fa::fa_fwd_kernel<false, false>),
                             reinterpret_cast<const void*>(&fa::fa_fwd_kernel<false, false, true>),
                             reinterpret_cast<const void*>(&fa::fa_fwd_kernel<false, true>),
                             reinterpret_cast<const void*>(&fa::fa_fwd_kernel<true, false>),
                             reinterpret_cast<const void*>(&fa::fa_fwd_kernel<true, false, true>),
                             reinterpret_cast<const void*>(&fa::fa_fwd_kernel<true, true>)};
  for (const void* fn : variants) {
    cudaFuncAttributes fattr;
    e = cudaFuncGetAttributes(&fattr, fn);
    if (e != cudaSuccess) { st.init_error = static_cast<int>(e); return; }
    if (fattr.numRegs != fa::kLaunchRegs) { st.init_error = FA_B200_ERR_BUILD; return; }
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::kSmemBytes);
    if (e != cudaSuccess) { st.init_error = static_cast<int>(e); return; }
    // Two CTAs of ~100 KB each must fit: ask for the largest shared-memory carveout.
    e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) { st.init_error = static_cast<int>(e); return; }
    // Two CTAs per SM each allocate half of tensor memory; a third resident CTA would block in
    // tcgen05.alloc until one of them exits.  Shared memory already limits residency to two; make
    // sure of it (a build with a much smaller footprint would break that assumption).
    int resident = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fn, fa::kNumThreads, fa::kSmemBytes);
    if (e != cudaSuccess) { st.init_error = static_cast<int>(e); return; }
    if (resident < 1 || resident > fa::kCtasPerSm) { st.init_error = FA_B200_ERR_BUILD; return; }
  }
  // The persistent grid is sized for kCtasPerSm per SM whatever the occupancy query answered: it
  // has been seen to answer 1 where the hardware co-schedules 2, and a CTA that has to wait for
  // a slot only starts later -- work items are partitioned by grid stride, no CTA waits on another.
  st.resident_ctas = fa::kCtasPerSm * prop.multiProcessorCount;
  st.sm_count = prop.multiProcessorCount;
  void* addr = nullptr;
  e = cudaGetSymbolAddress(&addr, g_fa_status);
  if (e != cudaSuccess) { st.init_error = static_cast<int>(e); return; }
  st.status = static_cast<unsigned int*>(addr);
  e = cudaMemset(st.status, 0, 4 * sizeof(unsigned int));
  if (e != cudaSuccess) { st.init_error = static_cast<int>(e); return; }
}

bool stride_ok(const int64_t s[3]) {
  for (int i = 0; i < 3; ++i)
    if (s[i] <= 0 || (s[i] % 8) != 0) return false;
  return true;
}

int encode_map_uncached(CUtensorMap* map, const void* base, const fa_b200_params* p,
                        const int64_t st[3], unsigned box_rows) {
  // dims, innermost first: d, N, H, B.  Strides (bytes) for dims 1..3: row, head, batch.
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(p->d), static_cast<cuuint64_t>(p->N),
                              static_cast<cuuint64_t>(p->H), static_cast<cuuint64_t>(p->B)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(st[2]) * 2, static_cast<cuuint64_t>(st[1]) * 2,
                                 static_cast<cuuint64_t>(st[0]) * 2};
  const cuuint32_t box[4] = {fa::kHeadDim, box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FA_B200_ERR_TENSORMAP;
}

// A tensor map is a pure function of (base, shape, strides, box): the driver call that encodes
// one costs about a microsecond, four of them per launch are a visible share of a small problem's
// launch path, and callers (a model's layers, a benchmark loop) present the same few buffers
// again and again.  Each host thread keeps a small direct-mapped cache of encoded maps; a hit
// needs no lock and can never be stale, because nothing outside the key enters the encoding.
struct MapKey {
  const void* base;
  int32_t B, H, N, box_rows;
  int64_t st[3];
  bool operator==(const MapKey& o) const {
    return base == o.base && B == o.B && H == o.H && N == o.N && box_rows == o.box_rows &&
           st[0] == o.st[0] && st[1] == o.st[1] && st[2] == o.st[2];
  }
};
struct MapSlot {
  MapKey key;
  bool valid = false;
  alignas(64) CUtensorMap map;
};
constexpr int kMapCacheSlots = 64;

int encode_map(CUtensorMap* map, const void* base, const fa_b200_params* p, const int64_t st[3],
               unsigned box_rows = fa::kBlockN) {
  static thread_local MapSlot cache[kMapCacheSlots];
  const MapKey key{base, p->B, p->H, p->N, static_cast<int32_t>(box_rows), {st[0], st[1], st[2]}};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
  h ^= (static_cast<uint64_t>(p->N) * 0x9E3779B97F4A7C15ull) ^ (static_cast<uint64_t>(st[2]) << 17) ^
       (static_cast<uint64_t>(box_rows) << 7) ^ (static_cast<uint64_t>(p->B) << 40) ^
       (static_cast<uint64_t>(p->H) << 52);
  h ^= h >> 29;
  MapSlot& slot = cache[(h * 0xBF58476D1CE4E5B9ull) >> 58];
  if (slot.valid && slot.key == key) {
    *map = slot.map;
    return 0;
  }
  const int rc = encode_map_uncached(&slot.map, base, p, st, box_rows);
  slot.valid = rc == 0;
  if (rc != 0) return rc;
  slot.key = key;
  *map = slot.map;
  return 0;
}

// How one forward call is scheduled (the rule behind fa_b200_fwd and fa_b200_fwd_plan).
struct FwdPlan {
  bool persistent;     // grid of resident CTAs striding through the work list
  bool paired;         // persistent causal schedule of complementary tile pairs
  int n_qtiles;
  long long items;     // B * H * n_qtiles
  unsigned grid;
};

FwdPlan plan_fwd(const fa_b200_params* p, const DeviceState& st) {
  FwdPlan pl;
  pl.n_qtiles = (p->N + fa::kBlockM - 1) / fa::kBlockM;
  pl.items = static_cast<long long>(p->B) * p->H * pl.n_qtiles;
  const int kv_tiles = (p->N + fa::kBlockN - 1) / fa::kBlockN;
  const bool causal = p->causal != 0;
  // Measured on B200: the causal schedule of complementary tile pairs wins up to N = 2048 at any
  // grid size (equal at 4096, behind beyond: long items amortise their own start-up, and the
  // hardware's dynamic placement of many CTAs balances better); without pairing, persistence pays
  // for short items (N <= 1024) once every CTA gets at least two of them.
  const bool can_pair = causal && pl.n_qtiles % 2 == 0;
  pl.persistent = can_pair ? kv_tiles <= 16
                           : (pl.items >= 2LL * st.resident_ctas && kv_tiles <= 8);
  pl.paired = pl.persistent && can_pair;
  long long work_units = pl.paired ? pl.items / 2 : pl.items;
  // a persistent CTA keeps its items in a table of fa::kItemTable entries
  if (pl.persistent && (work_units + st.resident_ctas - 1) / st.resident_ctas * (pl.paired ? 2 : 1) >
                           fa::kItemTable) {
    pl.persistent = pl.paired = false;
    work_units = pl.items;
  }
  pl.grid = static_cast<unsigned>(
      pl.persistent ? (work_units > st.resident_ctas ? st.resident_ctas : work_units) : pl.items);
  return pl;
}

// Device guard + per-device set-up shared by the forward entry points.
int ready_device(int device, DeviceState** out) {
  DeviceState& st = g_dev[device];
  std::call_once(st.once, init_device, device);
  if (st.init_error) return st.init_error;
  *out = &st;
  return 0;
}

}  // namespace

extern "C" {

int fa_b200_abi_version(void) { return FA_B200_ABI_VERSION; }

int fa_b200_validate(const fa_b200_params* p) {
  if (p == nullptr || p->q == nullptr || p->k == nullptr || p->v == nullptr || p->o == nullptr)
    return FA_B200_ERR_NULL;
  if (p->d != fa::kHeadDim) return FA_B200_ERR_HEAD_DIM;
  if (p->B < 0 || p->H < 0 || p->N < 0) return FA_B200_ERR_SHAPE;
  if (p->N > (1 << 24)) return FA_B200_ERR_SHAPE;
  {
    const long long ctas = static_cast<long long>(p->B) * p->H * ((p->N + 127) / 128);
    if (ctas > 0x7fffffffLL) return FA_B200_ERR_SHAPE;
  }
  if (!stride_ok(p->q_strides) || !stride_ok(p->k_strides) || !stride_ok(p->v_strides) ||
      !stride_ok(p->o_strides))
    return FA_B200_ERR_STRIDE;
  const uintptr_t ptrs[4] = {reinterpret_cast<uintptr_t>(p->q), reinterpret_cast<uintptr_t>(p->k),
                             reinterpret_cast<uintptr_t>(p->v), reinterpret_cast<uintptr_t>(p->o)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return FA_B200_ERR_ALIGN;
  if (p->lse != nullptr && (reinterpret_cast<uintptr_t>(p->lse) & 3u)) return FA_B200_ERR_ALIGN;
  if (!(p->softmax_scale >= 0.0f) || std::isinf(p->softmax_scale)) return FA_B200_ERR_SCALE;
  if (p->device < 0 || p->device >= kMaxDevices) return FA_B200_ERR_DEVICE;
  return FA_B200_OK;
}

int fa_b200_fwd(const fa_b200_params* p) {
  int rc = fa_b200_validate(p);
  if (rc != FA_B200_OK) return rc;
  if (p->B == 0 || p->H == 0 || p->N == 0) return FA_B200_OK;  // nothing to compute

  DeviceGuard guard(p->device);
  if (guard.error) return guard.error;
  DeviceState* stp = nullptr;
  if ((rc = ready_device(p->device, &stp)) != 0) return rc;
  const DeviceState& st = *stp;
  std::call_once(g_encode_once, resolve_encode);
  if (g_encode == nullptr) return FA_B200_ERR_DRIVER;

  CUtensorMap mq, mk, mv, mo;
  if ((rc = encode_map(&mq, p->q, p, p->q_strides)) != 0) return rc;
  if ((rc = encode_map(&mk, p->k, p, p->k_strides)) != 0) return rc;
  if ((rc = encode_map(&mv, p->v, p, p->v_strides)) != 0) return rc;
  if ((rc = encode_map(&mo, p->o, p, p->o_strides, 32)) != 0) return rc;   // one 32-row slab per warp

  const FwdPlan pl = plan_fwd(p, st);
  fa::FwdParams kp;
  kp.lse = p->lse;
  kp.B = p->B;
  kp.H = p->H;
  kp.N = p->N;
  kp.n_qtiles = pl.n_qtiles;
  kp.div_qtiles = fa::make_fast_div(static_cast<uint32_t>(kp.n_qtiles));
  kp.div_heads = fa::make_fast_div(static_cast<uint32_t>(p->H));
  kp.causal = p->causal ? 1 : 0;
  const float scale = p->softmax_scale > 0.0f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(p->d));
  kp.scale_log2 = scale * 1.4426950408889634f;
  kp.status = st.status;
  kp.n_items = static_cast<int>(pl.items);
  kp.paired = pl.paired ? 1 : 0;
  kp.n_units = static_cast<int>(pl.items / 2);
  kp.div_half = fa::make_fast_div(static_cast<uint32_t>(kp.n_qtiles > 1 ? kp.n_qtiles / 2 : 1));
  const cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  const bool ragged = (p->N % fa::kBlockN) != 0;   // non-causal only: the causal mask covers the columns past N
  if (pl.persistent) {
    if (kp.causal) fa::fa_fwd_kernel<true, true><<<pl.grid, fa::kNumThreads, fa::kSmemBytes, stream>>>(mq, mk, mv, mo, kp);
    else if (ragged) fa::fa_fwd_kernel<true, false, true><<<pl.grid, fa::kNumThreads, fa::kSmemBytes, stream>>>(mq, mk, mv, mo, kp);
    else fa::fa_fwd_kernel<true, false><<<pl.grid, fa::kNumThreads, fa::kSmemBytes, stream>>>(mq, mk, mv, mo, kp);
  } else {
    if (kp.causal) fa::fa_fwd_kernel<false, true><<<pl.grid, fa::kNumThreads, fa::kSmemBytes, stream>>>(mq, mk, mv, mo, kp);
    else if (ragged) fa::fa_fwd_kernel<false, false, true><<<pl.grid, fa::kNumThreads, fa::kSmemBytes, stream>>>(mq, mk, mv, mo, kp);
    else fa::fa_fwd_kernel<false, false><<<pl.grid, fa::kNumThreads, fa::kSmemBytes, stream>>>(mq, mk, mv, mo, kp);
  }
  return static_cast<int>(cudaGetLastError());
}

int fa_b200_fwd_plan(const fa_b200_params* p, int32_t* schedule, int32_t* grid) {
  int rc = fa_b200_validate(p);
  if (rc != FA_B200_OK) return rc;
  if (p->B == 0 || p->H == 0 || p->N == 0) {
    if (schedule != nullptr) *schedule = FA_B200_SCHEDULE_NONE;
    if (grid != nullptr) *grid = 0;
    return FA_B200_OK;
  }
  DeviceGuard guard(p->device);
  if (guard.error) return guard.error;
  DeviceState* stp = nullptr;
  if ((rc = ready_device(p->device, &stp)) != 0) return rc;
  const FwdPlan pl = plan_fwd(p, *stp);
  if (schedule != nullptr)
    *schedule = !pl.persistent ? FA_B200_SCHEDULE_CTA_PER_TILE
                : pl.paired    ? FA_B200_SCHEDULE_PERSISTENT_PAIRED
                : p->causal    ? FA_B200_SCHEDULE_PERSISTENT_ROTATED
                               : FA_B200_SCHEDULE_PERSISTENT_FULL;
  if (grid != nullptr) *grid = static_cast<int32_t>(pl.grid);
  return FA_B200_OK;
}

// ------------------------------------------------------------------------------------ decode
namespace {

// CTAs the split aims for.  Every CTA keeps a fixed 16 KB of loads in flight, so bandwidth grows
// with the number of resident CTAs: measured on B200 at B=8, H=25, kv_len=8192, 600 / 1800 / 2400
// CTAs give 4.3 / 4.6 / 5.2 TB/s.  Short caches are latency-bound and pay for the second launch
// and the partials instead (B=32, kv_len=1024: 4.8 TB/s unsplit, 4.4 split in two), so the high
// target and its coarser chunks apply from 2048 rows on.
constexpr int kDecodeTargetCtas = 592;        // 4 CTAs per SM on a 148-SM part
constexpr int kDecodeTargetCtasLong = 2368;   // 16 CTAs per SM: every thread slot of the part
constexpr int kDecodeLongLen = 2048;
constexpr int kDecodeMinRows = 64, kDecodeMinRowsLong = 512;   // rows per chunk, at least

constexpr int kDecodeWideMaxHeads = 296;   // two 1024-thread CTAs per SM on a 148-SM part
constexpr int kDecodeWideMaxLen = 4096;    // up to 1 MB of K/V per head through one SM

// How the keys of one head are cut: `splits` chunks of `rows` rows (a multiple of the 16 lane
// groups of a CTA).  The same rule sizes the workspace and launches the kernel.  Few heads with
// short caches take the one-launch form instead (`wide`: one 1024-thread CTA per head, no split).
// `fine_for_long` = false keeps the short-cache rule at every length: the allocation-free entry
// point cuts that way, so that what fits its fixed scratch buffer does not depend on this tuning.
void decode_split(int B, int H, int kv_len, int* splits, int* rows, bool* wide = nullptr,
                  bool fine_for_long = true) {
  const long long heads = static_cast<long long>(B) * H;
  const bool w = heads <= kDecodeWideMaxHeads && kv_len <= kDecodeWideMaxLen;
  if (wide != nullptr) *wide = w;
  if (w) {
    *splits = 1;
    *rows = (kv_len + 127) / 128 * 128;
    return;
  }
  const bool long_cache = fine_for_long && kv_len >= kDecodeLongLen;
  const long long target = long_cache ? kDecodeTargetCtasLong : kDecodeTargetCtas;
  const long long min_rows = long_cache ? kDecodeMinRowsLong : kDecodeMinRows;
  long long want = (target + heads - 1) / heads;
  const long long max_splits = (kv_len + min_rows - 1) / min_rows;
  if (want > max_splits) want = max_splits;
  if (want < 1) want = 1;
  long long r = (kv_len + want - 1) / want;
  r = (r + fa::kDecodeGroups - 1) / fa::kDecodeGroups * fa::kDecodeGroups;
  *rows = static_cast<int>(r);
  *splits = static_cast<int>((kv_len + r - 1) / r);
}

bool stride_ok_n(const int64_t* s, int n) {
  for (int i = 0; i < n; ++i)
    if (s[i] <= 0 || (s[i] % 8) != 0) return false;
  return true;
}

int decode_validate(const fa_b200_decode_params* p) {
  if (p == nullptr || p->q == nullptr || p->k_cache == nullptr || p->v_cache == nullptr ||
      p->o == nullptr)
    return FA_B200_ERR_NULL;
  if (p->d != fa::kHeadDim) return FA_B200_ERR_HEAD_DIM;
  if (p->B < 0 || p->H < 0 || p->kv_len < 1) return FA_B200_ERR_SHAPE;
  if (static_cast<long long>(p->B) * p->H > 0x7fffffffLL / 64) return FA_B200_ERR_SHAPE;
  if (!stride_ok_n(p->q_strides, 2) || !stride_ok_n(p->o_strides, 2) || !stride_ok_n(p->k_strides, 3) ||
      !stride_ok_n(p->v_strides, 3))
    return FA_B200_ERR_STRIDE;
  const uintptr_t ptrs[4] = {reinterpret_cast<uintptr_t>(p->q), reinterpret_cast<uintptr_t>(p->k_cache),
                             reinterpret_cast<uintptr_t>(p->v_cache), reinterpret_cast<uintptr_t>(p->o)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return FA_B200_ERR_ALIGN;
  if (p->lse != nullptr && (reinterpret_cast<uintptr_t>(p->lse) & 3u)) return FA_B200_ERR_ALIGN;
  if (p->kv_len_device != nullptr && (reinterpret_cast<uintptr_t>(p->kv_len_device) & 3u)) return FA_B200_ERR_ALIGN;
  if ((p->k_new == nullptr) != (p->v_new == nullptr)) return FA_B200_ERR_NULL;
  if (p->k_new != nullptr) {
    if (!stride_ok_n(p->new_strides, 2)) return FA_B200_ERR_STRIDE;
    if ((reinterpret_cast<uintptr_t>(p->k_new) & 15u) || (reinterpret_cast<uintptr_t>(p->v_new) & 15u))
      return FA_B200_ERR_ALIGN;
  }
  if (!(p->softmax_scale >= 0.0f) || std::isinf(p->softmax_scale)) return FA_B200_ERR_SCALE;
  if (p->device < 0 || p->device >= kMaxDevices) return FA_B200_ERR_DEVICE;
  return FA_B200_OK;
}

}  // namespace

int64_t fa_b200_decode_workspace_bytes(int32_t B, int32_t H, int32_t kv_len) {
  if (B < 0 || H < 0 || kv_len < 1) return FA_B200_ERR_SHAPE;
  if (B == 0 || H == 0) return 0;
  int splits = 1, rows = 0;
  decode_split(B, H, kv_len, &splits, &rows);
  if (splits == 1) return 0;
  return static_cast<int64_t>(B) * H * splits * fa::kDecodePartial * static_cast<int64_t>(sizeof(float));
}

namespace {

// The launch shared by fa_b200_decode and fa_b200_decode_static; they differ only in where the
// split-KV scratch lives.  `p` has been validated, the device is current and set up.
int decode_launch(const fa_b200_decode_params* p, float* scratch, int splits, int rows, bool wide) {
  fa::DecodeParams kp;
  kp.q = static_cast<const __nv_bfloat16*>(p->q);
  kp.k = static_cast<const __nv_bfloat16*>(p->k_cache);
  kp.v = static_cast<const __nv_bfloat16*>(p->v_cache);
  kp.o = static_cast<__nv_bfloat16*>(p->o);
  kp.lse = p->lse;
  kp.scratch = scratch;
  kp.q_sb = p->q_strides[0]; kp.q_sh = p->q_strides[1];
  kp.o_sb = p->o_strides[0]; kp.o_sh = p->o_strides[1];
  kp.k_sb = p->k_strides[0]; kp.k_sh = p->k_strides[1]; kp.k_sn = p->k_strides[2];
  kp.v_sb = p->v_strides[0]; kp.v_sh = p->v_strides[1]; kp.v_sn = p->v_strides[2];
  kp.B = p->B; kp.H = p->H; kp.kv_len = p->kv_len;
  kp.kv_len_ptr = p->kv_len_device;
  kp.k_new = static_cast<const __nv_bfloat16*>(p->k_new);
  kp.v_new = static_cast<const __nv_bfloat16*>(p->v_new);
  kp.new_sb = p->new_strides[0]; kp.new_sh = p->new_strides[1];
  kp.splits = splits;
  kp.rows_per_split = rows;
  const float scale = p->softmax_scale > 0.0f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(p->d));
  kp.scale_log2 = scale * 1.4426950408889634f;

  const cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  const dim3 grid(static_cast<unsigned>(p->B * p->H), static_cast<unsigned>(splits));
  if (wide) fa::fa_decode_partial_kernel<fa::kDecodeWideThreads><<<grid, fa::kDecodeWideThreads, 0, stream>>>(kp);
  else fa::fa_decode_partial_kernel<fa::kDecodeThreads><<<grid, fa::kDecodeThreads, 0, stream>>>(kp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (splits > 1) {
    fa::fa_decode_combine_kernel<<<static_cast<unsigned>(p->B * p->H), 64, 0, stream>>>(kp);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

}  // namespace

int fa_b200_decode(const fa_b200_decode_params* p) {
  int rc = decode_validate(p);
  if (rc != FA_B200_OK) return rc;
  if (p->B == 0 || p->H == 0) return FA_B200_OK;
  int splits = 1, rows = 0;
  bool wide = false;
  decode_split(p->B, p->H, p->kv_len, &splits, &rows, &wide);
  if (splits > 1) {
    const int64_t need = fa_b200_decode_workspace_bytes(p->B, p->H, p->kv_len);
    if (p->workspace == nullptr || p->workspace_bytes < need ||
        (reinterpret_cast<uintptr_t>(p->workspace) & 15u))
      return FA_B200_ERR_WORKSPACE;
  }
  DeviceGuard guard(p->device);
  if (guard.error) return guard.error;
  DeviceState* stp = nullptr;
  if ((rc = ready_device(p->device, &stp)) != 0) return rc;
  return decode_launch(p, static_cast<float*>(p->workspace), splits, rows, wide);
}

// ----------------------------------------------------------- decode without any allocation
namespace {

// Split-KV scratch compiled into the library image: one copy per GPU that loads the module.
// In host code this name is only a handle for the runtime's symbol functions, never a device
// address; kernels get the address that cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char g_fa_decode_static_scratch[FA_B200_STATIC_SCRATCH_BYTES];

struct StaticScratchState {
  std::once_flag once;
  int error = 0;          // cudaError_t of the address look-up, if it failed
  float* ptr = nullptr;   // device address of the buffer on this device
};
StaticScratchState g_static_scratch[kMaxDevices];

// Runs once per device, with that device current.
void init_static_scratch(int dev) {
  StaticScratchState& ss = g_static_scratch[dev];
  void* addr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&addr, g_fa_decode_static_scratch);
  if (e != cudaSuccess) { ss.error = static_cast<int>(e); return; }
  ss.ptr = static_cast<float*>(addr);
}

}  // namespace

int fa_b200_decode_static(const fa_b200_decode_params* p) {
  int rc = decode_validate(p);
  if (rc != FA_B200_OK) return rc;
  if (p->B == 0 || p->H == 0) return FA_B200_OK;
  int splits = 1, rows = 0;
  bool wide = false;
  decode_split(p->B, p->H, p->kv_len, &splits, &rows, &wide, /*fine_for_long=*/false);
  if (splits > 1 && static_cast<int64_t>(p->B) * p->H * splits * fa::kDecodePartial *
                            static_cast<int64_t>(sizeof(float)) > static_cast<int64_t>(FA_B200_STATIC_SCRATCH_BYTES))
    return FA_B200_ERR_STATIC_SCRATCH;

  DeviceGuard guard(p->device);
  if (guard.error) return guard.error;
  DeviceState* stp = nullptr;
  if ((rc = ready_device(p->device, &stp)) != 0) return rc;   // architecture check, no allocation
  StaticScratchState& ss = g_static_scratch[p->device];
  std::call_once(ss.once, init_static_scratch, p->device);  // first call on this device only
  if (ss.error) return ss.error;
  return decode_launch(p, ss.ptr, splits, rows, wide);
}

int fa_b200_device_ok(int device) {
  if (device < 0) return FA_B200_ERR_DEVICE;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (device >= count) return FA_B200_ERR_DEVICE;
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e != cudaSuccess) return static_cast<int>(e);
  return major == 10 ? 1 : 0;
}

int fa_b200_last_status(int device, void* stream) {
  if (device < 0 || device >= kMaxDevices) return FA_B200_ERR_DEVICE;
  DeviceGuard guard(device);
  if (guard.error) return guard.error;
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  DeviceState& st = g_dev[device];
  if (st.status == nullptr) return 0;  // no kernel was ever launched on this device
  unsigned int words[4] = {0, 0, 0, 0};
  e = cudaMemcpy(words, st.status, sizeof(words), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (words[0] != 0) {
    std::fprintf(stderr, "fa_b200: watchdog code 0x%x (block %u, thread %u, parity %u)\n", words[0],
                 words[1], words[2], words[3]);
    e = cudaMemset(st.status, 0, sizeof(words));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return static_cast<int>(words[0]);
}

// ------------------------------------------------------------------------- add + LayerNorm
extern "C++" {
namespace {

template <int kVec>
cudaError_t launch_add_ln(const fa::AddLnParams& kp, cudaStream_t stream) {
  const long long ctas = (kp.rows + fa::kLnWarpsPerCta - 1) / fa::kLnWarpsPerCta;
  fa::fa_add_layernorm_kernel<kVec><<<static_cast<unsigned>(ctas), fa::kLnWarpsPerCta * 32, 0, stream>>>(kp);
  return cudaGetLastError();
}

}  // namespace
}  // extern "C++"

int fa_b200_add_layernorm(const fa_b200_add_layernorm_params* p) {
  if (p == nullptr || p->a == nullptr || p->scale == nullptr || p->shift == nullptr ||
      p->norm_out == nullptr)
    return FA_B200_ERR_NULL;
  if (p->rows < 0 || p->cols <= 0 || (p->cols % 8) != 0 ||
      p->cols > fa::kLnMaxVecPerLane * 256)
    return FA_B200_ERR_SHAPE;
  if ((p->rows + fa::kLnWarpsPerCta - 1) / fa::kLnWarpsPerCta > 0x7fffffffLL) return FA_B200_ERR_SHAPE;
  const void* ptrs[6] = {p->a, p->resid, p->scale, p->shift, p->sum_out, p->norm_out};
  for (const void* q : ptrs)
    if (reinterpret_cast<uintptr_t>(q) & 15u) return FA_B200_ERR_ALIGN;
  if (!(p->eps >= 0.0f)) return FA_B200_ERR_SCALE;
  if (p->device < 0 || p->device >= kMaxDevices) return FA_B200_ERR_DEVICE;
  if (p->rows == 0) return FA_B200_OK;

  DeviceGuard guard(p->device);
  if (guard.error) return guard.error;
  DeviceState& st = g_dev[p->device];
  std::call_once(st.once, init_device, p->device);
  if (st.init_error) return st.init_error;

  fa::AddLnParams kp;
  kp.a = static_cast<const __nv_bfloat16*>(p->a);
  kp.resid = static_cast<const __nv_bfloat16*>(p->resid);
  kp.scale = static_cast<const __nv_bfloat16*>(p->scale);
  kp.shift = static_cast<const __nv_bfloat16*>(p->shift);
  kp.sum_out = static_cast<__nv_bfloat16*>(p->sum_out);
  kp.norm_out = static_cast<__nv_bfloat16*>(p->norm_out);
  kp.rows = p->rows;
  kp.cols = p->cols;
  kp.eps = p->eps;
  const cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  cudaError_t e;
  switch ((p->cols + 255) / 256) {   // 16-byte vectors per lane
    case 1: e = launch_add_ln<1>(kp, stream); break;
    case 2: e = launch_add_ln<2>(kp, stream); break;
    case 3: e = launch_add_ln<3>(kp, stream); break;
    case 4: e = launch_add_ln<4>(kp, stream); break;
    case 5: e = launch_add_ln<5>(kp, stream); break;
    case 6: e = launch_add_ln<6>(kp, stream); break;
    case 7: e = launch_add_ln<7>(kp, stream); break;
    default: e = launch_add_ln<8>(kp, stream); break;
  }
  return static_cast<int>(e);
}

// ------------------------------------------------------------------- Linear for a few rows
extern "C++" {
namespace {

constexpr int kLinSmemLimit = 128 * 1024;
std::once_flag g_lin_once[kMaxDevices];
int g_lin_error[kMaxDevices];

template <int kRows>
cudaError_t lin_prepare() {
  cudaError_t e = cudaFuncSetAttribute(
      reinterpret_cast<const void*>(&fa::fa_linear_small_kernel<kRows, fa::kLinUnrollShort>),
      cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmemLimit);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(
      reinterpret_cast<const void*>(&fa::fa_linear_small_kernel<kRows, fa::kLinUnrollLong>),
      cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmemLimit);
}
void lin_init(int dev) {   // with `dev` current
  cudaError_t e = lin_prepare<1>();
  if (e == cudaSuccess) e = lin_prepare<2>();
  if (e == cudaSuccess) e = lin_prepare<4>();
  if (e == cudaSuccess) e = lin_prepare<8>();
  g_lin_error[dev] = static_cast<int>(e);
}
template <int kRows>
cudaError_t lin_launch(const fa::LinearSmallParams& kp, cudaStream_t stream, int sm_count) {
  const size_t smem = static_cast<size_t>(kRows) * kp.K * 2;
  // as many CTAs per SM as ~200 KB of shared memory hold (1..8): every CTA stages x once
  long long per_sm = (200 * 1024) / static_cast<long long>(smem > 0 ? smem : 1);
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  long long ctas = (kp.N + fa::kLinWarps - 1) / fa::kLinWarps;
  if (ctas > per_sm * sm_count) ctas = per_sm * sm_count;
  // more loads in flight per lane pay for long rows and for many columns per warp (measured:
  // the vocabulary head 31 -> 28 us, K = 6400 9.2 -> 8.2 us; the short layers are better with 4)
  if (kp.K > 2048 || kp.N >= 16384)
    fa::fa_linear_small_kernel<kRows, fa::kLinUnrollLong><<<static_cast<unsigned>(ctas), fa::kLinWarps * 32, smem, stream>>>(kp);
  else
    fa::fa_linear_small_kernel<kRows, fa::kLinUnrollShort><<<static_cast<unsigned>(ctas), fa::kLinWarps * 32, smem, stream>>>(kp);
  return cudaGetLastError();
}

}  // namespace
}  // extern "C++"

int fa_b200_linear_small(const fa_b200_linear_small_params* p) {
  if (p == nullptr || p->x == nullptr || p->w == nullptr || p->y == nullptr) return FA_B200_ERR_NULL;
  if (p->M < 1 || p->M > fa::kLinMaxRows || p->N < 0 || p->K <= 0 || (p->K % 8) != 0)
    return FA_B200_ERR_SHAPE;
  const int rows = p->M <= 1 ? 1 : (p->M <= 2 ? 2 : (p->M <= 4 ? 4 : 8));
  if (static_cast<long long>(rows) * p->K * 2 > kLinSmemLimit) return FA_B200_ERR_SHAPE;
  if (p->act != 0 && p->act != 1) return FA_B200_ERR_SHAPE;
  if (p->ldw < p->K || (p->ldw % 8) != 0) return FA_B200_ERR_STRIDE;
  if ((reinterpret_cast<uintptr_t>(p->x) & 15u) || (reinterpret_cast<uintptr_t>(p->w) & 15u) ||
      (reinterpret_cast<uintptr_t>(p->y) & 15u) || (reinterpret_cast<uintptr_t>(p->bias) & 1u))
    return FA_B200_ERR_ALIGN;
  const bool prologue = p->resid != nullptr || p->ln_scale != nullptr || p->sum_out != nullptr;
  if (prologue) {
    if ((p->ln_scale == nullptr) != (p->ln_shift == nullptr)) return FA_B200_ERR_NULL;
    if (p->K > 256 * 8) return FA_B200_ERR_SHAPE;
    const void* extra[4] = {p->resid, p->ln_scale, p->ln_shift, p->sum_out};
    for (const void* q : extra)
      if (reinterpret_cast<uintptr_t>(q) & 15u) return FA_B200_ERR_ALIGN;
    if (p->sum_out != nullptr && (p->sum_out == p->x || p->sum_out == p->resid)) return FA_B200_ERR_ALIAS;
    if (p->ln_scale != nullptr && !(p->eps >= 0.0f)) return FA_B200_ERR_SCALE;
  }
  if (p->device < 0 || p->device >= kMaxDevices) return FA_B200_ERR_DEVICE;
  if (p->N == 0) return FA_B200_OK;

  DeviceGuard guard(p->device);
  if (guard.error) return guard.error;
  DeviceState& st = g_dev[p->device];
  std::call_once(st.once, init_device, p->device);
  if (st.init_error) return st.init_error;
  std::call_once(g_lin_once[p->device], lin_init, p->device);
  if (g_lin_error[p->device]) return g_lin_error[p->device];

  fa::LinearSmallParams kp;
  kp.x = static_cast<const __nv_bfloat16*>(p->x);
  kp.w = static_cast<const __nv_bfloat16*>(p->w);
  kp.bias = static_cast<const __nv_bfloat16*>(p->bias);
  kp.y = static_cast<__nv_bfloat16*>(p->y);
  kp.M = p->M; kp.N = p->N; kp.K = p->K;
  kp.ldw = p->ldw;
  kp.act = p->act;
  kp.resid = static_cast<const __nv_bfloat16*>(p->resid);
  kp.ln_scale = static_cast<const __nv_bfloat16*>(p->ln_scale);
  kp.ln_shift = static_cast<const __nv_bfloat16*>(p->ln_shift);
  kp.sum_out = static_cast<__nv_bfloat16*>(p->sum_out);
  kp.eps = p->eps;
  const cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  cudaError_t e;
  switch (rows) {
    case 1: e = lin_launch<1>(kp, stream, st.sm_count); break;
    case 2: e = lin_launch<2>(kp, stream, st.sm_count); break;
    case 4: e = lin_launch<4>(kp, stream, st.sm_count); break;
    default: e = lin_launch<8>(kp, stream, st.sm_count); break;
  }
  return static_cast<int>(e);
}

#ifdef FA_TRACE
// Trace builds only: choose the traced CTA / copy the trace buffer to the host (synchronises).
int fa_b200_trace_select(int block) {
  return static_cast<int>(cudaMemcpyToSymbol(fa::g_fa_trace_block, &block, sizeof(int)));
}
int fa_b200_trace_read(unsigned long long* out, int n) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (n > fa::kTraceSlots) n = fa::kTraceSlots;
  return static_cast<int>(cudaMemcpyFromSymbol(out, fa::g_fa_trace, sizeof(unsigned long long) * n));
}
#endif

const char* fa_b200_strerror(int code) {
  switch (code) {
    case FA_B200_OK: return "ok";
    case FA_B200_ERR_NULL: return "fa_b200: params, q, k, v or o is NULL";
    case FA_B200_ERR_HEAD_DIM: return "fa_b200: head dimension must be 64";
    case FA_B200_ERR_SHAPE: return "fa_b200: B, H, N must be non-negative and within kernel limits";
    case FA_B200_ERR_STRIDE: return "fa_b200: strides must be positive multiples of 8 elements (16 bytes)";
    case FA_B200_ERR_ALIGN: return "fa_b200: q, k, v, o must be 16-byte aligned (lse 4-byte)";
    case FA_B200_ERR_SCALE: return "fa_b200: softmax_scale must be finite and >= 0 (0 selects 1/sqrt(d))";
    case FA_B200_ERR_DEVICE: return "fa_b200: bad device ordinal";
    case FA_B200_ERR_ARCH: return "fa_b200: device is not compute capability 10.x (B200); there is no fallback";
    case FA_B200_ERR_TENSORMAP: return "fa_b200: the driver rejected a TMA tensor map (check strides and sizes)";
    case FA_B200_ERR_DRIVER: return "fa_b200: cuTensorMapEncodeTiled is not available from this driver";
    case FA_B200_ERR_STATIC_SCRATCH: return "fa_b200: this decode problem needs more split-KV scratch than the built-in buffer holds (FA_B200_STATIC_SCRATCH_BYTES); use fa_b200_decode with a workspace";
    case FA_B200_ERR_ALIAS: return "fa_b200: an output buffer overlaps an input it must not overlap";
    case FA_B200_ERR_WORKSPACE: return "fa_b200: decode workspace is NULL, too small or not 16-byte aligned";
    case FA_B200_ERR_BUILD: return "fa_b200: the kernel image does not match this library's launch configuration; rebuild it";
    default: break;
  }
  if (code > static_cast<int>(fa::kWatchdogBase)) {
    switch (code & 0xff) {
      case fa::kWaitQFull: return "fa_b200 watchdog: wait for the Q tile load ran out";
      case fa::kWaitKVFull: return "fa_b200 watchdog: wait for a K/V tile load ran out";
      case fa::kWaitKVEmpty: return "fa_b200 watchdog: wait for a free K/V slot ran out";
      case fa::kWaitSFull: return "fa_b200 watchdog: wait for S = QK^T ran out";
      case fa::kWaitPFull: return "fa_b200 watchdog: wait for P from the softmax warps ran out";
      case fa::kWaitSFree: return "fa_b200 watchdog: wait for the softmax warps to take S ran out";
      case fa::kWaitOFree: return "fa_b200 watchdog: wait for the epilogue to read O ran out";
      case fa::kWaitQEmpty: return "fa_b200 watchdog: wait for the Q slot to be released ran out";
      case fa::kWaitOFull: return "fa_b200 watchdog: wait for O += PV ran out";
      default: return "fa_b200 watchdog: a bounded wait ran out";
    }
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "fa_b200: unknown error code";
}

}  // extern "C"
