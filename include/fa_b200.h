/*
 * fa_b200.h -- C ABI of libfa_b200.so: FlashAttention forward for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a foreign-function binding (ctypes, pybind11, cgo ...) binds to.
 * It replaces the host launcher of the reference project,
 *
 *   template <typename T> cudaError_t flashattention_forward(T* O, const T* Q, const T* K,
 *       const T* V, int seq_len, int batch_size, int num_heads);
 *   (reference: src/cpp/v1.cu:4-38, declared again in src/cpp/torch_bind.cpp:9-11)
 *
 * which the reference's torch extension `custom_flash_attn.forward(Q, K, V)` calls
 * (reference: src/cpp/torch_bind.cpp:21-49).  Differences that a caller sees:
 *   - plain C symbols, plain pointers and sizes, no torch types, no exceptions;
 *   - explicit device and stream instead of device 0 / the legacy default stream;
 *   - explicit element strides (the innermost stride is always 1);
 *   - a `causal` flag (the reference is always causal) and an optional LSE output;
 *   - the error code is returned and has a message (the reference drops it).
 *
 * Conventions
 *   - q, k, v, o are bf16 device pointers addressing logical [B, H, N, d] tensors, d == 64.
 *   - strides are in ELEMENTS, order {batch, head, row}; each must be a multiple of 8
 *     (16 bytes) and the base pointers must be 16-byte aligned.
 *   - lse, when not NULL, is a contiguous fp32 [B, H, N] device buffer that receives
 *     logsumexp_j(softmax_scale * q_i . k_j) in natural-log units.
 *   - return value: 0 = kernel enqueued; < 0 = argument error, no CUDA call was made;
 *     > 0 = a cudaError_t from the CUDA runtime.
 *   - all entry points are thread-safe; calls on different devices do not share state.
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_B200_ABI_VERSION 4

/* argument errors (negative return values) */
#define FA_B200_OK                 0
#define FA_B200_ERR_NULL          -1  /* params, q, k, v or o is NULL                      */
#define FA_B200_ERR_HEAD_DIM      -2  /* d != 64                                           */
#define FA_B200_ERR_SHAPE         -3  /* B, H or N negative, or too large for the kernel   */
#define FA_B200_ERR_STRIDE        -4  /* a stride is <= 0 or not a multiple of 8 elements  */
#define FA_B200_ERR_ALIGN         -5  /* a base pointer is not 16-byte aligned             */
#define FA_B200_ERR_SCALE         -6  /* softmax_scale is NaN, infinite or negative        */
#define FA_B200_ERR_DEVICE        -7  /* device index negative                             */
#define FA_B200_ERR_ARCH          -8  /* device is not compute capability 10.x             */
#define FA_B200_ERR_TENSORMAP     -9  /* the driver refused a TMA descriptor               */
#define FA_B200_ERR_DRIVER       -10  /* cuTensorMapEncodeTiled could not be resolved      */
#define FA_B200_ERR_BUILD        -11  /* kernel image / launch configuration mismatch         */
#define FA_B200_ERR_WORKSPACE    -12  /* decode workspace NULL, too small or misaligned    */
#define FA_B200_ERR_STATIC_SCRATCH -13 /* problem needs more than FA_B200_STATIC_SCRATCH_BYTES */
#define FA_B200_ERR_ALIAS        -14  /* an output overlaps an input it must not overlap   */

typedef struct fa_b200_params {
  const void* q;            /* bf16 [B,H,N,d] */
  const void* k;            /* bf16 [B,H,N,d] */
  const void* v;            /* bf16 [B,H,N,d] */
  void*       o;            /* bf16 [B,H,N,d], written */
  float*      lse;          /* fp32 [B,H,N] contiguous, written; may be NULL */
  int32_t     B, H, N, d;   /* d must be 64 */
  int64_t     q_strides[3]; /* elements: {batch, head, row} */
  int64_t     k_strides[3];
  int64_t     v_strides[3];
  int64_t     o_strides[3];
  float       softmax_scale; /* 0 selects 1/sqrt(d), the reference's fixed scale (v1.cu:17) */
  int32_t     causal;        /* non-zero: row i attends columns j <= i (the reference's only mode,
                                v1_implementation.hpp:108-112); zero: full attention */
  int32_t     device;        /* CUDA device ordinal that owns all pointers */
  void*       stream;        /* cudaStream_t; NULL = that device's default stream */
} fa_b200_params;

/* Enqueue one attention forward on p->stream.  Asynchronous: returns once the kernel is
 * launched, like the reference launcher (v1.cu:29-37).  Replaces flashattention_forward<T>
 * (reference src/cpp/v1.cu:4-38). */
int fa_b200_fwd(const fa_b200_params* p);

/* How fa_b200_fwd would schedule this problem on p->device, without launching anything.  The
 * reference launcher has one fixed shape, a CTA per 32-row tile (grid (ceil(N/32), H, B),
 * src/cpp/v1.cu:13-14, 25-34); this library picks one of four kernel schedules per call and this
 * query reports the pick, so that a test or a tuning run can tell which code ran:
 *   FA_B200_SCHEDULE_CTA_PER_TILE        one CTA per 128-row query tile, heaviest causal tile first
 *   FA_B200_SCHEDULE_PERSISTENT_PAIRED   resident CTAs, causal, complementary tile pairs
 *   FA_B200_SCHEDULE_PERSISTENT_ROTATED  resident CTAs, causal, odd tile count (rotated order)
 *   FA_B200_SCHEDULE_PERSISTENT_FULL     resident CTAs, non-causal
 *   FA_B200_SCHEDULE_NONE                empty problem, nothing is launched
 * *grid receives the number of CTAs.  Either output pointer may be NULL.  Arguments are checked as
 * by fa_b200_fwd; the first call on a device performs the same one-time device set-up. */
#define FA_B200_SCHEDULE_NONE               -1
#define FA_B200_SCHEDULE_CTA_PER_TILE        0
#define FA_B200_SCHEDULE_PERSISTENT_PAIRED   1
#define FA_B200_SCHEDULE_PERSISTENT_ROTATED  2
#define FA_B200_SCHEDULE_PERSISTENT_FULL     3
int fa_b200_fwd_plan(const fa_b200_params* p, int32_t* schedule, int32_t* grid);

/* Check arguments exactly as fa_b200_fwd does, without touching CUDA.  Returns 0 or a negative
 * FA_B200_ERR_* code.  Covers what CHECK_INPUT and the dtype branch police in the reference
 * binding (src/cpp/torch_bind.cpp:13-19, 33-42), plus what it leaves unchecked (size(3)). */
int fa_b200_validate(const fa_b200_params* p);

/* Message for a value returned by any function here (negative: argument error, positive:
 * cudaGetErrorString).  The returned pointer stays valid for the life of the process. */
const char* fa_b200_strerror(int code);

/* 1 if `device` exists and is compute capability 10.x, 0 if it exists and is not, negative /
 * positive error otherwise.  The reference has no such check (it queries device 0 on every
 * call, src/cpp/v1.cu:7-8). */
int fa_b200_device_ok(int device);

/* Synchronise `stream` on `device`, then return and clear the device-side watchdog word.
 * Every wait inside the kernel is bounded; a wait that runs out records which one it was and
 * the kernel drains and exits.  0 = all kernels since the last call finished normally;
 * > 0x10000 = watchdog code (see fa_b200_strerror); other values = cudaError_t.
 * The reference has no counterpart (its cudaGetLastError result is dropped,
 * src/cpp/torch_bind.cpp:34-39). */
int fa_b200_last_status(int device, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Single-query ("decode") attention against a K/V cache: one new token per sequence.
 *
 *   o[b,h,:] = softmax_j(scale * q[b,h,:] . k[b,h,j,:]) v[b,h,j,:],   0 <= j < kv_len
 *
 * The reference has no such entry point: its generate() re-runs the whole prefix through the
 * prefill kernel for every new token (src/py/model_inference.py:199-228).  This is the attention
 * step of the same loop with a KV cache.
 *
 * q and o are bf16 [B, H, 64] (strides {batch, head} in elements, multiples of 8); the caches are
 * bf16 [B, H, >= kv_len, 64] with strides {batch, head, row}; lse (optional) is fp32 [B, H].
 * With few (batch, head) pairs and a long cache the keys of a head are processed in several chunks
 * whose partial results pass through `workspace` (few pairs with at most 4096 rows run as one
 * wide CTA per head and need none): device memory of at least
 * fa_b200_decode_workspace_bytes(B, H, kv_len) bytes, 16-byte aligned, owned by the caller and not
 * shared by calls that may overlap on the GPU (it may be NULL when that function returns 0).
 */
typedef struct fa_b200_decode_params {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  void*       o;
  float*      lse;            /* may be NULL */
  void*       workspace;      /* see above */
  int64_t     workspace_bytes;
  int32_t     B, H, kv_len, d;   /* d must be 64, kv_len >= 1 */
  int64_t     q_strides[2];   /* elements: {batch, head} */
  int64_t     o_strides[2];
  int64_t     k_strides[3];   /* elements: {batch, head, row} */
  int64_t     v_strides[3];
  float       softmax_scale;  /* 0 selects 1/sqrt(d) */
  int32_t     device;
  void*       stream;
  /* Optional (ABI version 2).  When not NULL: device address of an int32 that holds the current
   * number of valid cache rows; the kernel reads it when it RUNS, so one recorded launch (a CUDA
   * graph node) serves every step of a generation loop while the host only bumps that counter on
   * the device.  kv_len is then the upper bound the launch is sized for (grid, workspace); the
   * value read is clamped to [1, kv_len]. */
  const int32_t* kv_len_device;
  /* Optional (ABI version 3): the cache append of the step, folded into the kernel.  When k_new
   * is not NULL, k_new / v_new are bf16 [B, H, 64] (element strides new_strides = {batch, head},
   * multiples of 8; 16-byte aligned) holding the key / value of the token being generated: the
   * kernel uses them as row (length - 1), where length is kv_len or the value read through
   * kv_len_device, and stores them into that row of k_cache / v_cache (which it therefore
   * writes).  Both or neither. */
  const void* k_new;
  const void* v_new;
  int64_t     new_strides[2];
} fa_b200_decode_params;

/* Bytes of workspace fa_b200_decode needs for this problem size (0 when the keys of a head are
 * not split).  Negative on bad arguments.  No CUDA call is made. */
int64_t fa_b200_decode_workspace_bytes(int32_t B, int32_t H, int32_t kv_len);

/* Enqueue one decode-attention step on p->stream.  Return values as fa_b200_fwd;
 * FA_B200_ERR_WORKSPACE when the workspace is missing, too small or misaligned. */
int fa_b200_decode(const fa_b200_decode_params* p);

/* Largest split-KV scratch fa_b200_decode_static can serve, in bytes (the size of the buffer that
 * is compiled into the library; it occupies this much memory on every GPU that loads the library,
 * until the process exits). */
#define FA_B200_STATIC_SCRATCH_BYTES (256 * 1024)

/* fa_b200_decode for callers that must not allocate device memory and have none to lend: the
 * split-KV partial results go to a fixed buffer that lives inside the library image instead of
 * p->workspace (p->workspace and p->workspace_bytes are ignored).  Typical callers: a serving
 * process whose framework has already claimed all device memory for its own pool, so that a
 * cudaMalloc from a plug-in fails or is forbidden; a request path on which cudaMalloc / cudaFree
 * are banned because they can synchronise the whole device and stall every other stream; a small
 * C host with a fixed memory map and no allocator to call.  This function itself calls no
 * cudaMalloc, cudaFree or other allocating routine.
 *
 *   - The keys of a head are cut into 592 / (B * H) chunks of at least 64 rows (fa_b200_decode
 *     cuts caches of 2048 rows and more finer than that, which this entry point does not follow,
 *     so that what fits the buffer does not move with that tuning).  Problems whose partial
 *     results -- 264 bytes per (batch, head) pair and chunk -- exceed FA_B200_STATIC_SCRATCH_BYTES
 *     are refused with FA_B200_ERR_STATIC_SCRATCH; nothing is launched.  (Up to 496 (batch, head)
 *     pairs always fit; from 592 pairs on no scratch is used.)
 *   - The first call on each device looks up the buffer's device address; make that first call
 *     outside of any stream capture.
 *   - All calls on a device share the one buffer, and it keeps whatever the previous call left in
 *     it.  Nothing in it needs clearing -- every partial result is written before it is read --
 *     but two calls that may run on the GPU at the same time (different streams, different host
 *     threads) race on it: serialise them, or use fa_b200_decode with separate workspaces.
 *
 * Results are identical to fa_b200_decode wherever both cut the keys into the same chunks, and
 * equal within rounding otherwise.  This entry point has no counterpart in the reference. */
int fa_b200_decode_static(const fa_b200_decode_params* p);

/* Residual add + LayerNorm in one pass (bf16 in / out, fp32 arithmetic), for the transformer block
 * around the attention call:
 *
 *     s = a + resid                         resid may be NULL (plain LayerNorm)
 *     if (sum_out) sum_out = s              the new residual stream, rounded to bf16
 *     norm_out = (s - mean) / sqrt(var + eps) * scale + shift      (biased variance, per row)
 *
 * Replaces the reference's LayerNorm.forward (src/py/model_inference.py:102-107, about ten
 * elementwise kernels) together with the shortcut additions of TransformerBlock.forward
 * (:156, :163).  All matrices are dense row-major [rows, cols] bf16, scale / shift [cols] bf16;
 * every pointer 16-byte aligned; cols a positive multiple of 8 and at most 2048; rows >= 0
 * (rows == 0 is a no-op).  When sum_out is given, the row that is normalised is the bf16-rounded
 * sum, i.e. exactly what a later reader of sum_out sees.  sum_out may alias a or resid; norm_out
 * may alias a.  Asynchronous on p->stream.  Errors: FA_B200_ERR_NULL, _SHAPE, _ALIGN, _DEVICE,
 * _ARCH, or a positive cudaError_t. */
typedef struct fa_b200_add_layernorm_params {
  const void* a;
  const void* resid;      /* or NULL */
  const void* scale;
  const void* shift;
  void* sum_out;          /* or NULL */
  void* norm_out;
  int64_t rows;
  int32_t cols;
  float eps;
  int32_t device;
  void* stream;
} fa_b200_add_layernorm_params;

int fa_b200_add_layernorm(const fa_b200_add_layernorm_params* p);

/* y = act(x W^T + bias) for at most 8 rows of x (the Linear layers of a generation step):
 * x [M, K], W [N, K] with row stride ldw (elements; the layout of torch.nn.Linear.weight), bias
 * [N] or NULL, y [M, N]; all bf16, fp32 accumulation; act 0 = none, 1 = tanh-GELU.
 *
 * Replaces, for single-token steps, the nn.Linear calls of the reference's attention module
 * (src/py/model_inference.py:50-53, 93), feed-forward (:121-125 with the GELU of :109-117) and
 * output head (:190).  HBM-bound on reading W once.  1 <= M <= 8; K a positive multiple of 8 with
 * M_padded * K * 2 bytes <= 128 KiB (M_padded = M rounded up to 1, 2, 4 or 8); ldw >= K, a
 * multiple of 8; x, W, y 16-byte aligned, bias 2-byte aligned.  N == 0 is a no-op.  Asynchronous on
 * p->stream.  Errors: FA_B200_ERR_NULL, _SHAPE, _STRIDE, _ALIGN, _DEVICE, _ARCH or a positive
 * cudaError_t. */
typedef struct fa_b200_linear_small_params {
  const void* x;
  const void* w;
  const void* bias;       /* or NULL */
  void* y;
  int32_t M, N, K;
  int64_t ldw;
  int32_t act;
  int32_t device;
  void* stream;
  /* Optional prologue on x, fused into the kernel (all NULL = none; needs K <= 2048):
   *   x <- x + resid               resid [M, K] bf16 or NULL
   *   sum_out <- bf16(x)           [M, K] or NULL: the new residual stream; must not be x or resid
   *   x <- LayerNorm(x) * ln_scale + ln_shift     ln_scale / ln_shift [K] bf16, both or neither
   * i.e. fa_b200_add_layernorm followed by this layer, without the separate kernel: the shortcut
   * addition and LayerNorm that precede the QKV projection, the first MLP layer and the output
   * head in the reference's block (src/py/model_inference.py:102-107, 153-163, 188-190).  When
   * sum_out is given, the normalised row is the bf16-rounded sum. */
  const void* resid;
  const void* ln_scale;
  const void* ln_shift;
  void* sum_out;
  float eps;
} fa_b200_linear_small_params;

int fa_b200_linear_small(const fa_b200_linear_small_params* p);

/* FA_B200_ABI_VERSION the library was built with. */
int fa_b200_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
