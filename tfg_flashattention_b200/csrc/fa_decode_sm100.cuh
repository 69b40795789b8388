// Single-query ("decode") attention for sm_100a: one new token per sequence attends a K/V cache.
//
//   o[b,h,:] = softmax_j(scale * q[b,h,:] . k[b,h,j,:]) v[b,h,j,:],   j < kv_len
//
// This is the attention of autoregressive generation with a KV cache (the reference generates by
// re-running the whole prefix for every token, src/py/model_inference.py:199-228).  One query row
// gives the tensor cores nothing to do; the kernel is bound by reading K and V once from HBM
// (2 * kv_len * 128 bytes per head), so it is written for bandwidth: 16-byte loads, 8 lanes per
// 128-byte row, several rows in flight per lane group, fp32 online softmax in registers.
//
// Split-KV: with few (batch, head) pairs a head's keys are cut into `splits` chunks so that the
// grid fills the GPU; every chunk leaves an unnormalised partial (max, sum, o[64]) in a scratch
// buffer and a second, tiny kernel merges the chunks.  With splits == 1 the first kernel writes
// the final result and the scratch buffer is not touched.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace fa {

constexpr int kDecodeThreads = 128;          // a warp's 32 lanes = 4 groups of 8 lanes
constexpr int kDecodeGroups = kDecodeThreads / 8;   // 16 lane groups, each owns whole rows
constexpr int kDecodeWideThreads = 1024;            // the one-CTA-per-head form for few heads
constexpr int kDecodeUnroll = 4;             // rows in flight per lane group (8: 3.3-4.0 TB/s against 4.3-5.2)
constexpr int kDecodePartial = 66;           // floats per partial: m, l, o[64]

struct DecodeParams {
  const __nv_bfloat16* q;      // [B, H, 64]
  const __nv_bfloat16* k;      // [B, H, kv_len.., 64] with strides below
  const __nv_bfloat16* v;
  __nv_bfloat16* o;            // [B, H, 64]
  float* lse;                  // [B, H] or null
  float* scratch;              // [B*H, splits, 66] floats when splits > 1
  long long q_sb, q_sh;        // element strides of q and o: batch, head
  long long o_sb, o_sh;
  long long k_sb, k_sh, k_sn;  // element strides of the caches: batch, head, row
  long long v_sb, v_sh, v_sn;
  int B, H, kv_len;
  int splits;                  // chunks per head
  int rows_per_split;          // multiple of kDecodeGroups
  float scale_log2;            // softmax_scale * log2(e)
  // when set: the newest row (index length - 1) is taken from these [B, H, 64] buffers instead of
  // the caches and written into the caches by the CTA that owns it (the cache append of a
  // generation step, folded into the attention kernel)
  const __nv_bfloat16* k_new = nullptr;
  const __nv_bfloat16* v_new = nullptr;
  long long new_sb = 0, new_sh = 0;
  const int* kv_len_ptr = nullptr;   // when set: the current length lives in device memory (read
                                     // at run time, clamped to [1, kv_len]); kv_len is the bound
                                     // the grid and the chunks were sized for
};

__device__ __forceinline__ void bf16x8_to_float(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// grid (B*H, splits), block kThreads.  Lane group g = tid / 8 owns rows g, g + kGroups, ... of the
// chunk; lane c = tid % 8 owns columns 8c .. 8c+7 of every row.  kThreads = 128 is the split-KV
// form; kThreads = 1024 (always with splits == 1) serves problems with few (batch, head) pairs and
// short caches in ONE launch: a head's keys stream through one SM (a few hundred KB), and the
// 128 lane groups are merged inside the CTA, with no scratch buffer and no second kernel -- at
// batch 1 the two launches of the split form cost more than the attention itself.
template <int kThreads>
__global__ void __launch_bounds__(kThreads) fa_decode_partial_kernel(const DecodeParams p) {
  constexpr int kGroups = kThreads / 8;
  // rows in flight per lane group: the wide form has 64 registers per thread and 8x the threads
  constexpr int kUnroll = kThreads > 256 ? 2 : kDecodeUnroll;
  const int bh = blockIdx.x;
  const int split = blockIdx.y;
  const int b = bh / p.H;
  const int h = bh - b * p.H;
  const int tid = threadIdx.x;
  const int g = tid >> 3;
  const int c = tid & 7;

  float qf[8];
  {
    const uint4 raw = *reinterpret_cast<const uint4*>(p.q + b * p.q_sb + h * p.q_sh + 8 * c);
    bf16x8_to_float(raw, qf);
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[i] *= p.scale_log2;     // scores come out in exp2 units
  }
  const __nv_bfloat16* kbase = p.k + b * p.k_sb + h * p.k_sh + 8 * c;
  const __nv_bfloat16* vbase = p.v + b * p.v_sb + h * p.v_sh + 8 * c;
  const __nv_bfloat16* knew = p.k_new ? p.k_new + b * p.new_sb + h * p.new_sh + 8 * c : nullptr;
  const __nv_bfloat16* vnew = p.k_new ? p.v_new + b * p.new_sb + h * p.new_sh + 8 * c : nullptr;
  const int kv_len = p.kv_len_ptr ? max(1, min(__ldg(p.kv_len_ptr), p.kv_len)) : p.kv_len;
  const int row_begin = split * p.rows_per_split;
  const int row_end = min(kv_len, row_begin + p.rows_per_split);   // chunks past the end stay empty

  float m = -CUDART_INF_F, l = 0.f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  // The loop bounds are the same for every thread of the CTA (the shuffles below name the whole
  // warp); which rows exist is decided per lane group inside.
  for (int base = row_begin; base < row_end; base += kGroups * kUnroll) {
    const int r0 = base + g;
    uint4 kraw[kUnroll], vraw[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {           // all loads first: rows in flight
      const int r = r0 + u * kGroups;
      if (r < row_end) {
        const bool fresh = knew != nullptr && r == kv_len - 1;   // the row being appended
        // streaming loads: every cache byte is read once per step
        kraw[u] = __ldcs(reinterpret_cast<const uint4*>(fresh ? knew : kbase + (long long)r * p.k_sn));
        vraw[u] = __ldcs(reinterpret_cast<const uint4*>(fresh ? vnew : vbase + (long long)r * p.v_sn));
        if (fresh) {
          *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(kbase) + (long long)r * p.k_sn) = kraw[u];
          *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(vbase) + (long long)r * p.v_sn) = vraw[u];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int r = r0 + u * kGroups;
      // the 8 lanes of a group must all run the shuffles; rows past the end contribute nothing
      float kf[8], s = 0.f;
      if (r < row_end) {
        bf16x8_to_float(kraw[u], kf);
#pragma unroll
        for (int i = 0; i < 8; ++i) s = fmaf(qf[i], kf[i], s);
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (r < row_end) {
        const float m_new = fmaxf(m, s);
        const float f = exp2f(m - m_new);               // 0 on the first row (m = -inf)
        const float pr = exp2f(s - m_new);
        float vf[8];
        bf16x8_to_float(vraw[u], vf);
        l = l * f + pr;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(pr, vf[i], acc[i] * f);
        m = m_new;
      }
    }
  }

  // ---- merge the lane groups of the CTA: (m, l, acc) per group, columns stay with lane c.
  // The wide form first folds the four groups of every warp with shuffles, so that shared memory
  // and the final loop see one entry per warp (32) instead of one per group (128).
  constexpr int kEntries = kThreads > 256 ? kThreads / 32 : kGroups;
  if constexpr (kThreads > 256) {
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m, off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l, off);
      const float m_n = fmaxf(m, m_o);
      const float f_a = m == -CUDART_INF_F ? 0.f : exp2f(m - m_n);     // empty groups carry -inf
      const float f_b = m_o == -CUDART_INF_F ? 0.f : exp2f(m_o - m_n);
      l = l * f_a + l_o * f_b;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = acc[i] * f_a + __shfl_xor_sync(0xffffffffu, acc[i], off) * f_b;
      m = m_n;
    }
  }
  const int entry = kThreads > 256 ? tid >> 5 : g;
  const bool writer = kThreads > 256 ? (tid & 31) < 8 : true;          // one group per warp writes
  __shared__ float sm_m[kEntries], sm_l[kEntries];
  __shared__ float sm_o[kEntries][64];
  if (writer) {
    if (c == 0) { sm_m[entry] = m; sm_l[entry] = l; }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_o[entry][8 * c + i] = acc[i];
  }
  __syncthreads();
  if (tid < 64) {
    float mm = -CUDART_INF_F;
#pragma unroll 16
    for (int i = 0; i < kEntries; ++i) mm = fmaxf(mm, sm_m[i]);
    float ll = 0.f, oo = 0.f;
#pragma unroll 16
    for (int i = 0; i < kEntries; ++i) {
      const float f = sm_m[i] == -CUDART_INF_F ? 0.f : exp2f(sm_m[i] - mm);   // empty entries
      ll += sm_l[i] * f;
      oo += sm_o[i][tid] * f;
    }
    if (p.splits == 1) {
      p.o[b * p.o_sb + h * p.o_sh + tid] = __float2bfloat16_rn(oo / ll);
      if (tid == 0 && p.lse != nullptr)
        p.lse[bh] = 0.6931471805599453f * (mm + log2f(ll));
    } else {
      float* part = p.scratch + ((long long)bh * p.splits + split) * kDecodePartial;
      if (tid == 0) { part[0] = mm; part[1] = ll; }
      part[2 + tid] = oo;
    }
  }
}

// grid B*H, block 64: merge the `splits` partials of one head.
__global__ void __launch_bounds__(64) fa_decode_combine_kernel(const DecodeParams p) {
  const int bh = blockIdx.x;
  const int b = bh / p.H;
  const int h = bh - b * p.H;
  const int tid = threadIdx.x;
  const float* part = p.scratch + (long long)bh * p.splits * kDecodePartial;
  float mm = -CUDART_INF_F;
  for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, part[s * kDecodePartial]);
  float ll = 0.f, oo = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float ms = part[s * kDecodePartial];
    const float f = ms == -CUDART_INF_F ? 0.f : exp2f(ms - mm);   // chunk past kv_len
    ll += part[s * kDecodePartial + 1] * f;
    oo += part[s * kDecodePartial + 2 + tid] * f;
  }
  p.o[b * p.o_sb + h * p.o_sh + tid] = __float2bfloat16_rn(oo / ll);
  if (tid == 0 && p.lse != nullptr) p.lse[bh] = 0.6931471805599453f * (mm + log2f(ll));
}

}  // namespace fa
