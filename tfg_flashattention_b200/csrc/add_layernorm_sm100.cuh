// Residual add + LayerNorm in one pass over HBM, bf16 in / bf16 out, fp32 arithmetic.
//
//   s = a + resid            (resid optional; s optionally written: the new residual stream)
//   y = (s - mean(s)) / sqrt(var(s) + eps) * scale + shift     (biased variance)
//
// This is the reference's LayerNorm (src/py/model_inference.py:96-107: mean, var(unbiased=False),
// eps 1e-5, scale / shift) fused with the shortcut addition that precedes it in every transformer
// block (:156-163).  The reference spends ~10 elementwise launches on it; torch's fused
// layer_norm plus a separate add move the activation through HBM five times.  Here each row is
// read once (twice with a residual) and written once (twice when the sum is kept): the kernel is
// bound by HBM bandwidth, (2 or 4) * cols * 2 bytes per row.
//
// One warp per row: the row lives in registers (16-byte loads, 8 bf16 per lane and step), mean and
// variance are two warp reductions over registers (exact two-pass form, no E[x^2] cancellation),
// no shared memory.  kVecPerLane = ceil(cols / 256) steps per lane, a template parameter so that
// the register array is fully unrolled; cols must be a multiple of 8 and at most 256 * 8.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa {

constexpr int kLnWarpsPerCta = 8;
constexpr int kLnMaxVecPerLane = 8;     // cols <= 8 * 32 * 8 = 2048

struct AddLnParams {
  const __nv_bfloat16* a;       // [rows, cols]
  const __nv_bfloat16* resid;   // [rows, cols] or null
  const __nv_bfloat16* scale;   // [cols]
  const __nv_bfloat16* shift;   // [cols]
  __nv_bfloat16* sum_out;       // [rows, cols] or null
  __nv_bfloat16* norm_out;      // [rows, cols]
  long long rows;
  int cols;
  float eps;
};

__device__ __forceinline__ void ln_unpack8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 ln_pack8(const float (&f)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}
__device__ __forceinline__ float ln_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int kVecPerLane>
__global__ void __launch_bounds__(kLnWarpsPerCta * 32) fa_add_layernorm_kernel(const AddLnParams p) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kLnWarpsPerCta + (threadIdx.x >> 5);
  if (row >= p.rows) return;                       // whole warps leave together
  const int nvec = p.cols >> 3;                    // 16-byte vectors per row
  const uint4* a = reinterpret_cast<const uint4*>(p.a + row * p.cols);
  const uint4* rs = p.resid ? reinterpret_cast<const uint4*>(p.resid + row * p.cols) : nullptr;

  // all loads of the row first (the sum may be written over a or resid, so a store between two
  // loads would pin their order and expose the memory latency once per step)
  uint4 a_raw[kVecPerLane], r_raw[kVecPerLane];
#pragma unroll
  for (int i = 0; i < kVecPerLane; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      a_raw[i] = __ldcs(a + v);      // streaming: each activation byte is read once
      if (rs) r_raw[i] = __ldcs(rs + v);
    }
  }
  float x[kVecPerLane][8];
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < kVecPerLane; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      ln_unpack8(a_raw[i], x[i]);
      if (rs) {
        float r8[8];
        ln_unpack8(r_raw[i], r8);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[i][e] += r8[e];
      }
      if (p.sum_out) {
        // the residual stream is kept in bf16: normalise exactly what the next block will read
        const uint4 packed = ln_pack8(x[i]);
        reinterpret_cast<uint4*>(p.sum_out + row * p.cols)[v] = packed;
        ln_unpack8(packed, x[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) total += x[i][e];
    }
  }
  const float mean = ln_warp_sum(total) / (float)p.cols;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < kVecPerLane; ++i) {
    if (lane + 32 * i < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float d = x[i][e] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
  const float rstd = rsqrtf(ln_warp_sum(sq) / (float)p.cols + p.eps);
  const uint4* sc = reinterpret_cast<const uint4*>(p.scale);
  const uint4* sh = reinterpret_cast<const uint4*>(p.shift);
  uint4* out = reinterpret_cast<uint4*>(p.norm_out + row * p.cols);
#pragma unroll
  for (int i = 0; i < kVecPerLane; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      float g[8], b[8], y[8];
      ln_unpack8(__ldg(sc + v), g);
      ln_unpack8(__ldg(sh + v), b);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = fmaf((x[i][e] - mean) * rstd, g[e], b[e]);
      out[v] = ln_pack8(y);
    }
  }
}

}  // namespace fa
