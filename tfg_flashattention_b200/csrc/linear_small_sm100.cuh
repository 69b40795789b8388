// y = act(x W^T + bias) for a handful of rows of x -- the Linear layers of a generation step.
//
//   x [M, K] bf16 (M <= 8 tokens),  W [N, K] bf16 row-major as torch.nn.Linear stores it,
//   bias [N] bf16 or none,  y [M, N] bf16,  fp32 accumulation,  act: none or tanh-GELU.
//
// In the reference these are the nn.Linear calls of MultiHeadAttention (W_query / W_key / W_value,
// out_proj: src/py/model_inference.py:50-53, 93), FeedForward (:121-125, with the GELU of
// :109-117 between them) and the output head (:190), evaluated for one new token per sequence.
// With M this small the work is reading W once: N * K * 2 bytes, an HBM-bound matrix-vector
// product that a tiled GEMM kernel serves badly (cuBLAS: ~30 % of the copy bandwidth at M = 1).
//
// One warp per output column n: the 32 lanes stride over the K dimension in 16-byte vectors
// (8 bf16), four vectors in flight per lane, multiply with the matching slice of every x row
// (staged once per CTA in shared memory) and reduce with shuffles.  The grid is a few CTAs per
// SM; each warp takes several columns in turn.
//
// Optional prologue, fused into the staging of x: the shortcut addition and the LayerNorm that
// precede the layer in a transformer block (x <- x + resid, the sum kept as the new residual
// stream, x <- LayerNorm(x) * scale + shift; model_inference.py:102-107, 156, 163).  Every CTA
// recomputes the statistics of the few rows (K <= 2048: one 16-byte vector per thread and row),
// which removes a separate one-warp kernel from the dependency chain of a generation step.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "add_layernorm_sm100.cuh"   // ln_unpack8 / ln_pack8 / ln_warp_sum

namespace fa {

constexpr int kLinWarps = 8;            // output columns per CTA
constexpr int kLinMaxRows = 8;          // rows of x
constexpr int kLinUnrollShort = 4;      // 16-byte weight loads in flight per lane: short rows ...
constexpr int kLinUnrollLong = 8;       // ... and rows of K > 2048 or very many columns (measured)

struct LinearSmallParams {
  const __nv_bfloat16* x;      // [M, K]
  const __nv_bfloat16* w;      // [N, K], row stride ldw
  const __nv_bfloat16* bias;   // [N] or null
  __nv_bfloat16* y;            // [M, N]
  int M, N, K;
  long long ldw;
  int act;                     // 0 none, 1 tanh-GELU
  // optional prologue on x (K <= 2048): x <- x + resid; sum_out <- bf16(x); x <- LayerNorm(x)
  const __nv_bfloat16* resid;      // [M, K] or null
  const __nv_bfloat16* ln_scale;   // [K] or null: no LayerNorm
  const __nv_bfloat16* ln_shift;   // [K]
  __nv_bfloat16* sum_out;          // [M, K] or null; written by CTA 0 only; must not alias x / resid
  float eps;
};

__device__ __forceinline__ float gelu_tanh(float v) {
  // 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3)))   (model_inference.py:113-116)
  const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
  return 0.5f * v * (1.0f + tanhf(u));
}

template <int kRows, int kLinUnroll>
__global__ void __launch_bounds__(kLinWarps * 32) fa_linear_small_kernel(const LinearSmallParams p) {
  extern __shared__ uint4 lin_smem[];              // x: kRows rows of K/8 16-byte vectors
  const int nvec = p.K >> 3;
  if (p.resid == nullptr && p.ln_scale == nullptr) {
    for (int i = threadIdx.x; i < kRows * nvec; i += kLinWarps * 32) {
      const int m = i / nvec, v = i - m * nvec;
      lin_smem[i] = m < p.M ? reinterpret_cast<const uint4*>(p.x + (long long)m * p.K)[v]
                            : make_uint4(0u, 0u, 0u, 0u);
    }
  } else {
    // thread t owns vector t of every row (nvec <= 256, checked by the host)
    __shared__ float red[2][kRows][kLinWarps];
    const int v = threadIdx.x;
    const bool live = v < nvec;
    float xs[kRows][8];
    float part[kRows];
#pragma unroll
    for (int m = 0; m < kRows; ++m) {
      part[m] = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) xs[m][e] = 0.f;
      if (live && m < p.M) {
        ln_unpack8(reinterpret_cast<const uint4*>(p.x + (long long)m * p.K)[v], xs[m]);
        if (p.resid) {
          float r8[8];
          ln_unpack8(reinterpret_cast<const uint4*>(p.resid + (long long)m * p.K)[v], r8);
#pragma unroll
          for (int e = 0; e < 8; ++e) xs[m][e] += r8[e];
        }
        if (p.sum_out) {   // the kept sum is bf16: normalise exactly what its later readers see
          const uint4 packed = ln_pack8(xs[m]);
          if (blockIdx.x == 0) reinterpret_cast<uint4*>(p.sum_out + (long long)m * p.K)[v] = packed;
          ln_unpack8(packed, xs[m]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) part[m] += xs[m][e];
      }
    }
    if (p.ln_scale) {
      const int wid = threadIdx.x >> 5, ln_lane = threadIdx.x & 31;
      float mean[kRows], rstd[kRows];
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {       // pass 0: mean; pass 1: variance about it
#pragma unroll
        for (int m = 0; m < kRows; ++m) {
          const float w = ln_warp_sum(part[m]);
          if (ln_lane == 0) red[pass][m][wid] = w;
        }
        __syncthreads();
#pragma unroll
        for (int m = 0; m < kRows; ++m) {
          float tot = 0.f;
#pragma unroll
          for (int i = 0; i < kLinWarps; ++i) tot += red[pass][m][i];
          if (pass == 0) {
            mean[m] = tot / (float)p.K;
            part[m] = 0.f;
            if (live && m < p.M) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float d = xs[m][e] - mean[m];
                part[m] = fmaf(d, d, part[m]);
              }
            }
          } else {
            rstd[m] = rsqrtf(tot / (float)p.K + p.eps);
          }
        }
      }
      if (live) {
        float g[8], b[8];
        ln_unpack8(__ldg(reinterpret_cast<const uint4*>(p.ln_scale) + v), g);
        ln_unpack8(__ldg(reinterpret_cast<const uint4*>(p.ln_shift) + v), b);
#pragma unroll
        for (int m = 0; m < kRows; ++m) {
#pragma unroll
          for (int e = 0; e < 8; ++e) xs[m][e] = fmaf((xs[m][e] - mean[m]) * rstd[m], g[e], b[e]);
        }
      }
    }
    if (live) {
#pragma unroll
      for (int m = 0; m < kRows; ++m) lin_smem[m * nvec + v] = ln_pack8(xs[m]);   // rows >= M are zero
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  // a warp walks over output columns n, n + 8 * gridDim.x, ...: the grid is capped at a few CTAs
  // per SM so that staging x (above) stays small next to reading W
  for (int n = blockIdx.x * kLinWarps + (threadIdx.x >> 5); n < p.N; n += gridDim.x * kLinWarps) {
    const uint4* wrow = reinterpret_cast<const uint4*>(p.w + (long long)n * p.ldw);

    float acc[kRows];
#pragma unroll
    for (int m = 0; m < kRows; ++m) acc[m] = 0.f;
    for (int v0 = lane; v0 < nvec; v0 += 32 * kLinUnroll) {
      uint4 wv[kLinUnroll];
#pragma unroll
      for (int u = 0; u < kLinUnroll; ++u) {         // all loads first
        const int v = v0 + 32 * u;
        wv[u] = v < nvec ? __ldcs(wrow + v) : make_uint4(0u, 0u, 0u, 0u);   // streaming: read once
      }
#pragma unroll
      for (int u = 0; u < kLinUnroll; ++u) {
        const int v = v0 + 32 * u;
        if (v < nvec) {
          const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv[u]);
          float wf[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 t = __bfloat1622float2(w2[i]);
            wf[2 * i] = t.x;
            wf[2 * i + 1] = t.y;
          }
#pragma unroll
          for (int m = 0; m < kRows; ++m) {
            const uint4 xv = lin_smem[m * nvec + v];
            const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 t = __bfloat1622float2(x2[i]);
              acc[m] = fmaf(wf[2 * i], t.x, acc[m]);
              acc[m] = fmaf(wf[2 * i + 1], t.y, acc[m]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < kRows; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    }
    const float b = p.bias ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
    for (int m = 0; m < kRows; ++m) {
      if (lane == m && m < p.M) {
        float v = acc[m] + b;
        if (p.act == 1) v = gelu_tanh(v);
        p.y[(long long)m * p.N + n] = __float2bfloat16_rn(v);
      }
    }
  }
}

}  // namespace fa
