"""The element-wise work of a transformer block around the attention call, as single kernels.

`add_layernorm` is the reference's LayerNorm.forward (src/py/model_inference.py:102-107) fused
with the shortcut addition that precedes it (TransformerBlock.forward, :156 and :163); the
arithmetic is `fa_b200_add_layernorm` in libfa_b200.so (include/fa_b200.h).  CUDA bf16 only, no
fallback: the GPT-2 harness uses it on its bf16 inference path and keeps the torch ops elsewhere.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

__all__ = ["add_layernorm", "linear_small", "LINEAR_SMALL_MAX_ROWS"]

LINEAR_SMALL_MAX_ROWS = 8


def _dense2d(t: torch.Tensor, name: str, cols: int) -> torch.Tensor:
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16):
        raise RuntimeError(f"{name} must be a CUDA bfloat16 tensor")
    if t.shape[-1] != cols or not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous with {cols} columns")
    return t


def add_layernorm(a, resid, scale, shift, eps: float = 1e-5, return_sum: bool = True,
                  sum_out=None, norm_out=None):
    """`s = a + resid` (resid may be None), `y = LayerNorm(s) * scale + shift` over the last
    dimension, one pass.  Returns `(s, y)` when `return_sum` and a residual is given, else `y`.
    The normalised row is the bf16-rounded sum (what a later reader of `s` sees)."""
    cols = a.shape[-1]
    _dense2d(a, "a", cols)
    if resid is not None:
        _dense2d(resid, "resid", cols)
        if resid.shape != a.shape:
            raise RuntimeError("a and resid must have the same shape")
    for t, name in ((scale, "scale"), (shift, "shift")):
        _dense2d(t, name, cols)
        if t.numel() != cols:
            raise RuntimeError(f"{name} must have {cols} elements")
    keep = return_sum and resid is not None
    if keep and sum_out is None:
        sum_out = torch.empty_like(a)
    if norm_out is None:
        norm_out = torch.empty_like(a)
    p = _lib.FaAddLnParams()
    p.a, p.resid = a.data_ptr(), (resid.data_ptr() if resid is not None else None)
    p.scale, p.shift = scale.data_ptr(), shift.data_ptr()
    p.sum_out = sum_out.data_ptr() if keep else None
    p.norm_out = norm_out.data_ptr()
    p.rows, p.cols, p.eps = a.numel() // cols if cols else 0, cols, eps
    p.device = a.device.index
    p.stream = torch.cuda.current_stream(a.device).cuda_stream
    rc = _lib.load().fa_b200_add_layernorm(ctypes.byref(p))
    if rc != 0:
        raise RuntimeError(_lib.strerror(rc))
    return (sum_out, norm_out) if keep else norm_out


def linear_small(x, weight, bias=None, gelu: bool = False, out=None, resid=None, ln_scale=None,
                 ln_shift=None, eps: float = 1e-5, keep_sum: bool = False):
    """`act(x' @ weight.T + bias)` for at most 8 rows: `weight` [N, K] as nn.Linear stores it (rows
    may be strided), `x` [..., K] with at most 8 rows in total, tanh-GELU when `gelu`.  One pass
    over the weights (`fa_b200_linear_small`).

    Optional prologue inside the same kernel (K <= 2048): `x' = x + resid`, then
    `x' = LayerNorm(x') * ln_scale + ln_shift`; with `keep_sum` the sum `x + resid` is also
    returned (a new bf16 tensor: the next residual stream) and the result is `(sum, y)`."""
    K = x.shape[-1]
    _dense2d(x, "x", K)
    M = x.numel() // K
    if not (weight.is_cuda and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] == K
            and weight.stride(1) == 1):
        raise RuntimeError("weight must be a CUDA bfloat16 matrix [N, K] with dense rows")
    N = weight.shape[0]
    if bias is not None and not (bias.is_cuda and bias.dtype == torch.bfloat16 and bias.numel() == N
                                 and bias.is_contiguous()):
        raise RuntimeError("bias must be a contiguous CUDA bfloat16 vector of N elements")
    if resid is not None:
        _dense2d(resid, "resid", K)
        if resid.shape != x.shape:
            raise RuntimeError("x and resid must have the same shape")
    if (ln_scale is None) != (ln_shift is None):
        raise RuntimeError("ln_scale and ln_shift go together")
    for t, name in ((ln_scale, "ln_scale"), (ln_shift, "ln_shift")):
        if t is not None:
            _dense2d(t, name, K)
            if t.numel() != K:
                raise RuntimeError(f"{name} must have {K} elements")
    if out is None:
        out = torch.empty(*x.shape[:-1], N, dtype=torch.bfloat16, device=x.device)
    elif out.shape[-1] != N or out.numel() != M * N or not out.is_contiguous() or out.dtype != torch.bfloat16:
        raise RuntimeError("out must be a contiguous bfloat16 tensor [..., N]")
    total = torch.empty_like(x) if keep_sum else None
    p = _lib.FaLinearSmallParams()
    p.x, p.w, p.y = x.data_ptr(), weight.data_ptr(), out.data_ptr()
    p.bias = bias.data_ptr() if bias is not None else None
    p.M, p.N, p.K = M, N, K
    p.ldw = weight.stride(0) if N > 1 else K
    p.act = 1 if gelu else 0
    p.resid = resid.data_ptr() if resid is not None else None
    p.ln_scale = ln_scale.data_ptr() if ln_scale is not None else None
    p.ln_shift = ln_shift.data_ptr() if ln_shift is not None else None
    p.sum_out = total.data_ptr() if total is not None else None
    p.eps = eps
    p.device = x.device.index
    p.stream = torch.cuda.current_stream(x.device).cuda_stream
    rc = _lib.load().fa_b200_linear_small(ctypes.byref(p))
    if rc != 0:
        raise RuntimeError(_lib.strerror(rc))
    return (total, out) if keep_sum else out
