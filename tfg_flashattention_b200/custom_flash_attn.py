"""Drop-in for the reference project's torch extension module `custom_flash_attn`.

The reference builds a pybind11 extension of that name exporting one function,
`forward(Q, K, V) -> O` (src/cpp/torch_bind.cpp:21-49), imported by its GPT-2 attention module
(src/py/model_inference.py:13, 85-90) and by its tests (test/py/test_cuda_implementation.py:4).
This module keeps the name, the function and the positional call: `forward(q, k, v)` is causal,
uses scale 1/sqrt(d) and returns a new bf16 tensor shaped like q.  Added keyword arguments:

    causal=True         False gives full (unmasked) attention
    return_lse=False    True returns (O, LSE) with LSE = logsumexp_j(scale * q_i.k_j), fp32 [B,H,N]
    softmax_scale=None  overrides 1/sqrt(d)
    out=None            write O into this tensor instead of allocating one

Checks follow the reference binding (CUDA tensor, bfloat16; errors are RuntimeError as TORCH_CHECK
raises), with two differences: the head dimension is checked (the reference assumes 64 without
looking, torch_bind.cpp:27-29), and tensors need not be contiguous -- any layout whose last
dimension is dense and whose other strides are multiples of 8 elements is read in place, which
covers the `[B,N,H,d] -> transpose(1,2)` views the attention module produces
(model_inference.py:64-66), so the three `.contiguous()` copies at the call site are unnecessary.

PyTorch is used here for what it owns -- tensors, the current device and stream; the arithmetic
is in libfa_b200.so (C ABI: include/fa_b200.h).  There is no fallback path.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

__all__ = ["forward", "last_status"]


def _check_input(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if t.dtype != torch.bfloat16:
        raise RuntimeError("Unsupported tensor dtype. Use bfloat16.")
    if t.dim() != 4:
        raise RuntimeError(f"{name} must have shape [B, H, N, d]")


def _strides3(t: torch.Tensor, name: str):
    """Element strides {batch, head, row}; strides of size-1 dimensions are never dereferenced, so
    they are replaced by a canonical value that always passes the library's checks."""
    B, H, N, d = t.shape
    if d > 1 and t.stride(3) != 1:
        raise RuntimeError(f"{name}: the last dimension must be dense (stride 1)")
    sb, sh, sn = t.stride(0), t.stride(1), t.stride(2)
    if N == 1:
        sn = d
    if H == 1:
        sh = max(N * sn, 8)
    if B == 1:
        sb = max(H * sh, N * sn, 8)
    return (ctypes.c_int64 * 3)(sb, sh, sn)


def forward(Q, K, V, causal=True, return_lse=False, softmax_scale=None, out=None):
    """Attention forward on the current CUDA stream of Q's device.  See the module docstring."""
    _check_input(Q, "Q")
    _check_input(K, "K_mat")
    _check_input(V, "V")
    if K.shape != Q.shape or V.shape != Q.shape:
        raise RuntimeError("Q, K_mat and V must have the same shape [B, H, N, d]")
    if K.device != Q.device or V.device != Q.device:
        raise RuntimeError("Q, K_mat and V must be on the same device")
    B, H, N, d = Q.shape
    if out is None:
        O = torch.empty_like(Q)      # same allocation rule as the reference (torch_bind.cpp:31)
    else:
        _check_input(out, "out")
        if out.shape != Q.shape or out.device != Q.device:
            raise RuntimeError("out must match Q in shape and device")
        O = out
    lse = torch.empty((B, H, N), dtype=torch.float32, device=Q.device) if return_lse else None

    lib = _lib.load()
    p = _lib.FaParams()
    p.q, p.k, p.v, p.o = Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.B, p.H, p.N, p.d = B, H, N, d
    if Q.numel() > 0:
        p.q_strides = _strides3(Q, "Q")
        p.k_strides = _strides3(K, "K_mat")
        p.v_strides = _strides3(V, "V")
        p.o_strides = _strides3(O, "out")
    else:                            # empty problem: nothing is read, any valid strides do
        for name in ("q_strides", "k_strides", "v_strides", "o_strides"):
            setattr(p, name, (ctypes.c_int64 * 3)(8, 8, 8))
        for name in ("q", "k", "v", "o"):
            setattr(p, name, getattr(p, name) or 16)
    p.softmax_scale = 0.0 if softmax_scale is None else float(softmax_scale)
    p.causal = 1 if causal else 0
    p.device = Q.device.index if Q.device.index is not None else torch.cuda.current_device()
    p.stream = torch.cuda.current_stream(Q.device).cuda_stream
    rc = lib.fa_b200_fwd(ctypes.byref(p))
    if rc != 0:
        raise RuntimeError(f"custom_flash_attn.forward failed ({rc}): {_lib.strerror(rc)}")
    return (O, lse) if return_lse else O


def last_status(device=None) -> int:
    """Synchronise the current stream of `device` and return (and clear) the kernel's watchdog
    word: 0 when every kernel since the last call ran to completion."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    return _lib.load().fa_b200_last_status(idx, torch.cuda.current_stream(dev).cuda_stream)
