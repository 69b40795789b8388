"""The reference project's own CUDA kernel, as built by oracle/build_ref.py.
TEST / BENCHMARK INFRASTRUCTURE ONLY (a second checker next to the CPU oracle, and the timed
comparator of bench.py); nothing in the product imports this.

`forward(q, k, v)` does what the reference binding does around its launcher
(src/cpp/torch_bind.cpp:21-45): contiguous bf16 CUDA tensors [B, H, N, 64], O = empty_like(Q),
`flashattention_forward<__nv_bfloat16>(O, Q, K, V, N, B, H)` (src/cpp/v1.cu:4-38).  The launcher
reads device 0's properties and launches on the legacy default stream, so tensors must live on
cuda:0; the caller's current stream is synchronised with the default stream around the call.
"""
from __future__ import annotations

import ctypes
import os

import torch

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libref_v1.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def _load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(LIB_PATH)
        lib.ref_v1_forward.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 3
        lib.ref_v1_forward.restype = ctypes.c_int
        _lib = lib
    return _lib


def forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    for t in (q, k, v):
        if not (t.is_cuda and t.is_contiguous() and t.dtype == torch.bfloat16 and t.dim() == 4):
            raise RuntimeError("reference kernel: contiguous bf16 CUDA tensors [B, H, N, 64] only")
    if q.shape[3] != 64 or k.shape != q.shape or v.shape != q.shape:
        raise RuntimeError("reference kernel: head dimension is fixed at 64; q, k, v same shape")
    # the kernel's per-head offset is computed in 32-bit int (v1_implementation.hpp:26)
    if q.numel() >= 2 ** 31:
        raise RuntimeError("reference kernel: tensor too large for its 32-bit offsets")
    dev = q.device.index if q.device.index is not None else torch.cuda.current_device()
    if dev != torch.cuda.current_device():
        raise RuntimeError("reference kernel: tensors must be on the current device")
    B, H, N, _ = q.shape
    o = torch.empty_like(q) if out is None else out
    if q.numel() == 0:
        return o
    cur = torch.cuda.current_stream()
    legacy = torch.cuda.default_stream()       # stream 0: where the reference launches
    if cur != legacy:
        legacy.wait_stream(cur)
    with torch.cuda.stream(legacy):
        rc = _load().ref_v1_forward(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), N, B, H)
    if cur != legacy:
        cur.wait_stream(legacy)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: cudaError {rc}")
    return o
