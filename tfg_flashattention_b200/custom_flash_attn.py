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
import os

import torch

from . import _lib

__all__ = ["forward", "forward_host", "decode", "last_status", "plan", "binding", "set_binding"]

# Two bindings of `forward` over the same C ABI:
#   "ext"     the compiled pybind11 / torch extension (csrc/torch_binding.cpp, built by
#             build.build_torch_binding()): the counterpart of the reference's torch_bind.cpp, a few
#             microseconds of host time per call, GIL released around the launch;
#   "ctypes"  pure Python over ctypes: needs no compiler beyond the one that built the library.
# The extension is used when it has been built (FA_B200_BINDING=ctypes in the environment, or
# set_binding("ctypes"), selects the other one).  Neither is a fallback for the kernel itself.
_ext = None
_binding = None


def _load_ext():
    global _ext
    if _ext is None:
        from . import _custom_flash_attn_ext as ext      # ImportError when it was never built
        if ext.abi_version != _lib.ABI_VERSION:
            raise ImportError("the torch binding was built from a different include/fa_b200.h; rebuild it "
                              "(python -m tfg_flashattention_b200.build --binding --force)")
        _lib.load()                                       # same checks on the library itself
        _ext = ext
    return _ext


def set_binding(name: str) -> str:
    """Select "ext", "ctypes" or "auto" (the extension when it is importable); returns the choice."""
    global _binding
    if name not in ("ext", "ctypes", "auto"):
        raise ValueError("binding must be 'ext', 'ctypes' or 'auto'")
    if name == "ctypes":
        _binding = "ctypes"
    else:
        try:
            _load_ext()
            _binding = "ext"
        except ImportError:
            if name == "ext":
                raise
            _binding = "ctypes"
    return _binding


def binding() -> str:
    """The binding `forward` goes through: "ext" or "ctypes"."""
    if _binding is None:
        set_binding(os.environ.get("FA_B200_BINDING", "auto"))
    return _binding


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


def _fwd_params(Q, K, V, O, lse, causal, softmax_scale):
    """struct fa_b200_params for one call on the current stream of Q's device."""
    B, H, N, d = Q.shape
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
    return p


def _check_qkv(Q, K, V):
    _check_input(Q, "Q")
    _check_input(K, "K_mat")
    _check_input(V, "V")
    if K.shape != Q.shape or V.shape != Q.shape:
        raise RuntimeError("Q, K_mat and V must have the same shape [B, H, N, d]")
    if K.device != Q.device or V.device != Q.device:
        raise RuntimeError("Q, K_mat and V must be on the same device")


def forward(Q, K, V, causal=True, return_lse=False, softmax_scale=None, out=None):
    """Attention forward on the current CUDA stream of Q's device.  See the module docstring."""
    if binding() == "ext":
        return _ext.forward(Q, K, V, causal, return_lse, softmax_scale, out)
    _check_qkv(Q, K, V)
    B, H, N, d = Q.shape
    if out is None:
        O = torch.empty_like(Q)      # same allocation rule as the reference (torch_bind.cpp:31)
    else:
        _check_input(out, "out")
        if out.shape != Q.shape or out.device != Q.device:
            raise RuntimeError("out must match Q in shape and device")
        O = out
    lse = torch.empty((B, H, N), dtype=torch.float32, device=Q.device) if return_lse else None
    p = _fwd_params(Q, K, V, O, lse, causal, softmax_scale)
    rc = _lib.load().fa_b200_fwd(ctypes.byref(p))
    if rc != 0:
        raise RuntimeError(f"custom_flash_attn.forward failed ({rc}): {_lib.strerror(rc)}")
    return (O, lse) if return_lse else O


def plan(Q, K, V, causal=True):
    """Which kernel schedule `forward` would use for these tensors, without launching anything:
    (name, grid) with name one of "cta_per_tile", "persistent_paired", "persistent_rotated",
    "persistent_full", "none" (fa_b200_fwd_plan in include/fa_b200.h)."""
    _check_qkv(Q, K, V)
    p = _fwd_params(Q, K, V, Q, None, causal, None)
    schedule, grid = ctypes.c_int32(-1), ctypes.c_int32(0)
    rc = _lib.load().fa_b200_fwd_plan(ctypes.byref(p), ctypes.byref(schedule), ctypes.byref(grid))
    if rc != 0:
        raise RuntimeError(f"custom_flash_attn.plan failed ({rc}): {_lib.strerror(rc)}")
    return _lib.SCHEDULES[schedule.value], grid.value


_decode_workspaces = {}


def decode(Q, K_cache, V_cache, kv_len, return_lse=False, softmax_scale=None, out=None,
           k_new=None, v_new=None):
    """Single-query attention against a K/V cache (one generation step; the reference has no
    counterpart -- its generate() recomputes the whole prefix, model_inference.py:199-228).

    Q [B, H, 64] (or [B, H, 1, 64]) bf16; K_cache, V_cache [B, H, >= kv_len, 64] bf16 (any row /
    head / batch strides that are multiples of 8 elements); attends rows 0 .. kv_len-1.  kv_len is
    an int, or a one-element int32 CUDA tensor that is read by the kernel when it runs.
    k_new, v_new [B, H, 64] (optional, both): the key / value of the token being generated; the
    kernel uses them as row kv_len-1 and writes them into that row of the caches (the cache
    append of the step without a separate copy kernel).
    Returns O shaped like Q (and LSE [B, H] fp32 when asked).  The split-KV workspace is a cached
    torch buffer per device; calls on one stream may share it, calls that overlap on different
    streams of one device must not (pass through separate processes or serialise them)."""
    squeeze = Q.dim() == 4
    q3 = Q[:, :, 0, :] if squeeze else Q
    for t, name in ((q3, "Q"), (K_cache, "K_cache"), (V_cache, "V_cache")):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if t.dtype != torch.bfloat16:
            raise RuntimeError("Unsupported tensor dtype. Use bfloat16.")
    if squeeze and Q.shape[2] != 1:
        raise RuntimeError("Q must hold one query row per head: [B, H, 64] or [B, H, 1, 64]")
    if q3.dim() != 3 or K_cache.dim() != 4 or V_cache.dim() != 4:
        raise RuntimeError("expected Q [B, H, d] and caches [B, H, N, d]")
    B, H, d = q3.shape
    if K_cache.shape[:2] != (B, H) or V_cache.shape != K_cache.shape or K_cache.shape[3] != d:
        raise RuntimeError("Q, K_cache and V_cache disagree on B, H or d")
    kv_len_dev = None
    if isinstance(kv_len, torch.Tensor):
        # the length lives on the device (an int32 scalar that the caller advances between steps):
        # the launch is sized for the whole cache and the kernel reads the length when it runs,
        # which is what lets one recorded CUDA-graph launch serve every step of a generation loop
        if not (kv_len.is_cuda and kv_len.dtype == torch.int32 and kv_len.numel() == 1):
            raise RuntimeError("a tensor kv_len must be one int32 on the GPU")
        kv_len_dev, kv_len = kv_len, K_cache.shape[2]
    kv_len = int(kv_len)
    if not 1 <= kv_len <= K_cache.shape[2]:
        raise RuntimeError("kv_len must be between 1 and the cache length")
    for t, name in ((q3, "Q"), (K_cache, "K_cache"), (V_cache, "V_cache")):
        if t.stride(-1) != 1:
            raise RuntimeError(f"{name}: the last dimension must be dense (stride 1)")
    if out is None:
        O = torch.empty((B, H, d), dtype=torch.bfloat16, device=Q.device)
    else:
        O = out[:, :, 0, :] if out.dim() == 4 else out
        if O.shape != (B, H, d) or O.dtype != torch.bfloat16 or O.device != Q.device or O.stride(-1) != 1:
            raise RuntimeError("out must match Q in shape, dtype and device")
    lse = torch.empty((B, H), dtype=torch.float32, device=Q.device) if return_lse else None

    lib = _lib.load()
    need = lib.fa_b200_decode_workspace_bytes(B, H, kv_len)
    if need < 0:
        raise RuntimeError(f"custom_flash_attn.decode failed ({need}): {_lib.strerror(int(need))}")
    ws = None
    if need > 0:
        ws = _decode_workspaces.get(Q.device)
        if ws is None or ws.numel() < need:
            ws = _decode_workspaces[Q.device] = torch.empty(max(need, 1 << 20), dtype=torch.uint8,
                                                            device=Q.device)

    def two(t):      # {batch, head} strides; size-1 dimensions get a canonical stride
        sb, sh = t.stride(0), t.stride(1)
        if H == 1:
            sh = 64
        if B == 1:
            sb = max(H * sh, 64)
        return (ctypes.c_int64 * 2)(sb, sh)

    def three(t):
        sb, sh, sn = t.stride(0), t.stride(1), t.stride(2)
        if t.shape[2] == 1:
            sn = 64
        if H == 1:
            sh = max(t.shape[2] * sn, 64)
        if B == 1:
            sb = max(H * sh, 64)
        return (ctypes.c_int64 * 3)(sb, sh, sn)

    p = _lib.FaDecodeParams()
    p.q, p.k_cache, p.v_cache, p.o = q3.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(), O.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.workspace = ws.data_ptr() if ws is not None else None
    p.workspace_bytes = ws.numel() if ws is not None else 0
    p.B, p.H, p.kv_len, p.d = B, H, kv_len, d
    if B * H > 0:
        p.q_strides, p.o_strides = two(q3), two(O)
        p.k_strides, p.v_strides = three(K_cache), three(V_cache)
    else:
        p.q_strides = p.o_strides = (ctypes.c_int64 * 2)(64, 64)
        p.k_strides = p.v_strides = (ctypes.c_int64 * 3)(64, 64, 64)
        for name in ("q", "k_cache", "v_cache", "o"):
            setattr(p, name, getattr(p, name) or 16)
    p.softmax_scale = 0.0 if softmax_scale is None else float(softmax_scale)
    p.device = Q.device.index if Q.device.index is not None else torch.cuda.current_device()
    p.stream = torch.cuda.current_stream(Q.device).cuda_stream
    p.kv_len_device = kv_len_dev.data_ptr() if kv_len_dev is not None else None
    if (k_new is None) != (v_new is None):
        raise RuntimeError("k_new and v_new go together")
    if k_new is not None:
        kn = k_new[:, :, 0, :] if k_new.dim() == 4 else k_new
        vn = v_new[:, :, 0, :] if v_new.dim() == 4 else v_new
        for t, name in ((kn, "k_new"), (vn, "v_new")):
            if not (t.is_cuda and t.dtype == torch.bfloat16 and t.shape == (B, H, d) and t.stride(-1) == 1):
                raise RuntimeError(f"{name} must be a CUDA bfloat16 tensor [B, H, 64] with a dense last dimension")
        if two(kn)[:] != two(vn)[:]:
            raise RuntimeError("k_new and v_new must have the same strides")
        p.k_new, p.v_new, p.new_strides = kn.data_ptr(), vn.data_ptr(), two(kn)
    rc = lib.fa_b200_decode(ctypes.byref(p))
    if rc != 0:
        raise RuntimeError(f"custom_flash_attn.decode failed ({rc}): {_lib.strerror(rc)}")
    result = out if out is not None else (O.unsqueeze(2) if squeeze else O)
    return (result, lse) if return_lse else result


class _HostPipeline:
    """Device-side chunk buffers and streams for forward_host, cached per (device, chunk shape)."""

    def __init__(self, device, shape):
        self.copy_in = torch.cuda.Stream(device)
        self.copy_out = torch.cuda.Stream(device)
        # two sets of chunk buffers: chunk i+1 is uploaded while chunk i is computed
        self.bufs = [tuple(torch.empty(shape, dtype=torch.bfloat16, device=device) for _ in range(4))
                     for _ in range(2)]


_host_pipelines = {}


def forward_host(Q, K, V, out=None, causal=True, softmax_scale=None, device=None, chunks=4):
    """Attention forward for HOST-resident tensors: q, k, v [B,H,N,d] bf16 in (ideally pinned) host
    memory, O returned in host memory (`out`, pinned, is reused when given).

    The batch is cut into `chunks` slices that flow through a three-stage pipeline -- upload of
    slice i+1, kernel on slice i, download of slice i-1 -- on separate CUDA streams, so the PCIe
    transfers in both directions overlap each other and the kernel instead of running back to
    back.  Returns after the last download has completed."""
    for t, name in ((Q, "Q"), (K, "K_mat"), (V, "V")):
        if t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 4:
            raise RuntimeError(f"{name} must be a host bfloat16 tensor of shape [B, H, N, d]")
    if K.shape != Q.shape or V.shape != Q.shape:
        raise RuntimeError("Q, K_mat and V must have the same shape [B, H, N, d]")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B = Q.shape[0]
    if out is None:
        out = torch.empty(Q.shape, dtype=torch.bfloat16).pin_memory()
    if B == 0 or Q.numel() == 0:
        return out
    chunks = max(1, min(int(chunks), B))
    bounds = [(B * i) // chunks for i in range(chunks + 1)]
    cmax = max(bounds[i + 1] - bounds[i] for i in range(chunks))
    key = (dev.index, cmax) + tuple(Q.shape[1:])
    pipe = _host_pipelines.get(key)
    if pipe is None:
        pipe = _host_pipelines[key] = _HostPipeline(dev, (cmax,) + tuple(Q.shape[1:]))
    compute = torch.cuda.current_stream(dev)
    pipe.copy_in.wait_stream(compute)
    pipe.copy_out.wait_stream(compute)
    computed = [None, None]      # event: kernel that used buffer set s has finished
    downloaded = [None, None]    # event: O of buffer set s has been copied out
    for i in range(chunks):
        lo, hi = bounds[i], bounds[i + 1]
        n = hi - lo
        s = i & 1
        dq, dk, dv, do = (b[:n] for b in pipe.bufs[s])
        with torch.cuda.stream(pipe.copy_in):
            if computed[s] is not None:
                pipe.copy_in.wait_event(computed[s])      # q, k, v of this set are no longer read
            dq.copy_(Q[lo:hi], non_blocking=True)
            dk.copy_(K[lo:hi], non_blocking=True)
            dv.copy_(V[lo:hi], non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(pipe.copy_in)
        compute.wait_event(uploaded)
        if downloaded[s] is not None:
            compute.wait_event(downloaded[s])              # O of this set has left the device
        forward(dq, dk, dv, causal=causal, softmax_scale=softmax_scale, out=do)
        computed[s] = torch.cuda.Event()
        computed[s].record(compute)
        with torch.cuda.stream(pipe.copy_out):
            pipe.copy_out.wait_event(computed[s])
            out[lo:hi].copy_(do, non_blocking=True)
            downloaded[s] = torch.cuda.Event()
            downloaded[s].record(pipe.copy_out)
    compute.wait_stream(pipe.copy_out)
    pipe.copy_out.synchronize()
    return out


def last_status(device=None) -> int:
    """Synchronise the current stream of `device` and return (and clear) the kernel's watchdog
    word: 0 when every kernel since the last call ran to completion."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    return _lib.load().fa_b200_last_status(idx, torch.cuda.current_stream(dev).cuda_stream)
