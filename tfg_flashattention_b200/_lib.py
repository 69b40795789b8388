"""ctypes binding of libfa_b200.so -- the declarations in include/fa_b200.h, one to one.

There is no fallback: if the library is missing, or the device is not a B200, calls raise.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfa_b200.so")

ABI_VERSION = 4


class FaParams(ctypes.Structure):
    """struct fa_b200_params (include/fa_b200.h)."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("N", ctypes.c_int32), ("d", ctypes.c_int32),
        ("q_strides", ctypes.c_int64 * 3), ("k_strides", ctypes.c_int64 * 3),
        ("v_strides", ctypes.c_int64 * 3), ("o_strides", ctypes.c_int64 * 3),
        ("softmax_scale", ctypes.c_float), ("causal", ctypes.c_int32),
        ("device", ctypes.c_int32), ("stream", ctypes.c_void_p),
    ]


class FaDecodeParams(ctypes.Structure):
    """struct fa_b200_decode_params (include/fa_b200.h)."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64),
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("kv_len", ctypes.c_int32), ("d", ctypes.c_int32),
        ("q_strides", ctypes.c_int64 * 2), ("o_strides", ctypes.c_int64 * 2),
        ("k_strides", ctypes.c_int64 * 3), ("v_strides", ctypes.c_int64 * 3),
        ("softmax_scale", ctypes.c_float), ("device", ctypes.c_int32), ("stream", ctypes.c_void_p),
        ("kv_len_device", ctypes.c_void_p),
        ("k_new", ctypes.c_void_p), ("v_new", ctypes.c_void_p), ("new_strides", ctypes.c_int64 * 2),
    ]


class FaAddLnParams(ctypes.Structure):
    """struct fa_b200_add_layernorm_params (include/fa_b200.h)."""
    _fields_ = [
        ("a", ctypes.c_void_p), ("resid", ctypes.c_void_p), ("scale", ctypes.c_void_p),
        ("shift", ctypes.c_void_p), ("sum_out", ctypes.c_void_p), ("norm_out", ctypes.c_void_p),
        ("rows", ctypes.c_int64), ("cols", ctypes.c_int32), ("eps", ctypes.c_float),
        ("device", ctypes.c_int32), ("stream", ctypes.c_void_p),
    ]


class FaLinearSmallParams(ctypes.Structure):
    """struct fa_b200_linear_small_params (include/fa_b200.h)."""
    _fields_ = [
        ("x", ctypes.c_void_p), ("w", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("y", ctypes.c_void_p),
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32), ("ldw", ctypes.c_int64),
        ("act", ctypes.c_int32), ("device", ctypes.c_int32), ("stream", ctypes.c_void_p),
        ("resid", ctypes.c_void_p), ("ln_scale", ctypes.c_void_p), ("ln_shift", ctypes.c_void_p),
        ("sum_out", ctypes.c_void_p), ("eps", ctypes.c_float),
    ]


EXPORTS = ("fa_b200_fwd", "fa_b200_fwd_plan", "fa_b200_validate", "fa_b200_strerror", "fa_b200_device_ok",
           "fa_b200_last_status", "fa_b200_abi_version", "fa_b200_decode", "fa_b200_decode_workspace_bytes", "fa_b200_decode_static",
           "fa_b200_add_layernorm", "fa_b200_linear_small")

SCHEDULES = {-1: "none", 0: "cta_per_tile", 1: "persistent_paired", 2: "persistent_rotated",
             3: "persistent_full"}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once and declare every exported symbol's signature."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m tfg_flashattention_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for this kernel)")
    lib = ctypes.CDLL(LIB_PATH)
    missing = [name for name in EXPORTS if not hasattr(lib, name)]
    if missing:
        raise RuntimeError(f"{LIB_PATH} lacks {', '.join(missing)}: it was built from older sources; "
                           "rebuild it with `python -m tfg_flashattention_b200.build --force`")
    P = ctypes.POINTER(FaParams)
    lib.fa_b200_fwd.argtypes = [P]
    lib.fa_b200_fwd.restype = ctypes.c_int
    lib.fa_b200_fwd_plan.argtypes = [P, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
    lib.fa_b200_fwd_plan.restype = ctypes.c_int
    lib.fa_b200_validate.argtypes = [P]
    lib.fa_b200_validate.restype = ctypes.c_int
    lib.fa_b200_strerror.argtypes = [ctypes.c_int]
    lib.fa_b200_strerror.restype = ctypes.c_char_p
    lib.fa_b200_device_ok.argtypes = [ctypes.c_int]
    lib.fa_b200_device_ok.restype = ctypes.c_int
    lib.fa_b200_last_status.argtypes = [ctypes.c_int, ctypes.c_void_p]
    lib.fa_b200_last_status.restype = ctypes.c_int
    lib.fa_b200_decode.argtypes = [ctypes.POINTER(FaDecodeParams)]
    lib.fa_b200_decode.restype = ctypes.c_int
    lib.fa_b200_decode_static.argtypes = [ctypes.POINTER(FaDecodeParams)]
    lib.fa_b200_decode_static.restype = ctypes.c_int
    lib.fa_b200_decode_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.fa_b200_decode_workspace_bytes.restype = ctypes.c_int64
    lib.fa_b200_add_layernorm.argtypes = [ctypes.POINTER(FaAddLnParams)]
    lib.fa_b200_add_layernorm.restype = ctypes.c_int
    lib.fa_b200_linear_small.argtypes = [ctypes.POINTER(FaLinearSmallParams)]
    lib.fa_b200_linear_small.restype = ctypes.c_int
    lib.fa_b200_abi_version.argtypes = []
    lib.fa_b200_abi_version.restype = ctypes.c_int
    if lib.fa_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libfa_b200.so was built from a different include/fa_b200.h; rebuild it")
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().fa_b200_strerror(code).decode()
