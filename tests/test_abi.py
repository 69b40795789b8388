"""The C-ABI library: it loads, exports every symbol include/fa_b200.h declares, and rejects bad
arguments before touching CUDA (so these run on a machine without a GPU)."""
import ctypes
import os
import re

import pytest

from tfg_flashattention_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported(fa_lib):
    declared = _declared_symbols()
    assert set(_lib.EXPORTS) <= set(declared)
    for name in declared:
        assert hasattr(fa_lib, name), f"{name} declared in include/fa_b200.h but not exported"


def test_abi_version(fa_lib):
    assert fa_lib.fa_b200_abi_version() == _lib.ABI_VERSION


def _good_params():
    p = _lib.FaParams()
    p.q, p.k, p.v, p.o = 0x1000, 0x2000, 0x3000, 0x4000
    p.lse = None
    p.B, p.H, p.N, p.d = 2, 3, 100, 64
    for name in ("q_strides", "k_strides", "v_strides", "o_strides"):
        setattr(p, name, (ctypes.c_int64 * 3)(3 * 100 * 64, 100 * 64, 64))
    p.softmax_scale = 0.0
    p.causal = 1
    p.device = 0
    p.stream = None
    return p


def test_validate_accepts_good_params(fa_lib):
    assert fa_lib.fa_b200_validate(ctypes.byref(_good_params())) == 0


@pytest.mark.parametrize("mutate,code", [
    (lambda p: setattr(p, "q", None), -1),
    (lambda p: setattr(p, "o", None), -1),
    (lambda p: setattr(p, "d", 128), -2),
    (lambda p: setattr(p, "d", 32), -2),
    (lambda p: setattr(p, "N", -1), -3),
    (lambda p: setattr(p, "B", -5), -3),
    (lambda p: setattr(p, "q_strides", (ctypes.c_int64 * 3)(100, 64, 60)), -4),
    (lambda p: setattr(p, "v_strides", (ctypes.c_int64 * 3)(0, 6400, 64)), -4),
    (lambda p: setattr(p, "o_strides", (ctypes.c_int64 * 3)(19200, 6400, -64)), -4),
    (lambda p: setattr(p, "k", 0x2004), -5),
    (lambda p: setattr(p, "lse", 0x5002), -5),
    (lambda p: setattr(p, "softmax_scale", float("nan")), -6),
    (lambda p: setattr(p, "softmax_scale", float("inf")), -6),
    (lambda p: setattr(p, "softmax_scale", -1.0), -6),
    (lambda p: setattr(p, "device", -1), -7),
])
def test_validate_rejects(fa_lib, mutate, code):
    p = _good_params()
    mutate(p)
    assert fa_lib.fa_b200_validate(ctypes.byref(p)) == code
    # fa_b200_fwd and fa_b200_fwd_plan apply the same checks first and make no CUDA call when they fail
    assert fa_lib.fa_b200_fwd(ctypes.byref(p)) == code
    schedule, grid = ctypes.c_int32(99), ctypes.c_int32(99)
    assert fa_lib.fa_b200_fwd_plan(ctypes.byref(p), ctypes.byref(schedule), ctypes.byref(grid)) == code
    assert (schedule.value, grid.value) == (99, 99)            # outputs untouched on error
    assert _lib.strerror(code).startswith("fa_b200")


def test_null_params_pointer(fa_lib):
    assert fa_lib.fa_b200_validate(None) == -1
    assert fa_lib.fa_b200_fwd(None) == -1
    assert fa_lib.fa_b200_fwd_plan(None, None, None) == -1


def test_plan_of_an_empty_problem_needs_no_device(fa_lib):
    p = _good_params()
    p.N = 0
    schedule, grid = ctypes.c_int32(99), ctypes.c_int32(99)
    assert fa_lib.fa_b200_fwd_plan(ctypes.byref(p), ctypes.byref(schedule), ctypes.byref(grid)) == 0
    assert (schedule.value, grid.value) == (-1, 0)             # FA_B200_SCHEDULE_NONE, nothing to launch


def test_strerror_covers_codes(fa_lib):
    assert _lib.strerror(0) == "ok"
    for code in range(-13, 0):
        assert "unknown" not in _lib.strerror(code)
    assert "watchdog" in _lib.strerror(0x10004)


def test_decode_workspace_query_and_validation(fa_lib):
    ws = fa_lib.fa_b200_decode_workspace_bytes
    assert ws(32, 25, 1024) == 0                       # 800 heads fill the GPU: keys are not split
    assert ws(1, 25, 1024) == 0                        # few heads, short cache: one wide CTA per head
    assert ws(1, 25, 8192) == 25 * 16 * 66 * 4         # long cache: 16 chunks of 512 rows per head
    assert ws(12, 25, 300) == 300 * 2 * 66 * 4         # 300 heads are too many for the wide form
    assert ws(1, 1, 100) == 0
    assert ws(1, 1, 64) == 0
    assert ws(0, 5, 10) == 0
    assert ws(1, 1, 0) == -3 and ws(-1, 1, 5) == -3
    p = _lib.FaDecodeParams()
    p.q, p.k_cache, p.v_cache, p.o = 0x1000, 0x2000, 0x3000, 0x4000
    p.B, p.H, p.kv_len, p.d = 1, 25, 8192, 64
    p.q_strides = p.o_strides = (ctypes.c_int64 * 2)(1600, 64)
    p.k_strides = p.v_strides = (ctypes.c_int64 * 3)(25 * 8192 * 64, 8192 * 64, 64)
    p.device = 0
    assert fa_lib.fa_b200_decode(ctypes.byref(p)) == -12     # needs a workspace, none given
    p.d = 128
    assert fa_lib.fa_b200_decode(ctypes.byref(p)) == -2
    p.d, p.kv_len = 64, 0
    assert fa_lib.fa_b200_decode(ctypes.byref(p)) == -3
    p.kv_len = 8192
    p.k_strides = (ctypes.c_int64 * 3)(25 * 8192 * 64, 8192 * 64, 60)
    assert fa_lib.fa_b200_decode(ctypes.byref(p)) == -4
    assert fa_lib.fa_b200_decode(None) == -1


def test_python_shim_rejects_cpu_and_dtype():
    import torch
    from tfg_flashattention_b200 import custom_flash_attn
    q = torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        custom_flash_attn.forward(q, q, q)


def test_add_layernorm_rejects_before_any_cuda_call(fa_lib):
    def params(**kw):
        p = _lib.FaAddLnParams()
        p.a, p.resid, p.scale, p.shift = 0x1000, 0x2000, 0x3000, 0x4000
        p.sum_out, p.norm_out = 0x5000, 0x6000
        p.rows, p.cols, p.eps, p.device, p.stream = 4, 768, 1e-5, 0, None
        for k, v in kw.items():
            setattr(p, k, v)
        return p
    call = lambda p: fa_lib.fa_b200_add_layernorm(ctypes.byref(p))
    assert fa_lib.fa_b200_add_layernorm(None) == -1
    assert call(params(a=None)) == -1
    assert call(params(norm_out=None)) == -1
    assert call(params(cols=0)) == -3
    assert call(params(cols=770)) == -3            # not a multiple of 8
    assert call(params(cols=2056)) == -3           # more than 2048 columns
    assert call(params(rows=-1)) == -3
    assert call(params(resid=0x2008)) == -5
    assert call(params(eps=-1.0)) == -6
    assert call(params(device=-2)) == -7
    assert call(params(rows=0)) == 0               # nothing to do, nothing launched


def test_linear_small_rejects_before_any_cuda_call(fa_lib):
    def params(**kw):
        p = _lib.FaLinearSmallParams()
        p.x, p.w, p.bias, p.y = 0x1000, 0x2000, 0x3000, 0x4000
        p.M, p.N, p.K, p.ldw, p.act, p.device, p.stream = 1, 4800, 1600, 1600, 0, 0, None
        for k, v in kw.items():
            setattr(p, k, v)
        return p
    call = lambda p: fa_lib.fa_b200_linear_small(ctypes.byref(p))
    assert fa_lib.fa_b200_linear_small(None) == -1
    assert call(params(w=None)) == -1
    assert call(params(M=0)) == -3 and call(params(M=9)) == -3
    assert call(params(K=1604)) == -3
    assert call(params(M=8, K=8200, ldw=8200)) == -3     # 8 rows x 8200 x 2 bytes > 128 KiB
    assert call(params(act=2)) == -3
    assert call(params(ldw=1592)) == -4
    assert call(params(x=0x1008)) == -5
    assert call(params(device=-1)) == -7
    assert call(params(N=0)) == 0
    # the fused add + LayerNorm prologue
    assert call(params(ln_scale=0x5000)) == -1                       # scale without shift
    assert call(params(K=4096, ldw=4096, ln_scale=0x5000, ln_shift=0x6000)) == -3
    assert call(params(resid=0x5008)) == -5
    assert call(params(resid=0x5000, sum_out=0x5000)) == -14         # sum over its own input
    assert call(params(resid=0x5000, sum_out=0x1000)) == -14
    assert call(params(ln_scale=0x5000, ln_shift=0x6000, eps=-1.0)) == -6
    assert b"overlap" in fa_lib.fa_b200_strerror(-14)
