"""The allocation-free decode entry point, fa_b200_decode_static, against fa_b200_decode.

For hosts that cannot give the kernel a workspace: a serving process whose framework owns every
byte of device memory, a request path where cudaMalloc / cudaFree are banned because they can stall
the device, a bare C host without an allocator.  The split-KV partials then live in a buffer
compiled into the library.  Called through the C ABI directly (ctypes), twice in a row with
different problems -- the buffer is shared and keeps the previous call's contents -- and compared
with the workspace-taking entry point.  Collected last (file name), and independent of the tests
before it: passes alone in a fresh process and after the rest of the suite.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(lib_mod, q, k, v, o, kv_len, workspace=None):
    B, H, _ = q.shape
    p = lib_mod.FaDecodeParams()
    p.q, p.k_cache, p.v_cache, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    p.lse = None
    p.workspace = workspace.data_ptr() if workspace is not None else None
    p.workspace_bytes = workspace.numel() if workspace is not None else 0
    p.B, p.H, p.kv_len, p.d = B, H, kv_len, 64
    p.q_strides = (ctypes.c_int64 * 2)(q.stride(0), q.stride(1))
    p.o_strides = (ctypes.c_int64 * 2)(o.stride(0), o.stride(1))
    p.k_strides = (ctypes.c_int64 * 3)(k.stride(0), k.stride(1), k.stride(2))
    p.v_strides = (ctypes.c_int64 * 3)(v.stride(0), v.stride(1), v.stride(2))
    p.softmax_scale = 0.0
    p.device = q.device.index
    p.stream = torch.cuda.current_stream(q.device).cuda_stream
    return p


def test_decode_static_matches_decode_on_two_calls_in_a_row(fa_lib):
    from tfg_flashattention_b200 import _lib
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(2024)
    # first a problem that uses many chunks per head, then a smaller one with fewer: stale partials
    # of the first call sit in the shared buffer while the second runs
    for (B, H, kv_len) in ((1, 25, 6000), (12, 25, 300)):
        need = fa_lib.fa_b200_decode_workspace_bytes(B, H, kv_len)
        assert need > 0                          # fa_b200_decode splits this problem over chunks
        q = torch.randn(B, H, 64, device=dev, generator=g).bfloat16()
        k = torch.randn(B, H, kv_len + 5, 64, device=dev, generator=g).bfloat16()
        v = torch.randn(B, H, kv_len + 5, 64, device=dev, generator=g).bfloat16()
        o_ref = torch.empty_like(q)
        o_new = torch.full_like(q, float("nan"))
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        assert fa_lib.fa_b200_decode(ctypes.byref(_params(_lib, q, k, v, o_ref, kv_len, ws))) == 0
        rc = fa_lib.fa_b200_decode_static(ctypes.byref(_params(_lib, q, k, v, o_new, kv_len)))
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize(dev)
        assert torch.isfinite(o_new.float()).all()
        # same kernels; the suite's tolerance is the stated bound.  Caches under 2048 rows are cut
        # into the same chunks by both entry points: equal to the bit there
        assert (o_new.float() - o_ref.float()).abs().max().item() <= 2e-2
        if kv_len < 2048:
            assert torch.equal(o_new, o_ref)
        # the point of the entry point: a call allocates no device memory.  The first call on the
        # device has done its one-time set-up; repeat it and compare the driver's count of free
        # memory before and after (cudaMemGetInfo, not torch's caching allocator).
        torch.cuda.synchronize(dev)
        free_before, _ = torch.cuda.mem_get_info(dev)
        rc = fa_lib.fa_b200_decode_static(ctypes.byref(_params(_lib, q, k, v, o_new, kv_len)))
        torch.cuda.synchronize(dev)
        free_after, _ = torch.cuda.mem_get_info(dev)
        assert rc == 0 and free_after == free_before
        assert (o_new.float() - o_ref.float()).abs().max().item() <= 2e-2
        # and against plain torch on the first kv_len rows
        s = torch.einsum("bhd,bhnd->bhn", q.float(), k[:, :, :kv_len].float()) / 8.0
        want = torch.einsum("bhn,bhnd->bhd", torch.softmax(s, -1), v[:, :, :kv_len].float())
        assert (o_new.float() - want).abs().max().item() <= 2e-2


def test_decode_static_needs_no_scratch_for_large_batches_and_refuses_oversize(fa_lib):
    from tfg_flashattention_b200 import _lib
    dev = torch.device("cuda", 0)
    # 800 (batch, head) pairs: keys are not split, the buffer is not used at all
    q = torch.randn(32, 25, 64, device=dev).bfloat16()
    k = torch.randn(32, 25, 128, 64, device=dev).bfloat16()
    v = torch.randn(32, 25, 128, 64, device=dev).bfloat16()
    o_ref, o_new = torch.empty_like(q), torch.empty_like(q)
    assert fa_lib.fa_b200_decode_workspace_bytes(32, 25, 128) == 0
    assert fa_lib.fa_b200_decode(ctypes.byref(_params(_lib, q, k, v, o_ref, 128))) == 0
    assert fa_lib.fa_b200_decode_static(ctypes.byref(_params(_lib, q, k, v, o_new, 128))) == 0
    torch.cuda.synchronize(dev)
    assert torch.equal(o_new, o_ref)
    # 500 pairs with two chunks each need 264,000 bytes: more than the 262,144 built in
    q = torch.randn(20, 25, 64, device=dev).bfloat16()
    k = torch.randn(20, 25, 256, 64, device=dev).bfloat16()
    o = torch.zeros_like(q)
    assert fa_lib.fa_b200_decode_workspace_bytes(20, 25, 256) > 256 * 1024
    rc = fa_lib.fa_b200_decode_static(ctypes.byref(_params(_lib, q, k, k, o, 256)))
    assert rc == -13 and "built-in buffer" in _lib.strerror(rc)
    torch.cuda.synchronize(dev)
    assert (o == 0).all()                          # nothing was launched
