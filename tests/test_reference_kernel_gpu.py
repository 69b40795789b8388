"""The reference project's own CUDA kernel as a second checker.

oracle/build_ref.py compiles the reference's src/cpp/v1.cu (+ headers/v1_implementation.hpp)
unmodified into oracle/_ref/libref_v1.so where the reference sources are available; the built file
travels with the tree.  These tests (i) validate the CPU oracle against what the reference's kernel
actually computes, at the lengths and the tolerance of the reference's own tests
(test/py/test_cuda_implementation.py:72-117: rtol = atol = 1e-2), and (ii) compare this library's
kernel with the reference's on identical bf16 inputs.  Skipped where the library was never built.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_kernel():
    from oracle import ref_kernel as rk
    if not rk.available():
        pytest.skip("oracle/_ref/libref_v1.so was not built (needs the reference sources: python oracle/build_ref.py)")
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return rk


@pytest.mark.parametrize("T", [10, 11, 15, 33, 63, 65, 128, 300])
def test_oracle_matches_the_reference_kernel(ref_kernel, T):
    from oracle.attention_oracle import manual_attention
    torch.manual_seed(500 + T)
    q, k, v = (torch.randn(2, 4, T, 64).bfloat16() for _ in range(3))
    o = ref_kernel.forward(q.cuda(), k.cuda(), v.cuda())
    torch.cuda.synchronize()
    assert torch.isfinite(o).all()
    want = manual_attention(q.float(), k.float(), v.float(), causal=True)
    assert torch.allclose(want, o.float().cpu(), rtol=1e-2, atol=1e-2), \
        f"max diff {(want - o.float().cpu()).abs().max().item():.3e}"


@pytest.mark.parametrize("B,H,N", [(2, 4, 128), (1, 3, 333), (2, 2, 1024)])
def test_this_library_matches_the_reference_kernel(ref_kernel, fa_lib, B, H, N):
    from tfg_flashattention_b200 import custom_flash_attn as cfa
    torch.manual_seed(600 + N)
    q, k, v = (torch.randn(B, H, N, 64, device="cuda").bfloat16() for _ in range(3))
    ours = cfa.forward(q, k, v)                      # the reference binding's call: causal, scale 1/8
    theirs = ref_kernel.forward(q, k, v)
    assert cfa.last_status() == 0
    assert torch.allclose(theirs.float(), ours.float(), rtol=1e-2, atol=1e-2), \
        f"max diff {(theirs.float() - ours.float()).abs().max().item():.3e}"
