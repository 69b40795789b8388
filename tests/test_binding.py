"""The compiled binding of `forward` (csrc/torch_binding.cpp), without a GPU: it imports, carries
the header version of the library next to it, and polices its arguments the way the reference's
binding does (src/cpp/torch_bind.cpp:13-19, 33-42: CUDA tensor, bfloat16; RuntimeError)."""
import pytest
import torch


def test_extension_imports_and_matches_the_library(fa_lib, torch_binding):
    if torch_binding is None:
        pytest.skip("the torch extension binding could not be built here")
    from tfg_flashattention_b200 import _lib, custom_flash_attn
    assert torch_binding.abi_version == _lib.ABI_VERSION == fa_lib.fa_b200_abi_version()
    assert custom_flash_attn.set_binding("auto") == "ext"
    assert custom_flash_attn.set_binding("ctypes") == "ctypes"
    assert custom_flash_attn.set_binding("auto") == "ext"


@pytest.mark.parametrize("which", ["ext", "ctypes"])
def test_argument_errors_are_runtime_errors(which, fa_lib, torch_binding):
    if which == "ext" and torch_binding is None:
        pytest.skip("the torch extension binding could not be built here")
    from tfg_flashattention_b200 import custom_flash_attn as cfa
    cfa.set_binding(which)
    try:
        t = torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16)
        with pytest.raises(RuntimeError, match="must be a CUDA tensor"):    # CHECK_CUDA, torch_bind.cpp:13
            cfa.forward(t, t, t)
    finally:
        cfa.set_binding("auto")
