"""A bounded wait that runs out: the kernel reports it and returns, and the context stays usable.

Every mbarrier wait in the attention kernel has a time limit; when one runs out the kernel writes
a code to a status word, every role drains and leaves through the normal exit, and
fa_b200_last_status hands the code to the host (the reference has nothing of the kind: its
cudaGetLastError result is dropped, src/cpp/torch_bind.cpp:34-39).  To see that path run, a second
build of the library (-DFA_WAIT_TEST) shortens the limit to 2 ms and has the TMA producer leave out
the second K tile, whose barrier is then armed by nobody -- a flag that nothing sets.  No trap, no
bad address, no endless loop: the launch ends by itself within a few tens of milliseconds.
"""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

WATCHDOG_BASE = 0x10000
# The missing K tile stalls three waits at once: the issuer's for that tile (2), and behind it the
# producer's for the Q slot (9) and the softmax warps' for the next S (4).  They started within a
# microsecond or two of each other, so which one runs out first -- and gets to write the word -- is
# a matter of that microsecond; any of the three is the right report.
EXPECTED_WAITS = {2: b"K/V tile load", 9: b"Q slot", 4: b"S = QK^T"}


def test_wait_runs_out_is_reported_and_the_next_launch_is_correct(fa_lib):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from tfg_flashattention_b200 import _lib, build
    from tfg_flashattention_b200 import custom_flash_attn as cfa
    wt = ctypes.CDLL(build.build_wait_test_library())
    wt.fa_b200_fwd.argtypes = [ctypes.POINTER(_lib.FaParams)]
    wt.fa_b200_fwd.restype = ctypes.c_int
    wt.fa_b200_last_status.argtypes = [ctypes.c_int, ctypes.c_void_p]
    wt.fa_b200_last_status.restype = ctypes.c_int
    wt.fa_b200_strerror.argtypes = [ctypes.c_int]
    wt.fa_b200_strerror.restype = ctypes.c_char_p

    torch.manual_seed(3)
    # one CTA: B = H = 1, N = 256 is a single pair of causal tiles; its first item needs two K tiles
    q, k, v = (torch.randn(1, 1, 256, 64, device="cuda").bfloat16() for _ in range(3))
    assert cfa.plan(q, k, v) == ("persistent_paired", 1)
    good = cfa.forward(q, k, v)
    assert cfa.last_status() == 0

    o = torch.empty_like(q)
    p = cfa._fwd_params(q, k, v, o, None, True, None)
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    assert wt.fa_b200_fwd(ctypes.byref(p)) == 0          # the launch itself succeeds
    code = wt.fa_b200_last_status(0, stream)             # synchronises: the kernel has returned
    elapsed = time.perf_counter() - t0
    assert code & ~0xff == WATCHDOG_BASE and (code & 0xff) in EXPECTED_WAITS, hex(code)
    message = wt.fa_b200_strerror(code)
    assert b"watchdog" in message and EXPECTED_WAITS[code & 0xff] in message
    assert elapsed < 2.0, f"the kernel took {elapsed:.2f} s to give up"
    assert wt.fa_b200_last_status(0, stream) == 0        # reading the word cleared it

    # the context is intact: the product library computes the same bits as before
    again = cfa.forward(q, k, v)
    assert cfa.last_status() == 0
    assert torch.equal(again, good)
