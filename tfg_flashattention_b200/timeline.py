"""Clock-stamp timeline of one CTA of the attention forward kernel.

    python -m tfg_flashattention_b200.timeline --build            # here: nvcc -DFA_TRACE, no GPU needed
    python -m tfg_flashattention_b200.timeline B,H,N,causal [cta]  # on a B200

The trace variant of the library (libfa_b200_trace.so, next to the product library) is the same
source compiled with -DFA_TRACE: lane 0 of softmax warps 0 and 3 and of the tcgen05 issuer warp of
one chosen CTA store clock64() at every hand-off of their first 64 K/V tiles.  This prints, per
tile, how long each phase of the softmax warp's serial chain took, and when the issuer acted
relative to it.  A measuring aid: the product library carries no trace code.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import sys

from . import build as _build

TRACE_LIB = os.path.join(_build.HERE, "libfa_b200_trace.so")


def build_trace_library() -> str:
    cmd = [_build._nvcc(), *_build.NVCC_FLAGS, "-DFA_TRACE", "-o", TRACE_LIB, *_build.SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building the trace library")
    return TRACE_LIB


SOFTMAX_PHASES = [  # (label, from event, to event)
    ("wait_S", 0, 1), ("ld_S", 1, 2), ("mask+max", 2, 3), ("wait_O", 3, 4), ("exp+stP", 4, 5),
    ("wait_st", 5, 6), ("arrive", 6, 8),
]
# "tail" = from the arrive to the next tile's start: the loop's way back and, on the first tile of
# an item, the epilogue owed to the previous item


def main(argv: list[str]) -> None:
    if "--build" in argv:
        print(build_trace_library())
        return
    import numpy as np
    import torch
    from . import _lib
    if not os.path.exists(TRACE_LIB):
        raise SystemExit("build the trace library first: python -m tfg_flashattention_b200.timeline --build")
    _lib.LIB_PATH = TRACE_LIB
    from . import custom_flash_attn as cfa
    cfa.set_binding("ctypes")      # the compiled binding is linked to the product library, not this one
    lib = _lib.load()
    B, H, N, causal = 8, 25, 4096, 0
    if argv:
        B, H, N, causal = (int(x) for x in argv[0].split(","))
    cta = int(argv[1]) if len(argv) > 1 else 100
    torch.manual_seed(0)
    q, k, v = (torch.randn(B, H, N, 64, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    for _ in range(3):
        cfa.forward(q, k, v, causal=bool(causal))
    torch.cuda.synchronize()
    lib.fa_b200_trace_select(ctypes.c_int(cta))
    cfa.forward(q, k, v, causal=bool(causal))
    n_slots = 4 * 64 * 16
    buf = (ctypes.c_ulonglong * n_slots)()
    rc = lib.fa_b200_trace_read(buf, n_slots)
    print(f"# B={B} H={H} N={N} causal={causal} cta={cta} rc={rc} status={cfa.last_status():#x}")
    t = np.array(buf[:], dtype=np.int64).reshape(4, 64, 16)
    for role, name in ((0, "softmax warp 0"), (1, "softmax warp 3")):
        print(f"## {name}: clocks per phase; ITEM marks the first tile of a work item")
        print("  g      " + " ".join(f"{lab:>9s}" for lab, _, _ in SOFTMAX_PHASES) + "      tail    period")
        rows = []
        for g in range(64):
            a = t[role, g]
            if a[0] == 0:
                break
            d = [int(a[e1] - a[e0]) if a[e0] and a[e1] else 0 for _, e0, e1 in SOFTMAX_PHASES]
            nxt = int(t[role, g + 1, 0]) if g + 1 < 64 else 0
            tail = nxt - int(a[8]) if nxt and a[8] else 0
            period = nxt - int(a[0]) if nxt else 0
            rows.append(d + [tail, period])
            print(f" {g:2d} {'ITEM' if a[9] else '    '} " + " ".join(f"{x:9d}" for x in d) + f" {tail:9d} {period:9d}")
        if len(rows) > 4:
            body = np.array(rows[2:-1])
            print("  median " + " ".join(f"{int(x):9d}" for x in np.median(body, axis=0)))
    print("## issuer (relative to softmax warp 0's tile start): K ready, S freed, S issued, V ready, P ready, PV issued")
    for g in range(64):
        a, s0 = t[2, g], t[0, g, 0]
        if a[0] == 0 or s0 == 0:
            break
        print(f" {g:2d} top {int(a[0]-s0):6d} | " + " ".join(f"{int(a[e]-s0) if a[e] else 0:7d}" for e in range(1, 7)))


if __name__ == "__main__":
    main(sys.argv[1:])
