"""Build libfa_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m tfg_flashattention_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is written next to this file so that it travels
with the source tree; nothing is installed into site-packages and nothing is JIT-cached elsewhere.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libfa_b200.so")
SOURCES = [os.path.join(CSRC, "fa_b200_api.cu")]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put it on PATH")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))] + [
        os.path.join(HERE, "..", "include", "fa_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps if os.path.isfile(d))


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB_PATH, *SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libfa_b200.so")
    return LIB_PATH


WAIT_TEST_LIB = os.path.join(HERE, "libfa_b200_waittest.so")


def build_wait_test_library(force: bool = False) -> str:
    """The library compiled with -DFA_WAIT_TEST, for tests/test_watchdog_gpu.py only: every bounded
    wait in the attention kernel gives up after 2 ms and the TMA producer leaves out one K tile, so
    a launch through it runs into the watchdog by construction, reports it and returns."""
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    if (not force and os.path.exists(WAIT_TEST_LIB)
            and all(os.path.getmtime(d) <= os.path.getmtime(WAIT_TEST_LIB) for d in deps)):
        return WAIT_TEST_LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-DFA_WAIT_TEST", "-o", WAIT_TEST_LIB, *SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building the wait-test library")
    return WAIT_TEST_LIB


EXT_NAME = "_custom_flash_attn_ext"
EXT_SOURCE = os.path.join(CSRC, "torch_binding.cpp")


def ext_path() -> str:
    import sysconfig
    return os.path.join(HERE, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build_torch_binding(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/torch_binding.cpp -- the pybind11 / torch-extension `forward`, the compiled
    counterpart of the reference's torch_bind.cpp -- into an extension module next to this file,
    linked against libfa_b200.so (found through $ORIGIN at run time).  Plain g++ with the include
    and library paths torch reports: in-tree like the library, no JIT cache elsewhere."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce
    out = ext_path()
    build_library()
    deps = [EXT_SOURCE, os.path.join(HERE, "..", "include", "fa_b200.h")]
    if not force and os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    # The system g++ first: the module must share libstdc++.so with torch (one C++ runtime in the
    # process; an exception thrown through a second, statically linked copy crashed in the
    # unwinder).  -lstdc++ and -shared-libgcc spell that out for compilers that default otherwise.
    cxx = shutil.which("g++") or os.environ.get("CXX") or "g++"
    cmd = [cxx, "-std=c++17", "-O2", "-shared", "-fPIC", "-fvisibility=hidden",
           f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{d}" for d in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    cmd += [EXT_SOURCE, "-o", out]
    cmd += [f"-L{d}" for d in ce.library_paths("cuda")] + [f"-L{HERE}"]
    cmd += ["-l:libfa_b200.so", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-lstdc++", "-shared-libgcc", "-Wl,-rpath,$ORIGIN"] + [f"-Wl,-rpath,{d}" for d in ce.library_paths("cuda")[:1]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("g++ failed building the torch binding")
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--wait-test" in sys.argv:
        print(build_wait_test_library(force="--force" in sys.argv))
    if "--binding" in sys.argv:
        print(build_torch_binding(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
