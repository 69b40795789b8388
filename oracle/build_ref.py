"""Compile the reference project's own CUDA attention kernel into oracle/_ref/libref_v1.so.

    python oracle/build_ref.py [/path/to/reference]
    (default: $FA_REFERENCE_ROOT, else the folder `reference` next to this repository)

TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference's translation unit src/cpp/v1.cu (launcher,
:4-42) with its header src/cpp/headers/v1_implementation.hpp (kernel, :7-171) is compiled from
where it lies, unmodified and uncopied, with the reference's own flags (-O3 --use_fast_math,
src/py/setup.py:17-20) for sm_100a, next to oracle/ref_v1_shim.cu, which puts a C entry point
(`ref_v1_forward`) in front of the launcher template.  The reference's build system (setuptools
CUDAExtension, which also needs libtorch for the binding file) is not run.  Output goes to
oracle/_ref/ only; that folder is kept out of the history and travels to the GPU box as a built
file.  Where the reference sources are absent (the GPU box), this does nothing and whatever was
built before is used.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB_PATH = os.path.join(OUT_DIR, "libref_v1.so")
DEFAULT_REF_ROOT = os.environ.get("FA_REFERENCE_ROOT") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def build(ref_root: str | None = None, force: bool = False) -> str | None:
    """Returns the library path, or None when the reference sources are not available."""
    ref_root = ref_root or DEFAULT_REF_ROOT
    src = os.path.join(ref_root, "src", "cpp", "v1.cu")
    inc = os.path.join(ref_root, "src", "cpp", "headers")
    if not os.path.isfile(src):
        return LIB_PATH if os.path.exists(LIB_PATH) else None
    shim = os.path.join(HERE, "ref_v1_shim.cu")
    if (not force and os.path.exists(LIB_PATH)
            and os.path.getmtime(LIB_PATH) >= max(os.path.getmtime(shim), os.path.getmtime(src))):
        return LIB_PATH
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++17", "-O3", "--use_fast_math", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-I", inc, "-o", LIB_PATH, src, shim]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building the reference kernel")
    return LIB_PATH


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
