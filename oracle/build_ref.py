"""Compiles the REFERENCE's optimizer kernels for sm_100a into oracle/_ref/libref_amp.so.

    python oracle/build_ref.py [/path/to/cuda-transformer]

The checkout is the argument, else $B200AMP_REFERENCE_DIR, else a directory named
`reference` beside this repository.

Sources are compiled where they lie in the reference checkout (cuda/kernels/scaler.cu,
cuda/kernels/adamw_multi.cu, with -DFP16 as the reference's fp16 build, Makefile:44-48,
only the arch flag changed from sm_75 to sm_100a); oracle/ref_wrap.cu adds extern "C"
doors. Nothing of the reference is copied into this repository: the output directory is
git-ignored and travels to a GPU box only as a built object. Without the checkout this
is a no-op that reports the library as unavailable.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB_PATH = os.path.join(OUT_DIR, "libref_amp.so")


def default_ref() -> str:
    """Where the reference checkout is looked for when no path is given."""
    return os.environ.get("B200AMP_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root: str = None, force: bool = False):
    """Path of the built library, or None if the reference checkout is absent."""
    ref_root = ref_root or default_ref()
    srcs = [os.path.join(ref_root, "cuda", "kernels", f) for f in ("scaler.cu", "adamw_multi.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return LIB_PATH if os.path.exists(LIB_PATH) else None
    wrap = os.path.join(HERE, "ref_wrap.cu")
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= os.path.getmtime(wrap):
        return LIB_PATH
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-DFP16",
           "-Xcompiler", "-fPIC", "-shared",
           "-I", os.path.join(ref_root, "cuda"), "-I", os.path.join(ref_root, "cuda", "kernels"),
           wrap] + srcs + ["-o", LIB_PATH + ".tmp"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("building the reference kernels failed:\n" + " ".join(cmd) + "\n" + proc.stderr)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
