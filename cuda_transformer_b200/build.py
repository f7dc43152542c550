"""Build recipe of the native library: nvcc, sm_100a only, in-tree output.

    python -m cuda_transformer_b200.build            # build if sources are newer than the .so
    python -m cuda_transformer_b200.build --force

The shared object lands in cuda_transformer_b200/lib/libb200amp.so. It is built
with the static CUDA runtime, so loading it needs nothing but the NVIDIA driver.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PKG_DIR)
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
INCLUDE_DIR = os.path.join(REPO_DIR, "include")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libb200amp.so")

SOURCES = ["api.cu", "scaler.cu", "adamw.cu", "pass2.cu", "zero1.cu"]
HEADERS = [os.path.join(CSRC_DIR, "internal.cuh"), os.path.join(CSRC_DIR, "adamw_math.cuh"),
           os.path.join(CSRC_DIR, "pass1_common.cuh"),
           os.path.join(INCLUDE_DIR, "b200amp.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-shared",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found (looked on PATH and in /usr/local/cuda/bin)")
    return nvcc


def stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC_DIR, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if needed and return its path."""
    if not force and not stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [find_nvcc()] + NVCC_FLAGS
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-I", INCLUDE_DIR, "-I", CSRC_DIR]
    cmd += [os.path.join(CSRC_DIR, s) for s in SOURCES]
    cmd += ["-o", LIB_PATH + ".tmp"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / spill / shared-memory figures")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))
    sys.exit(0)
