"""Builds tests/cpp/bin/test_amp_host from test_amp_host.cpp (host-only C++ over the C ABI),
linked against the in-tree libb200amp.so with an rpath relative to the binary."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
SRC = os.path.join(HERE, "test_amp_host.cpp")
BIN_DIR = os.path.join(HERE, "bin")
BIN = os.path.join(BIN_DIR, "test_amp_host")
LIB_DIR = os.path.join(REPO, "cuda_transformer_b200", "lib")


def build(force: bool = False) -> str:
    deps = [SRC, os.path.join(REPO, "include", "b200amp.h"), os.path.join(REPO, "include", "b200amp_host.hpp"),
            os.path.join(REPO, "include", "compat", "fast_shim.h")]
    if not force and os.path.exists(BIN) and all(os.path.getmtime(BIN) >= os.path.getmtime(d) for d in deps):
        return BIN
    os.makedirs(BIN_DIR, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O2", "-std=c++17", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(REPO, "include"), SRC, "-o", BIN,
           "-L", LIB_DIR, "-lb200amp", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../cuda_transformer_b200/lib"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("building test_amp_host failed:\n" + " ".join(cmd) + "\n" + proc.stderr)
    return BIN


if __name__ == "__main__":
    print(build(force=True))
