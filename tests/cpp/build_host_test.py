"""Builds the C++ test programs of the host layers (host-only C++ over the C ABI) into
tests/cpp/bin/, linked against the in-tree libb200amp.so with an rpath relative to the binary:
test_amp_host (one GPU: shim + AmpOptimizer), test_zero1_host (one process, R ranks, collectives fused into the
kernels), test_zero1_nccl_host (one process, R ranks on R GPUs, NCCL around the passes) and the
NVLink measurement program peer_bandwidth (two or more GPUs; plain CUDA, does not use the library; its output is
checked by tests/test_gpu_host_cpp.py)."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
BIN_DIR = os.path.join(HERE, "bin")
LIB_DIR = os.path.join(REPO, "cuda_transformer_b200", "lib")
INCLUDE = os.path.join(REPO, "include")
PROGRAMS = {     # name -> (source file, headers it depends on)
    "test_amp_host": ("test_amp_host.cpp", ["b200amp.h", "b200amp_host.hpp", os.path.join("compat", "fast_shim.h")]),
    "test_zero1_host": ("test_zero1_host.cpp", ["b200amp.h", "b200amp_host.hpp", "b200amp_zero1_host.hpp"]),
    "peer_bandwidth": ("peer_bandwidth.cu", []),
    "test_zero1_nccl_host": ("test_zero1_nccl_host.cpp", ["b200amp.h", "b200amp_host.hpp", "b200amp_zero1_host.hpp",
                                                          "b200amp_zero1_nccl_host.hpp"]),
}
NCCL_PROGRAMS = ("test_zero1_nccl_host",)


def nccl_paths():
    """(include dir, lib dir) of the NCCL that ships with the Python environment (nvidia-nccl wheel),
    or None. The programs that use NCCL are linked against that libnccl.so.2 by full path."""
    try:
        import nvidia.nccl as pkg
    except Exception:
        return None
    for root in list(getattr(pkg, "__path__", [])):
        inc, lib = os.path.join(root, "include"), os.path.join(root, "lib")
        if os.path.exists(os.path.join(inc, "nccl.h")) and os.path.exists(os.path.join(lib, "libnccl.so.2")):
            return inc, lib
    return None

BIN = os.path.join(BIN_DIR, "test_amp_host")


def build(force: bool = False, program: str = "test_amp_host") -> str:
    source, headers = PROGRAMS[program]
    src = os.path.join(HERE, source)
    exe = os.path.join(BIN_DIR, program)
    deps = [src] + [os.path.join(INCLUDE, h) for h in headers]
    if not force and os.path.exists(exe) and all(os.path.getmtime(exe) >= os.path.getmtime(d) for d in deps):
        return exe
    os.makedirs(BIN_DIR, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O2", "-std=c++17", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", INCLUDE, src, "-o", exe,
           "-L", LIB_DIR, "-lb200amp", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../cuda_transformer_b200/lib"]
    if program in NCCL_PROGRAMS:
        paths = nccl_paths()
        if paths is None:
            raise RuntimeError(f"{program} needs NCCL (nccl.h and libnccl.so.2 of the nvidia-nccl wheel): not found")
        # by name through the linker: with -x cu a bare path to the .so would be taken for a source file
        cmd += ["-I", paths[0], "-L", paths[1], "-l:libnccl.so.2", "-Xlinker", "-rpath", "-Xlinker", paths[1]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"building {program} failed:\n" + " ".join(cmd) + "\n" + proc.stderr)
    return exe


def build_all(force: bool = False) -> list:
    """Every program that can be built here (the NCCL one only where the nvidia-nccl wheel is installed)."""
    have_nccl = nccl_paths() is not None
    return [build(force, program) for program in PROGRAMS if have_nccl or program not in NCCL_PROGRAMS]


if __name__ == "__main__":
    print(build_all(force=True))
