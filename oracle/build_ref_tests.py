"""Builds the REFERENCE's own test programs for sm_100a, twice: as they are ("stock"), and with
the reference's optimizer objects replaced by the link shim over libb200amp.so ("b200amp").

    python oracle/build_ref_tests.py [/path/to/cuda-transformer]

Everything is compiled from the reference checkout where it lies (its Makefile's FAST_SRC list,
-DFP16, -arch changed from sm_75 to sm_100a; Makefile:44-48,93-117); objects and binaries go to
oracle/_ref/ (git-ignored). Nothing of the reference is copied into this repository. Also writes
the answer-key dump the programs read (oracle/_ref/data/debug.bin) by running the reference's
own reference/dump.py on the random-token fallback its tests use. Without the checkout this is a
no-op.

    stock:    common dump gpt weights data kernels/*.cu gpt_fast graph checkpoint  + test_X.cu
    b200amp:  the same minus kernels/scaler.cu, kernels/adamw_multi.cu, graph.cu
              plus oracle/link_shim.cu and -lb200amp

The reference's trainer, cuda/train_fast.cu (+ tokenizer/bpe.cpp, Makefile:147-148), is built the
same two ways, and two token files of seeded random ids in its BPE1 format (cuda/data.cu:30-69) are
written next to the dump, so that a test can run the whole training program on the library.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")
OBJ = os.path.join(OUT, "obj")
BIN = os.path.join(OUT, "bin")
DUMP = os.path.join(OUT, "data", "debug.bin")
ROUNDTRIP = os.path.join(BIN, "ckpt_roundtrip")
WEIGHTS_ROUNDTRIP = os.path.join(BIN, "weights_roundtrip")
REPLACED = ("kernels/scaler.cu", "kernels/adamw_multi.cu", "graph.cu")
PROGRAMS = ("test_fast", "test_checkpoint")
TRAINER = "train_fast"
TOKENS = os.path.join(OUT, "data", "synth")         # synth_train.bin, synth_val.bin


def _nvcc() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _compile(src: str, obj: str, includes, defines=()) -> None:
    if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
        return
    os.makedirs(os.path.dirname(obj), exist_ok=True)
    cmd = [_nvcc(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-DFP16"]
    cmd += [f"-D{d}" for d in defines]
    for inc in includes:
        cmd += ["-I", inc]
    cmd += ["-c", src, "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("compile failed: " + " ".join(cmd) + "\n" + proc.stderr[-4000:])


def binaries() -> dict:
    return {f"{prog}_{kind}": os.path.join(BIN, f"{prog}_{kind}") for prog in PROGRAMS for kind in ("stock", "b200amp")}


def trainer_binaries() -> dict:
    """stock; b200amp = the compat link shim (the reference's results bit for bit); b200amp_native = the
    link shim built with -DB200AMP_SHIM_NATIVE (bridge + fp16-arena step under the same three calls)."""
    return {kind: os.path.join(BIN, f"{TRAINER}_{kind}") for kind in ("stock", "b200amp", "b200amp_native")}


def trainer_available() -> bool:
    return (all(os.path.exists(p) for p in trainer_binaries().values()) and os.path.exists(DUMP)
            and all(os.path.exists(f"{TOKENS}_{part}.bin") for part in ("train", "val")))


def write_tokens() -> str:
    """BPE1 files (u32 magic 0x31455042, u32 version 1, u32 count, u16 ids; cuda/data.cu:30-69) of
    seeded random ids below the tiny model's vocabulary: nothing to learn, but every code path of
    the trainer runs."""
    import struct

    import numpy as np
    os.makedirs(os.path.dirname(TOKENS), exist_ok=True)
    for part, count, seed in (("train", 200_000, 11), ("val", 20_000, 12)):
        path = f"{TOKENS}_{part}.bin"
        if os.path.exists(path):
            continue
        ids = np.random.default_rng(seed).integers(0, 4098, size=count).astype("<u2")
        with open(path, "wb") as f:
            f.write(struct.pack("<III", 0x31455042, 1, count))
            f.write(ids.tobytes())
    return TOKENS


def available() -> bool:
    return all(os.path.exists(p) for p in binaries().values()) and os.path.exists(DUMP)


def write_dump(ref_root: str) -> str:
    """The tiny answer key (L2 H4 C64, B4 T64, perturbed 1-D parameters) through the reference's
    own dump module, on 100,000 seeded random token ids (reference/test_reference.py:40-45)."""
    if os.path.exists(DUMP):
        return DUMP
    os.makedirs(os.path.dirname(DUMP), exist_ok=True)
    code = (
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {ref_root!r})\n"
        "from reference import dump\n"
        "from reference.config import DUMP_BATCH, TrainConfig, tiny_model_config\n"
        "rng = np.random.default_rng(0)\n"
        "tokens = rng.integers(0, 4098, size=100_000).astype(np.uint16)\n"
        "header, records = dump.build_records(tiny_model_config(4098), TrainConfig(), tokens, DUMP_BATCH, 'cpu', "
        "perturb=True)\n"
        f"dump.write_dump({DUMP!r}, header, records)\n")
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env)
    if proc.returncode != 0:
        raise RuntimeError("writing the reference dump failed:\n" + proc.stderr[-4000:])
    return DUMP


def build(ref_root: str = None, jobs: int = 8):
    """Dict name -> path of the four binaries, or None without the reference checkout."""
    if ref_root is None:
        from oracle.build_ref import default_ref
        ref_root = default_ref()
    cuda = os.path.join(ref_root, "cuda")
    if not os.path.exists(os.path.join(cuda, "gpt_fast.cu")):
        return binaries() if available() else None
    from cuda_transformer_b200 import build as lib_build
    lib_build.build()
    rel = ["common.cu", "dump.cu", "gpt.cu", "weights.cu", "data.cu", "gpt_fast.cu", "graph.cu", "checkpoint.cu"]
    rel += sorted("kernels/" + os.path.basename(p) for p in glob.glob(os.path.join(cuda, "kernels", "*.cu")))
    rel += [f"tests/{prog}.cu" for prog in PROGRAMS]
    includes = [cuda, os.path.join(ref_root, "tokenizer")]
    jobs_list = [(os.path.join(cuda, r), os.path.join(OBJ, r[:-3] + ".o"), includes) for r in rel]
    shim_obj = os.path.join(OBJ, "link_shim.o")
    jobs_list.append((os.path.join(HERE, "link_shim.cu"), shim_obj, includes + [os.path.join(REPO, "include")]))
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        for f in [pool.submit(_compile, *job) for job in jobs_list]:
            f.result()
    os.makedirs(BIN, exist_ok=True)
    common = [r for r in rel if not r.startswith("tests/")]
    lib_dir = os.path.join(REPO, "cuda_transformer_b200", "lib")
    out = binaries()
    for prog in PROGRAMS:
        test_obj = os.path.join(OBJ, f"tests/{prog}.o")
        stock = [os.path.join(OBJ, r[:-3] + ".o") for r in common]
        ours = [os.path.join(OBJ, r[:-3] + ".o") for r in common if r not in REPLACED] + [shim_obj]
        for kind, objs, extra in (("stock", stock, []),
                                  ("b200amp", ours, ["-L", lib_dir, "-lb200amp", "-Xlinker", "-rpath", "-Xlinker",
                                                     "$ORIGIN/../../../cuda_transformer_b200/lib"])):
            cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-o", out[f"{prog}_{kind}"], test_obj] + \
                objs + extra
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError("link failed: " + " ".join(cmd) + "\n" + proc.stderr[-4000:])
    # the trainer: cuda/train_fast.cu + tokenizer/bpe.cpp, stock and on the library
    trainer_obj = os.path.join(OBJ, "train_fast.o")
    bpe_obj = os.path.join(OBJ, "tokenizer_bpe.o")
    _compile(os.path.join(cuda, "train_fast.cu"), trainer_obj, includes)
    _compile(os.path.join(ref_root, "tokenizer", "bpe.cpp"), bpe_obj, includes)
    stock = [os.path.join(OBJ, r[:-3] + ".o") for r in common]
    ours = [os.path.join(OBJ, r[:-3] + ".o") for r in common if r not in REPLACED] + [shim_obj]
    native_shim_obj = os.path.join(OBJ, "link_shim_native.o")
    _compile(os.path.join(HERE, "link_shim.cu"), native_shim_obj, includes + [os.path.join(REPO, "include")],
             defines=("B200AMP_SHIM_NATIVE",))
    native = [o for o in ours if o != shim_obj] + [native_shim_obj]
    with_lib = ["-L", lib_dir, "-lb200amp", "-Xlinker", "-rpath", "-Xlinker",
                "$ORIGIN/../../../cuda_transformer_b200/lib"]
    for kind, objs, extra in (("stock", stock, []), ("b200amp", ours, with_lib), ("b200amp_native", native, with_lib)):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-o", trainer_binaries()[kind], trainer_obj,
               bpe_obj] + objs + extra
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("link failed: " + " ".join(cmd) + "\n" + proc.stderr[-4000:])
    write_tokens()
    # ckpt_roundtrip: the reference's checkpoint reader + writer behind a two-argument command line
    rt_obj = os.path.join(OBJ, "ckpt_roundtrip.o")
    _compile(os.path.join(HERE, "ckpt_roundtrip.cu"), rt_obj, includes)
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-o", ROUNDTRIP, rt_obj] + \
        [os.path.join(OBJ, r[:-3] + ".o") for r in common]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed: " + " ".join(cmd) + "\n" + proc.stderr[-4000:])
    # weights_roundtrip: the same for weights.bin
    wr_obj = os.path.join(OBJ, "weights_roundtrip.o")
    _compile(os.path.join(HERE, "weights_roundtrip.cu"), wr_obj, includes)
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-o", WEIGHTS_ROUNDTRIP, wr_obj] + \
        [os.path.join(OBJ, r[:-3] + ".o") for r in common]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed: " + " ".join(cmd) + "\n" + proc.stderr[-4000:])
    write_dump(ref_root)
    return out


if __name__ == "__main__":
    sys.path.insert(0, REPO)
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
