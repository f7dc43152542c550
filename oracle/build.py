"""Build recipe of the CPU oracle (test infrastructure, never linked into the library).

    python oracle/build.py          # oracle/lib/libref_step.so from oracle/ref_step.c

-ffp-contract=off: every fused multiply-add in ref_step.c is an explicit fmaf(), the
compiler must not add its own. OpenMP is used when the compiler has it (the loops it
covers are elementwise or reduce over fixed chunks, so results do not depend on it).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "ref_step.c")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libref_step.so")

BASE = ["-O2", "-ffp-contract=off", "-fPIC", "-Wall", "-Wextra", "-std=c11", "-shared"]


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= os.path.getmtime(SRC):
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    errors = []
    for cc in ("/usr/bin/gcc", "gcc", "cc"):
        for extra in (["-fopenmp"], []):
            cmd = [cc] + BASE + extra + ["-o", LIB_PATH + ".tmp", SRC, "-lm"]
            try:
                proc = subprocess.run(cmd, capture_output=True, text=True)
            except FileNotFoundError as e:
                errors.append(str(e))
                continue
            if proc.returncode == 0:
                os.replace(LIB_PATH + ".tmp", LIB_PATH)
                return LIB_PATH
            errors.append(" ".join(cmd) + "\n" + proc.stderr)
    raise RuntimeError("could not build the oracle:\n" + "\n".join(errors))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
