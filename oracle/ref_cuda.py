"""ctypes binding of oracle/_ref/libref_amp.so: the REFERENCE's own CUDA optimizer
kernels (cuda/kernels/scaler.cu, adamw_multi.cu) built for sm_100a by oracle/build_ref.py.

TEST INFRASTRUCTURE ONLY: the GPU-side oracle ("the reference's own AMP step") and the
kernel the library is timed against. available() is False where the object was not
built (no reference checkout at build time); callers skip, they never substitute.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libref_amp.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    lib = C.CDLL(LIB_PATH)
    P, LL, I, F = C.c_void_p, C.c_longlong, C.c_int, C.c_float
    protos = {
        "refamp_sizeof_state": (I, []),
        "refamp_initial_state": (None, [F, P]),
        "refamp_begin_step": (None, [P, P]),
        "refamp_unscale_and_norm": (None, [P, LL, P, P, P]),
        "refamp_finalize_step": (None, [P, P, P, P, I, P]),
        "refamp_adamw_multi": (None, [P, P, P, P, P, LL, P, I, P, F, F, F, P]),
        "refamp_lr_on_gpu": (C.c_double, [I, P]),
    }
    for name, (res, args) in protos.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    assert lib.refamp_sizeof_state() == 60
    _lib = lib
    return lib


def optimizer_step(lib, grads, n, state, partial, sched_ptr, history, history_len, params, params_x, m, v, tensors,
                   ntensors, beta1, beta2, eps, stream):
    """The reference's sequence (cuda/gpt_fast.cu:438-450) on raw device pointers."""
    lib.refamp_unscale_and_norm(grads, n, state, partial, stream)
    lib.refamp_finalize_step(state, partial, sched_ptr, history, history_len, stream)
    lib.refamp_adamw_multi(params, params_x, grads, m, v, n, tensors, ntensors, state, beta1, beta2, eps, stream)
