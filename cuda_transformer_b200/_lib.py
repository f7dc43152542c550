"""ctypes binding of libb200amp.so, the C ABI declared in include/b200amp.h.

The library is the only implementation of the step: there is no Python or CPU
fallback. If the shared object is missing, load() raises with the command that builds
it; it never substitutes another code path.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

OK, ERR_ARG, ERR_CUDA, ERR_DEVICE, ERR_LIMIT = 0, 1, 2, 3, 4
NORM_BLOCKS = 512
MAX_TENSORS = 1024


class StepState(C.Structure):
    """b200amp_step_state: bit-compatible with the reference's StepState (cuda/kernels/fast.h:104-121)."""
    _fields_ = [
        ("loss_scale", C.c_float), ("inv_scale", C.c_float),
        ("good_steps", C.c_int), ("found_inf", C.c_int), ("skipped", C.c_int),
        ("step", C.c_int), ("adam_t", C.c_int),
        ("lr", C.c_float), ("grad_norm", C.c_float), ("clip_coef", C.c_float),
        ("step_size", C.c_float), ("bc2_sqrt", C.c_float), ("decay", C.c_float),
        ("loss", C.c_float), ("n_valid", C.c_int),
    ]

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_}


class ScheduleConfig(C.Structure):
    """b200amp_schedule: the reference's ScheduleConfig (cuda/kernels/fast.h:123-133)."""
    _fields_ = [
        ("lr", C.c_float), ("min_lr", C.c_float),
        ("warmup_steps", C.c_int), ("max_steps", C.c_int),
        ("beta1", C.c_float), ("beta2", C.c_float),
        ("weight_decay", C.c_float), ("grad_clip", C.c_float),
        ("growth_interval", C.c_int), ("dynamic_scale", C.c_int), ("decay_steps", C.c_int),
    ]


class TensorInfo(C.Structure):
    """b200amp_tensor_info: the reference's TensorInfo (cuda/kernels/fast.h:153-158)."""
    _fields_ = [("offset", C.c_longlong), ("count", C.c_longlong), ("decay", C.c_int)]


class Zero1Sync(C.Structure):
    """b200amp_zero1_sync: every rank's block of flag words as mapped in this process, and the
    number of polls after which a wait on another rank gives up (0 = the library's default)."""
    _fields_ = [("block_by_rank", C.c_void_p * 8), ("wait_limit", C.c_uint)]


class DecayRuns(C.Structure):
    """b200amp_decay_runs: the tensor table merged into runs of equal decay flag."""
    _fields_ = [("first4", C.c_uint * 256), ("nruns", C.c_int), ("flag0", C.c_int)]


ZERO1_SYNC_BYTES = 1024
SYNC_SIGNAL, SYNC_WAIT, SYNC_ADVANCE, SYNC_STAMP = 1, 2, 4, 8
PHASE_GRADS, PHASE_PAIRS, PHASE_WEIGHTS = 0, 1, 2

assert C.sizeof(StepState) == 60 and C.sizeof(ScheduleConfig) == 44 and C.sizeof(TensorInfo) == 24
assert C.sizeof(Zero1Sync) == 72

_P = C.c_void_p
_LL = C.c_longlong
_I = C.c_int
_F = C.c_float

# name -> (restype, argtypes); every symbol include/b200amp.h declares
PROTOTYPES = {
    "b200amp_last_error": (C.c_char_p, []),
    "b200amp_version": (C.c_char_p, []),
    "b200amp_device_check": (_I, []),
    "b200amp_check_tensor_table": (_I, [_P, _I, _LL]),
    "b200amp_initial_state": (_I, [_F, C.POINTER(StepState)]),
    "b200amp_begin_step": (_I, [_P, _P]),
    "b200amp_unscale_and_norm_f32": (_I, [_P, _LL, _P, _P, _P]),
    "b200amp_finalize_step": (_I, [_P, _P, C.POINTER(ScheduleConfig), _P, _I, _P]),
    "b200amp_adamw_multi_f32": (_I, [_P, _P, _P, _P, _P, _LL, _P, _I, _P, _F, _F, _F, _P]),
    "b200amp_lr_on_gpu": (_I, [_I, C.POINTER(ScheduleConfig), C.POINTER(C.c_double)]),
    "b200amp_cast_to_x": (_I, [_P, _P, _LL, _P]),
    "b200amp_workspace_bytes": (C.c_size_t, []),
    "b200amp_workspace_init": (_I, [_P, _P]),
    "b200amp_pass1_f16": (_I, [_P, _LL, _P, _P, _P]),
    "b200amp_pass1_f16_static": (_I, [_P, _LL, _P, _P, _P]),
    "b200amp_cast_pass1_f32": (_I, [_P, _P, _LL, _I, _P, _P, C.POINTER(ScheduleConfig), _P, _I, _P]),
    "b200amp_finalize_sums": (_I, [_P, _P, _I, C.POINTER(ScheduleConfig), _P, _I, _P]),
    "b200amp_pass1_finalize_f16": (_I, [_P, _LL, _P, _P, C.POINTER(ScheduleConfig), _P, _I, _P]),
    "b200amp_pass2_f16": (_I, [_P, _P, _P, _P, _P, _LL, _LL, _P, _I, _P, _F, _F, _F, _P]),
    "b200amp_decay_runs_build": (_I, [_P, _I, C.POINTER(DecayRuns)]),
    "b200amp_pass2_f16_runs": (_I, [_P, _P, _P, _P, _P, _LL, _LL, C.POINTER(DecayRuns), _P, _F, _F, _F, _P]),
    "b200amp_rs_pass1_f16": (_I, [_P, _I, _I, _P, _LL, _P, _P, _P, _P]),
    "b200amp_pass2_ag_f16": (_I, [_P, _P, _P, _P, _P, _I, _LL, _LL, _P, _I, _P, _F, _F, _F, _P]),
    "b200amp_rs_pass1_f16_part": (_I, [_P, _I, _I, _P, _LL, _I, _I, _I, _P, _P, _P, _P]),
    "b200amp_pass1_partition": (_I, [_LL, C.POINTER(_I), C.POINTER(_LL)]),
    "b200amp_copy_async": (_I, [_P, _P, _LL, _P]),
    "b200amp_zero1_sync_init": (_I, [_P, _P]),
    "b200amp_zero1_sync_read": (_I, [_P, C.POINTER(C.c_uint), C.POINTER(C.c_uint)]),
    "b200amp_zero1_barrier": (_I, [C.POINTER(Zero1Sync), _I, _I, _I, _I, _P]),
    "b200amp_rs_pass1_f16_sync": (_I, [_P, _I, _I, _P, _LL, _P, _P, _P, C.POINTER(Zero1Sync), _P]),
    "b200amp_finalize_sums_sync": (_I, [_P, _P, _I, _I, C.POINTER(ScheduleConfig), _P, _I, C.POINTER(Zero1Sync), _P]),
    "b200amp_rs_pass1_f16_ce": (_I, [_P, _I, _I, _P, _P, _LL, _I, _P, _P, _P, C.POINTER(Zero1Sync), _P]),
    "b200amp_rs_push_f16_ce": (_I, [_P, _P, _I, _I, _LL, _I, C.POINTER(Zero1Sync), _P]),
    "b200amp_rs_pass1_f16_pushed": (_I, [_P, _P, _I, _I, _P, _LL, _I, _P, _P, _P, C.POINTER(Zero1Sync), _P]),
    "b200amp_pass2_ag_f16_ce": (_I, [_P, _P, _P, _P, _P, _I, _I, _LL, _LL, _P, _I, _P, _F, _F, _F, _I, _P]),
    "b200amp_step_f16": (_I, [_P, _P, _P, _P, _P, _LL, _P, _I, _P, _P, C.POINTER(ScheduleConfig), _P, _I,
                              _F, _F, _F, _P]),
    "b200amp_graph_begin_capture": (_I, [_P]),
    "b200amp_graph_end_capture": (_I, [_P, C.POINTER(_P)]),
    "b200amp_graph_launch": (_I, [_P, _P]),
    "b200amp_graph_destroy": (_I, [_P]),
    "b200amp_tune_set": (_I, [C.c_char_p, _I]),
    "b200amp_tune_get": (_I, [C.c_char_p, C.POINTER(_I)]),
    "b200amp_device_error": (_I, [C.POINTER(_I)]),
    "b200amp_launch_count": (_LL, []),
}

_lib = None


class B200AmpError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"b200amp status {status}: {text}")
        self.status = status


def lib_path() -> str:
    return _build.LIB_PATH


def load() -> C.CDLL:
    """The loaded library, prototypes set. Raises if the .so is absent: no fallback exists."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing. Build it with `python -m cuda_transformer_b200.build` "
            "(needs nvcc). There is no CPU or PyTorch fallback for the optimizer step.")
    lib = C.CDLL(path)
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)         # AttributeError here = the .so does not match the header
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        raise B200AmpError(status, load().b200amp_last_error().decode())
