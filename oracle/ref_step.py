"""ctypes binding of oracle/ref_step.c plus a numpy-level driver of the whole step.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
leg of the benchmark, always as the checker. The library never imports it.

OracleStep runs the reference's sequence (cuda/gpt_fast.cu:438-450: unscale_and_norm ->
finalize_step -> adamw_multi, after begin_step) on numpy arrays, for fp32 gradients
(the reference's own arena type) or for an fp16 gradient arena (the widening is exact,
so the per-element inputs are identical).
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

from . import build as _oracle_build    # oracle/build.py


class StepState(C.Structure):
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


class Schedule(C.Structure):
    _fields_ = [
        ("lr", C.c_float), ("min_lr", C.c_float),
        ("warmup_steps", C.c_int), ("max_steps", C.c_int),
        ("beta1", C.c_float), ("beta2", C.c_float),
        ("weight_decay", C.c_float), ("grad_clip", C.c_float),
        ("growth_interval", C.c_int), ("dynamic_scale", C.c_int), ("decay_steps", C.c_int),
    ]


class TensorInfo(C.Structure):
    _fields_ = [("offset", C.c_longlong), ("count", C.c_longlong), ("decay", C.c_int)]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    lib = C.CDLL(_oracle_build.build())
    P, LL, I, F, D = C.c_void_p, C.c_longlong, C.c_int, C.c_float, C.c_double
    protos = {
        "oracle_sizeof_state": (I, []),
        "oracle_sizeof_schedule": (I, []),
        "oracle_sizeof_tensor_info": (I, []),
        "oracle_half_to_float": (F, [C.c_uint16]),
        "oracle_float_to_half": (C.c_uint16, [F]),
        "oracle_initial_state": (None, [F, C.POINTER(StepState)]),
        "oracle_begin_step": (None, [C.POINTER(StepState)]),
        "oracle_lr": (D, [I, C.POINTER(Schedule)]),
        "oracle_finalize_sumsq": (None, [C.POINTER(StepState), D, C.POINTER(Schedule), P, I]),
        "oracle_tree_sum": (D, [P]),
        "oracle_finalize": (None, [C.POINTER(StepState), P, C.POINTER(Schedule), P, I]),
        "oracle_unscale_and_norm_f32": (None, [P, LL, C.POINTER(StepState), P, I]),
        "oracle_adamw_multi": (None, [P, P, P, P, P, LL, LL, P, I, C.POINTER(StepState), F, F, F, I]),
        "oracle_pass1_f16": (None, [P, LL, F, C.POINTER(D), C.POINTER(I)]),
        "oracle_unscale_f16": (None, [P, LL, F, P]),
        "oracle_cast_to_half": (None, [P, P, LL]),
    }
    for name, (res, args) in protos.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    assert lib.oracle_sizeof_state() == 60 and lib.oracle_sizeof_schedule() == 44
    assert lib.oracle_sizeof_tensor_info() == 24
    _lib = lib
    return lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def make_schedule(lr=6e-4, min_lr=6e-4, warmup_steps=0, max_steps=1 << 30, beta1=0.9, beta2=0.95,
                  weight_decay=0.1, grad_clip=1.0, growth_interval=2000, dynamic_scale=1, decay_steps=0) -> Schedule:
    return Schedule(lr, min_lr, warmup_steps, max_steps, beta1, beta2, weight_decay, grad_clip, growth_interval,
                    dynamic_scale, decay_steps)


def initial_state(scale: float) -> StepState:
    st = StepState()
    load().oracle_initial_state(scale, C.byref(st))
    return st


def lr_at(step: int, cfg: Schedule) -> float:
    return load().oracle_lr(step, C.byref(cfg))


def half_to_float(bits: np.ndarray) -> np.ndarray:
    lib = load()
    return np.array([lib.oracle_half_to_float(int(b)) for b in bits.reshape(-1)], dtype=np.float32)


def float_to_half(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    load().oracle_cast_to_half(_p(out), _p(x), x.size)
    return out


def tensor_table(table) -> C.Array:
    return (TensorInfo * len(table))(*[TensorInfo(o, c, d) for o, c, d in table])


class OracleStep:
    """The step on numpy arrays. master/m/v fp32, weights16 as uint16 bit patterns.

    contract: 0 = every operation rounded separately (torch's CPU arithmetic);
              bit 0 = fused multiply-adds, bits 1 and 2 pick which product of a two-product sum
              is fused (see ref_step.c). 3 is what nvcc 12.9 makes of the reference's expressions:
              on a B200 it reproduces the reference's compiled kernels bit for bit.
    arena_offset / n: a shard of a larger arena may be driven on its own (ZeRO-1 checks).
    """

    def __init__(self, master: np.ndarray, table, cfg: Schedule, eps: float = 1e-8, loss_scale: float = 65536.0,
                 history_len: int = 256, contract: int = 3, arena_offset: int = 0):
        self.lib = load()
        self.master = np.ascontiguousarray(master, dtype=np.float32).copy()
        self.n = self.master.size
        assert self.n % 4 == 0
        self.m = np.zeros(self.n, dtype=np.float32)
        self.v = np.zeros(self.n, dtype=np.float32)
        self.weights16 = float_to_half(self.master)
        self.table = tensor_table(table)
        self.ntensors = len(table)
        self.cfg = cfg
        self.eps = eps
        self.contract = contract
        self.arena_offset = arena_offset
        self.state = initial_state(loss_scale)
        self.history_len = history_len
        self.history = (StepState * history_len)()
        self.partial = np.zeros(512, dtype=np.float32)

    # -- the reference's sequence on its own arena type (fp32 gradients, unscaled in place)
    def step_f32(self, grads_scaled: np.ndarray) -> np.ndarray:
        """begin_step, unscale_and_norm, finalize_step, adamw_multi. Returns the unscaled gradients."""
        g = np.ascontiguousarray(grads_scaled, dtype=np.float32).copy()
        lib = self.lib
        lib.oracle_begin_step(C.byref(self.state))
        lib.oracle_unscale_and_norm_f32(_p(g), self.n, C.byref(self.state), _p(self.partial), self.contract)
        lib.oracle_finalize(C.byref(self.state), _p(self.partial), C.byref(self.cfg),
                            C.cast(self.history, C.c_void_p), self.history_len)
        self._adamw(g)
        return g

    # -- the same step fed from an fp16 gradient arena (uint16 bit patterns)
    def pass1_f16(self, grads16: np.ndarray):
        """(sum of squares, flag) of the unscaled slice; touches no state."""
        g16 = np.ascontiguousarray(grads16, dtype=np.uint16)
        sumsq, bad = C.c_double(), C.c_int()
        self.lib.oracle_pass1_f16(_p(g16), g16.size, self.state.loss_scale, C.byref(sumsq), C.byref(bad))
        return sumsq.value, bad.value

    def finalize_sums(self, pairs) -> None:
        """pairs: [(sumsq, flag), ...] in rank order; sets inv_scale/found_inf, then scaler.cu:131-170."""
        total, bad = 0.0, 0
        for s, f in pairs:
            total += s
            bad |= 1 if f else 0
        self.state.inv_scale = np.float32(1.0) / np.float32(self.state.loss_scale)
        self.state.found_inf = bad
        self.lib.oracle_finalize_sumsq(C.byref(self.state), total, C.byref(self.cfg),
                                       C.cast(self.history, C.c_void_p), self.history_len)

    def pass2_f16(self, grads16: np.ndarray) -> None:
        g16 = np.ascontiguousarray(grads16, dtype=np.uint16)
        g = np.empty(self.n, dtype=np.float32)
        self.lib.oracle_unscale_f16(_p(g16), self.n, self.state.inv_scale, _p(g))
        self._adamw(g)

    def step_f16(self, grads16: np.ndarray) -> None:
        self.finalize_sums([self.pass1_f16(grads16)])
        self.pass2_f16(grads16)

    def _adamw(self, g_unscaled: np.ndarray) -> None:
        self.lib.oracle_adamw_multi(_p(self.master), _p(self.weights16), _p(g_unscaled), _p(self.m), _p(self.v),
                                    self.n, self.arena_offset, C.cast(self.table, C.c_void_p), self.ntensors,
                                    C.byref(self.state), self.cfg.beta1, self.cfg.beta2, self.eps, self.contract)
