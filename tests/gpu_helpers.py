"""GPU-side twin of oracle.ref_step.OracleStep for the parity tests: the same arenas in
device memory, stepped through the library's C ABI (cuda_transformer_b200.amp wrappers)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from cuda_transformer_b200 import amp
from cuda_transformer_b200._lib import StepState, TensorInfo, load


def to_dev(a: np.ndarray, dtype=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype)
    return t.cuda()


def table_dev(table) -> torch.Tensor:
    arr = (TensorInfo * len(table))(*[TensorInfo(o, c, d) for o, c, d in table])
    return torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).cuda()


def read_struct(t: torch.Tensor, index: int = 0) -> StepState:
    size = C.sizeof(StepState)
    raw = t.cpu().numpy().tobytes()
    return StepState.from_buffer_copy(raw[index * size:(index + 1) * size])


class GpuStep:
    """master/m/v fp32, weights16 + grads16 fp16 on cuda:0; table = [(offset, count, decay)]."""

    def __init__(self, master: np.ndarray, table, cfg, eps: float = 1e-8, loss_scale: float = 65536.0,
                 history_len: int = 256, arena_offset: int = 0):
        self.lib = load()
        self.n = int(master.size)
        self.cfg = cfg
        self.eps = eps
        self.arena_offset = arena_offset
        self.master = to_dev(master.astype(np.float32))
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.weights16 = torch.zeros(self.n, dtype=torch.float16, device="cuda")
        amp.cast_to_x(self.weights16, self.master, self.n)
        self.grads16 = torch.zeros(self.n, dtype=torch.float16, device="cuda")
        self.grads32 = None
        self.tensors = table_dev(table)
        self.ntensors = len(table)
        self.history_len = history_len
        self.history = torch.zeros(C.sizeof(StepState) * history_len, dtype=torch.uint8, device="cuda")
        self.state = torch.frombuffer(bytearray(bytes(amp.initial_state(loss_scale))), dtype=torch.uint8).cuda()
        self.workspace = torch.zeros(self.lib.b200amp_workspace_bytes(), dtype=torch.uint8, device="cuda")
        self.partial = torch.zeros(512, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()

    # ---- native path
    def set_grads16(self, bits: np.ndarray) -> None:
        self.grads16.copy_(torch.from_numpy(np.ascontiguousarray(bits, dtype=np.uint16)).view(torch.float16))

    def step_f16(self) -> None:
        amp.step_f16(self.master, self.m, self.v, self.grads16, self.weights16, self.n, self.tensors, self.ntensors,
                     self.state, self.workspace, self.cfg, self.history, self.history_len, self.cfg.beta1,
                     self.cfg.beta2, self.eps)

    # ---- compat path (the reference's arguments: fp32 gradients unscaled in place)
    def step_f32(self, grads_scaled: np.ndarray) -> torch.Tensor:
        g = to_dev(grads_scaled.astype(np.float32))
        amp.begin_step(self.state)
        amp.unscale_and_norm(g, self.n, self.state, self.partial)
        amp.finalize_step(self.state, self.partial, self.cfg, self.history, self.history_len)
        amp.adamw_multi(self.master, self.weights16, g, self.m, self.v, self.n, self.tensors, self.ntensors,
                        self.state, self.cfg.beta1, self.cfg.beta2, self.eps)
        return g

    def read_state(self) -> StepState:
        return read_struct(self.state)

    def host(self):
        """(master, m, v, weights16 bits) as numpy."""
        torch.cuda.synchronize()
        return (self.master.cpu().numpy(), self.m.cpu().numpy(), self.v.cpu().numpy(),
                self.weights16.cpu().view(torch.int16).numpy().view(np.uint16))


def assert_states_equal(got: StepState, want, exact_fields=("loss_scale", "inv_scale", "good_steps", "found_inf",
                                                             "skipped", "step", "adam_t"),
                        close_fields=("lr", "grad_norm", "clip_coef", "step_size", "bc2_sqrt", "decay"),
                        tol: float = 1e-6) -> None:
    for f in exact_fields:
        assert getattr(got, f) == getattr(want, f), (f, getattr(got, f), getattr(want, f))
    for f in close_fields:
        a, b = float(getattr(got, f)), float(getattr(want, f))
        if np.isnan(b):
            assert np.isnan(a), f
        elif np.isinf(b):
            assert a == b, f
        else:
            assert abs(a - b) <= tol * max(abs(b), 1e-30), (f, a, b)
