"""GPTC version 2 checkpoints: the reference's resume format (cuda/checkpoint.h:5-22), written
and read on the host so that the optimizer state of this library (one GPU or ZeRO-1 shards)
can be resumed by the reference's `train_fast -r`, and the other way round.

Layout, little endian (cuda/checkpoint.cu:69-113 writes it, :195-270 reads it):
    "GPTC", u32 version = 2
    i32 V, Vp, n_ctx, L, H, C; f32 ln_eps
    i32 B, max_steps, eval_every, warmup_steps, sft; f32 lr, min_lr; f32 best_val; i32 best_step
    u32 sizeof(StepState) = 60, the 60 StepState bytes
    str data, str starts                       (u32 length + bytes)
    i32 decay_steps, f32 beta2, str keep, str branch
    u64 n, f32 params[n], m[n], v[n]
The write goes to path.tmp, is fsync'ed and renamed over path (cuda/checkpoint.cu:114-135), so
a crash never leaves half a file under the real name.
"""
from __future__ import annotations

import ctypes as C
import os
import struct
from dataclasses import dataclass, field

import numpy as np

from ._lib import StepState

MAGIC = b"GPTC"
VERSION = 2


@dataclass
class ModelShape:          # cuda/config.h:7-21
    V: int = 0
    Vp: int = 0
    n_ctx: int = 0
    L: int = 0
    H: int = 0
    C: int = 0
    ln_eps: float = 1e-5


@dataclass
class RunInfo:             # cuda/checkpoint.h:31-46
    B: int = 0
    max_steps: int = 0
    eval_every: int = 0
    warmup_steps: int = 0
    sft: int = 0
    lr: float = 0.0
    min_lr: float = 0.0
    data: str = ""
    starts: str = ""
    decay_steps: int = 0
    beta2: float = 0.95
    keep: str = ""
    branch: str = ""
    best_val: float = 0.0
    best_step: int = 0


@dataclass
class Checkpoint:          # cuda/checkpoint.h:48-54
    cfg: ModelShape = field(default_factory=ModelShape)
    run: RunInfo = field(default_factory=RunInfo)
    state: StepState = field(default_factory=StepState)
    params: np.ndarray = field(default_factory=lambda: np.zeros(0, dtype=np.float32))
    m: np.ndarray = field(default_factory=lambda: np.zeros(0, dtype=np.float32))
    v: np.ndarray = field(default_factory=lambda: np.zeros(0, dtype=np.float32))


class CheckpointError(RuntimeError):
    pass


def _s(text: str) -> bytes:
    raw = text.encode()
    return struct.pack("<I", len(raw)) + raw


def write_checkpoint(path: str, c: Checkpoint) -> None:
    n = c.params.size
    if c.m.size != n or c.v.size != n:
        raise CheckpointError(f"checkpoint arrays of {n}, {c.m.size} and {c.v.size} values")
    head = bytearray()
    head += MAGIC + struct.pack("<I", VERSION)
    m = c.cfg
    head += struct.pack("<6if", m.V, m.Vp, m.n_ctx, m.L, m.H, m.C, m.ln_eps)
    r = c.run
    head += struct.pack("<5i2ffi", r.B, r.max_steps, r.eval_every, r.warmup_steps, r.sft, r.lr, r.min_lr, r.best_val,
                        r.best_step)
    head += struct.pack("<I", C.sizeof(StepState)) + bytes(c.state)
    head += _s(r.data) + _s(r.starts)
    head += struct.pack("<if", r.decay_steps, r.beta2)
    head += _s(r.keep) + _s(r.branch)
    head += struct.pack("<Q", n)
    tmp = path + ".tmp"
    try:
        with open(tmp, "wb") as f:
            f.write(head)
            for arr in (c.params, c.m, c.v):
                f.write(np.ascontiguousarray(arr, dtype="<f4").tobytes())
            f.flush()
            os.fsync(f.fileno())
    except OSError as e:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise CheckpointError(f"writing {tmp} failed ({e}); the last checkpoint is still {path}") from e
    os.replace(tmp, path)


class _Reader:
    def __init__(self, buf: bytes):
        self.buf, self.at = buf, 0

    def take(self, n: int) -> bytes:
        if len(self.buf) - self.at < n:
            raise CheckpointError("the file is cut short")
        out = self.buf[self.at:self.at + n]
        self.at += n
        return out

    def unpack(self, fmt: str):
        return struct.unpack("<" + fmt, self.take(struct.calcsize("<" + fmt)))

    def text(self) -> str:
        (n,) = self.unpack("I")
        return self.take(n).decode()


def read_checkpoint(path: str) -> Checkpoint:
    """Versions 1 and 2 (a version 1 file reads as decay_steps 0, beta2 0.95, no keep list, no branch)."""
    try:
        with open(path, "rb") as f:
            buf = f.read()
    except OSError as e:
        raise CheckpointError(f"cannot open {path}") from e
    r = _Reader(buf)
    if len(buf) < 4 or r.take(4) != MAGIC:
        raise CheckpointError("not a GPTC checkpoint")
    (version,) = r.unpack("I")
    if version not in (1, VERSION):
        raise CheckpointError(f"version {version}, this code reads versions 1 and 2")
    c = Checkpoint()
    V, Vp, n_ctx, L, H, Cw, eps = r.unpack("6if")
    c.cfg = ModelShape(V, Vp, n_ctx, L, H, Cw, eps)
    B, max_steps, eval_every, warmup, sft, lr, min_lr, best_val, best_step = r.unpack("5i2ffi")
    (state_bytes,) = r.unpack("I")
    if state_bytes != C.sizeof(StepState):
        raise CheckpointError(f"its StepState is {state_bytes} bytes, this build's is {C.sizeof(StepState)}")
    c.state = StepState.from_buffer_copy(r.take(state_bytes))
    data, starts = r.text(), r.text()
    decay_steps, beta2, keep, branch = 0, 0.95, "", ""
    if version >= 2:
        decay_steps, beta2 = r.unpack("if")
        keep, branch = r.text(), r.text()
    c.run = RunInfo(B, max_steps, eval_every, warmup, sft, lr, min_lr, data, starts, decay_steps, beta2, keep, branch,
                    best_val, best_step)
    (n,) = r.unpack("Q")
    if len(buf) - r.at != 12 * n:
        raise CheckpointError(f"{n} parameters announced, {len(buf) - r.at} bytes of arrays follow")
    arrays = np.frombuffer(buf, dtype="<f4", count=3 * n, offset=r.at).astype(np.float32)
    c.params, c.m, c.v = arrays[:n].copy(), arrays[n:2 * n].copy(), arrays[2 * n:].copy()
    return c


# ---------------------------------------------------------------- optimizer <-> checkpoint

def checkpoint_of(opt, cfg: ModelShape, run: RunInfo) -> Checkpoint:
    """The optimizer's weights, moments and step state (cuda/checkpoint.cu:288-299). Works for
    AmpOptimizer (whole arena) and for the ZeRO-1 optimizers: there every rank must call it (the
    shards are all-gathered) and every rank gets the full checkpoint; write it from one rank."""
    import torch
    n = opt.n_params
    if hasattr(opt, "world"):
        full = []
        for shard in (opt.master, opt.m, opt.v):
            out = torch.empty(opt.n, dtype=torch.float32, device=shard.device)
            opt.dist.all_gather_into_tensor(out, shard.contiguous(), group=opt.group)
            full.append(out[:n].cpu().numpy())
    else:
        full = [t[:n].cpu().numpy() for t in (opt.master, opt.m, opt.v)]
    return Checkpoint(cfg, run, opt.read_state(), full[0], full[1], full[2])


def restore(opt, c: Checkpoint) -> None:
    """Back into an optimizer of the same size; rebuilds the fp16 weight copy
    (cuda/checkpoint.cu:301-315). On a ZeRO-1 optimizer every rank calls it with the same file."""
    import torch
    if c.params.size != opt.n_params:
        raise CheckpointError(f"{c.params.size} parameters in the checkpoint, the optimizer holds {opt.n_params}")
    opt.set_params(torch.from_numpy(c.params))
    begin, end = (opt.begin, opt.end) if hasattr(opt, "world") else (0, opt.n)
    for dst, src in ((opt.m, c.m), (opt.v, c.v)):
        padded = np.zeros(opt.n, dtype=np.float32)
        padded[:opt.n_params] = src
        dst.copy_(torch.from_numpy(padded[begin:end]))
    opt.grads16.zero_()
    opt.write_state(c.state)
