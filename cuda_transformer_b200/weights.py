"""weights.bin, the reference's one weight file (cuda/weights.h:1-14): what `train_fast` writes
after training (cuda/train_fast.cu:915) and what `GPT::load`, `FastGPT` and `generate` read.
Written and read on the host so that the arenas this library updates leave and enter in the
format every program of the reference understands.

Layout, little endian (cuda/weights.cu:16-27 is the 48-byte header):
    u32 magic 0x57545047 ("GPTW"), u32 version = 1
    u32 V, Vp, n_ctx, L, H, C; f32 ln_eps
    u32 dtype (0 = float32, 1 = float16); u64 count
    count values in arena order (the unpadded parameter count of a model of these sizes)
The write goes to path.tmp and is renamed over path (cuda/weights.cu:110-138).
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass

import numpy as np

from .checkpoint import ModelShape
from .layout import ModelConfig, num_params, param_layout

MAGIC = 0x57545047
VERSION = 1
HEADER = struct.Struct("<8I f I Q")
assert HEADER.size == 48


class WeightsError(RuntimeError):
    pass


@dataclass
class Weights:
    cfg: ModelShape
    params: np.ndarray          # float32, as the reference's reader returns them
    dtype: int                  # what the file held: 0 = float32, 1 = float16


def expected_count(cfg: ModelShape) -> int:
    """Parameters of a model of these sizes (cuda/weights.cu:29-33)."""
    return num_params(param_layout(ModelConfig("file", L=cfg.L, H=cfg.H, C=cfg.C, Vp=cfg.Vp, n_ctx=cfg.n_ctx)))


def _host(values) -> np.ndarray:
    if hasattr(values, "detach"):                       # a torch tensor, on any device
        values = values.detach().cpu().numpy()
    return np.ascontiguousarray(values)


def write_weights(path: str, cfg: ModelShape, values, fp16: bool = False) -> None:
    """`values`: the master arena (float32) or the fp16 weight arena (float16), numpy or torch,
    padded or not: the first expected_count(cfg) elements are written. A float32 arena written
    with fp16=True is rounded to nearest even, which is what the reference's writer
    (`__float2half`, cuda/weights.cu:120-126) and pass 2 of this library both do, so the file
    equals the one written from the fp16 arena."""
    n = expected_count(cfg)
    arr = _host(values).reshape(-1)
    if arr.size < n:
        raise WeightsError(f"writing {arr.size} values, a model of these sizes has {n}")
    if arr.dtype not in (np.float32, np.float16):
        raise WeightsError(f"weights must be float32 or float16, not {arr.dtype}")
    arr = arr[:n]
    if fp16:
        with np.errstate(over="ignore"):                # beyond 65504 becomes inf, as __float2half does
            body = arr.astype(np.float16, copy=False)
    else:
        body = arr.astype(np.float32, copy=False)
    head = HEADER.pack(MAGIC, VERSION, cfg.V, cfg.Vp, cfg.n_ctx, cfg.L, cfg.H, cfg.C, cfg.ln_eps, 1 if fp16 else 0, n)
    tmp = path + ".tmp"
    try:
        with open(tmp, "wb") as f:
            f.write(head)
            f.write(body.tobytes())
    except OSError as e:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise WeightsError(f"writing {tmp} failed ({e})") from e
    os.replace(tmp, path)


def read_weights(path: str) -> Weights:
    """The checks of the reference's reader (cuda/weights.cu:35-98), as exceptions."""
    try:
        raw = open(path, "rb").read()
    except OSError as e:
        raise WeightsError(f"cannot open {path}") from e
    if len(raw) < HEADER.size or int.from_bytes(raw[:4], "little") != MAGIC:
        raise WeightsError(f"{path} is not a weights.bin file")
    magic, version, V, Vp, n_ctx, L, H, C, ln_eps, dtype, count = HEADER.unpack_from(raw)
    if version != VERSION or dtype > 1:
        raise WeightsError(f"{path} has version {version} dtype {dtype}, this reader takes version 1, dtype 0 or 1")
    if H <= 0 or C % H != 0 or Vp < V:
        raise WeightsError(f"bad sizes in {path} (C {C}, H {H}, V {V}, Vp {Vp})")
    cfg = ModelShape(V, Vp, n_ctx, L, H, C, ln_eps)
    n = expected_count(cfg)
    if count != n:
        raise WeightsError(f"{path} holds {count} values, a model of its sizes has {n}")
    width = 2 if dtype == 1 else 4
    if len(raw) != HEADER.size + n * width:
        raise WeightsError(f"{path} is the wrong size for {n} values")
    body = np.frombuffer(raw, dtype=np.float16 if dtype == 1 else np.float32, count=n, offset=HEADER.size)
    return Weights(cfg, body.astype(np.float32), dtype)


def load_into(opt, w: Weights) -> None:
    """Puts the file's parameters into an optimizer's master arena and rebuilds its fp16 copy,
    as FastGPT::set_params does after read_weights (cuda/gpt_fast.cu:274-286)."""
    import torch
    opt.set_params(torch.from_numpy(w.params))
