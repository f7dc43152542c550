"""Shared by the tests: the reference's error metric, golden loading, arena helpers."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

from cuda_transformer_b200.layout import CONFIGS, param_layout, tensor_table

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances, from the benchmark definition: fp32 master/m/v within 1e-6 relative, fp16
# weights within 1 ulp, skip decisions and the loss-scale trajectory bit-exact.
STATE_TOL = 1e-6
REF_STEP_TOL = 1e-4         # the reference's own bar for AdamW (cuda/tests/test_fast.cu:40)


def rel_err(ref, got) -> float:
    """max |ref - got| / max finite |ref|: the reference's metric (cuda/dump.cu:244-268).
    NaN on either side is a failure (inf is returned)."""
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    assert ref.shape == got.shape, (ref.shape, got.shape)
    if np.isnan(ref).any() or np.isnan(got).any():
        return float("inf")
    scale = np.abs(ref[np.isfinite(ref)]).max() if ref.size else 0.0
    diff = np.abs(ref - got).max() if ref.size else 0.0
    return float(diff / scale) if scale > 0 else float(diff)


def half_ulp_distance(a_bits, b_bits) -> int:
    """Largest distance between two fp16 arrays in units of the last place (finite values)."""
    def ordered(bits):
        bits = np.asarray(bits, dtype=np.uint16).astype(np.int32)
        return np.where(bits & 0x8000, -(bits & 0x7FFF), bits & 0x7FFF)
    return int(np.abs(ordered(a_bits) - ordered(b_bits)).max())


def golden_meta() -> dict:
    with open(os.path.join(GOLDEN, "golden_meta.json")) as f:
        return json.load(f)


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


def debug_slots():
    return param_layout(CONFIGS["debug"])


def debug_shapes():
    return [s.shape for s in debug_slots()]


def debug_init() -> np.ndarray:
    return golden("debug_init.npz")["params"].astype(np.float32)


def table_of(slots):
    return tensor_table(slots)


def flat_np(tensors) -> np.ndarray:
    return torch.cat([t.reshape(-1) for t in tensors]).numpy()


def f16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)
