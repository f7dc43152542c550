"""The flat parameter arena: which tensor lives where.

Mirrors param_layout() of the reference (cuda/gpt.cu:71-103, cuda/layout.h:35-51):
parameters sit back to back in model.named_parameters() order, and gradients, m, v
and the fp16 weight copy use the same offsets. Weight decay applies to tensors with
ndim >= 2 (reference/model.py:254-256, cuda/gpt_fast.cu:108-113).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

ARENA_ALIGN = 8 * 128       # elements: shards of 1/2/4/8 ranks stay 256-byte aligned in fp16


@dataclass(frozen=True)
class ModelConfig:
    name: str
    L: int          # layers
    H: int          # heads (does not change the parameter count)
    C: int          # width
    Vp: int         # padded vocabulary
    n_ctx: int


@dataclass(frozen=True)
class ParamSlot:
    name: str
    offset: int     # elements from the start of the arena
    count: int
    ndim: int
    shape: Tuple[int, ...]


# The configurations the benchmark definition names.
CONFIGS = {
    "debug": ModelConfig("debug", L=2, H=4, C=64, Vp=4160, n_ctx=64),                   # 370,432 params
    "readme": ModelConfig("readme", L=6, H=6, C=384, Vp=4160, n_ctx=256),               # 12,343,296
    "gpt2-small": ModelConfig("gpt2-small", L=12, H=12, C=768, Vp=50304, n_ctx=1024),   # 124,475,904
    "1.3b": ModelConfig("1.3b", L=24, H=16, C=2048, Vp=50304, n_ctx=2048),              # 1,315,819,520
}


def param_layout(cfg: ModelConfig) -> List[ParamSlot]:
    """Slots in arena order: wte, wpe, 12 tensors per layer, ln_f.w, ln_f.b."""
    slots: List[ParamSlot] = []
    offset = 0
    C = cfg.C

    def add(name: str, shape: Tuple[int, ...]) -> None:
        nonlocal offset
        count = 1
        for d in shape:
            count *= d
        slots.append(ParamSlot(name, offset, count, len(shape), shape))
        offset += count

    add("wte", (cfg.Vp, C))
    add("wpe", (cfg.n_ctx, C))
    for l in range(cfg.L):
        p = f"h.{l}."
        add(p + "ln1.w", (C,))
        add(p + "ln1.b", (C,))
        add(p + "attn.c_attn.w", (3 * C, C))
        add(p + "attn.c_attn.b", (3 * C,))
        add(p + "attn.c_proj.w", (C, C))
        add(p + "attn.c_proj.b", (C,))
        add(p + "ln2.w", (C,))
        add(p + "ln2.b", (C,))
        add(p + "mlp.c_fc.w", (4 * C, C))
        add(p + "mlp.c_fc.b", (4 * C,))
        add(p + "mlp.c_proj.w", (C, 4 * C))
        add(p + "mlp.c_proj.b", (C,))
    add("ln_f.w", (C,))
    add("ln_f.b", (C,))
    return slots


def num_params(slots: List[ParamSlot]) -> int:
    return slots[-1].offset + slots[-1].count


def padded(n: int, align: int = ARENA_ALIGN) -> int:
    """Arena length: n rounded up so every 1/2/4/8-way shard is a multiple of 128 elements."""
    return (n + align - 1) // align * align


def tensor_table(slots: List[ParamSlot]) -> List[Tuple[int, int, int]]:
    """(offset, count, decay) per tensor; decay = 1 for >= 2-D tensors (cuda/gpt_fast.cu:108-113).
    Padding past the last tensor takes the last tensor's flag, as the reference's search would."""
    return [(s.offset, s.count, 1 if s.ndim >= 2 else 0) for s in slots]


def shard_range(n_padded: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the arena owned by rank: equal contiguous slices."""
    assert n_padded % (world * 128) == 0, "arena must be padded to a multiple of world * 128 elements"
    per = n_padded // world
    return rank * per, (rank + 1) * per
