"""Seeded synthetic inputs shared by the fixture generator and the tests.

Gradients follow the benchmark definition: for every step, for every parameter in
arena order, randn(shape) * 1e-3 from one torch CPU generator seeded once. The AMP
variants multiply by the CURRENT loss scale before rounding to fp16, so the unscaled
values stay N(0, 1e-3) whatever the scale does.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


class GradStream:
    def __init__(self, shapes: Sequence[Tuple[int, ...]], seed: int = 1, std: float = 1e-3):
        self.shapes = list(shapes)
        self.gen = torch.Generator().manual_seed(seed)
        self.std = std

    def next_fp32(self) -> List[torch.Tensor]:
        return [torch.randn(s, generator=self.gen) * self.std for s in self.shapes]

    def next_fp16_scaled(self, loss_scale: float) -> List[torch.Tensor]:
        return [(torch.randn(s, generator=self.gen) * self.std * loss_scale).half() for s in self.shapes]


def flatten(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat([t.reshape(-1) for t in tensors])


def inject(grads: List[torch.Tensor], tensor_index: int, element_index, value: float) -> None:
    """Overwrite elements of one tensor of a per-tensor gradient list (host-side fault injection)."""
    flat = grads[tensor_index].reshape(-1)
    flat[torch.as_tensor(element_index, dtype=torch.long)] = value
