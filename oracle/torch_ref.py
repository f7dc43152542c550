"""The reference's PyTorch optimizer path on CPU, restated call for call.

TEST INFRASTRUCTURE and the timed CPU baseline of the benchmark; the library never
imports it. The arithmetic is torch's (third party, unpinned by the reference:
README.md:66 installs "torch numpy pytest" with no version); this file only repeats
the reference's sequence of calls:

    reference/model.py:254-260   two AdamW groups: weight decay on tensors with
                                 dim >= 2, none on the rest; foreach=False on CPU
    reference/train.py:69-74     torch.amp.GradScaler
    reference/train.py:147-153   scaler.unscale_(opt); clip_grad_norm_(params, clip);
                                 group["lr"] = lr; scaler.step(opt); scaler.update()

Parameters are separate tensors shaped as in the model (cuda_transformer_b200.layout
gives the same shapes as model.named_parameters()), so torch sees the same tensor
sizes the reference gives it.

accurate_norm=True replaces clip_grad_norm_ by clip_grads_with_norm_ with the norm
taken in fp64 and rounded to fp32 (what cuda/kernels/scaler.cu:118-138 computes):
torch's fp32 CPU norm is off by 1e-5..1e-2 at these tensor sizes, which moves the clip
coefficient far more than the 1e-6 parity bar allows.
"""
from __future__ import annotations

import math
import time
from typing import List, Sequence, Tuple

import torch


class TorchAmpStep:
    def __init__(self, shapes: Sequence[Tuple[int, ...]], init: Sequence[torch.Tensor], lr=6e-4, betas=(0.9, 0.95),
                 eps=1e-8, weight_decay=0.1, grad_clip=1.0, loss_scale=65536.0, growth_interval=2000,
                 use_scaler=True, accurate_norm=False):
        self.params: List[torch.nn.Parameter] = [torch.nn.Parameter(t.detach().clone().float().reshape(s))
                                                 for s, t in zip(shapes, init)]
        decay = [p for p in self.params if p.dim() >= 2]
        no_decay = [p for p in self.params if p.dim() < 2]
        groups = [{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}]
        self.opt = torch.optim.AdamW(groups, lr=lr, betas=betas, eps=eps, foreach=False)
        self.scaler = torch.amp.GradScaler("cpu", init_scale=loss_scale, growth_interval=growth_interval,
                                           enabled=use_scaler)
        if use_scaler:
            self.scaler.scale(torch.zeros(1))       # creates the scale tensor, as the first scale(loss) would
        self.lr = lr
        self.grad_clip = grad_clip
        self.accurate_norm = accurate_norm
        self.use_scaler = use_scaler
        self.last_norm = float("nan")

    def loss_scale(self) -> float:
        return float(self.scaler.get_scale()) if self.use_scaler else 1.0

    def set_grads(self, grads: Sequence[torch.Tensor]) -> None:
        """grads: loss-scaled gradients per tensor (fp16 or fp32); the parameters' .grad gets the
        fp32 widening, which is what a backward pass over fp32 parameters leaves."""
        for p, g in zip(self.params, grads):
            p.grad = g.detach().float().reshape(p.shape).clone()

    def step(self) -> None:
        """reference/train.py:147-153."""
        self.scaler.unscale_(self.opt)
        if self.accurate_norm:
            sq = sum(float(p.grad.double().pow(2).sum()) for p in self.params)
            total = torch.tensor(math.sqrt(sq), dtype=torch.float32) if math.isfinite(sq) else \
                torch.tensor(float("nan") if math.isnan(sq) else float("inf"), dtype=torch.float32)
            torch.nn.utils.clip_grads_with_norm_(self.params, self.grad_clip, total)
            self.last_norm = float(total)
        else:
            norm = torch.nn.utils.clip_grad_norm_(self.params, self.grad_clip)
            self.last_norm = float(norm)
        for group in self.opt.param_groups:
            group["lr"] = self.lr
        self.scaler.step(self.opt)
        self.scaler.update()

    def adam_steps(self) -> int:
        st = self.opt.state.get(self.params[0])
        return int(st["step"]) if st else 0

    def flat(self, what: str) -> torch.Tensor:
        """'p', 'm' or 'v' of every tensor, concatenated in arena order."""
        out = []
        for p in self.params:
            if what == "p":
                out.append(p.detach().reshape(-1))
            else:
                st = self.opt.state.get(p)
                key = "exp_avg" if what == "m" else "exp_avg_sq"
                out.append(st[key].reshape(-1) if st else torch.zeros(p.numel()))
        return torch.cat(out)


def _from_pool(pool: torch.Tensor, at: int, count: int) -> torch.Tensor:
    """count values of the pool starting at `at`, wrapping around (a fresh tensor)."""
    size = pool.numel()
    at %= size
    if at + count <= size:
        return pool[at:at + count].clone()
    reps = (at + count + size - 1) // size
    return pool.repeat(reps)[at:at + count].clone()


def time_cpu_step(shapes: Sequence[Tuple[int, ...]], steps: int = 5, warmup: int = 1, loss_scale: float = 32768.0,
                  seed: int = 0) -> dict:
    """Time the stock path (clip_grad_norm_) on the host cores with all torch threads.
    Returns {"seconds_per_step", "params", "threads"}. Parameters and gradients are N(0, 0.02) and
    N(0, 1e-3) * loss_scale drawn from one seeded pool of 2^26 normal values that the tensors
    slice (with wrap-around): the distributions are the workload's, and drawing 1.3 G fresh
    normals per step on one host thread would take longer than the steps being timed. Every step
    sees the same fp16 gradients, widened to fp32 again before it (outside the timer: unscale_
    overwrites .grad in place)."""
    gen = torch.Generator().manual_seed(seed)
    pool = torch.randn(1 << 26, generator=gen)
    sizes = [int(torch.Size(s).numel()) for s in shapes]
    init, grads, at = [], [], 0
    for s, k in zip(shapes, sizes):
        init.append((_from_pool(pool, at, k) * 0.02).reshape(s))
        grads.append((_from_pool(pool, at + 12345, k) * (1e-3 * loss_scale)).half().reshape(s))
        at += k
    del pool
    ref = TorchAmpStep(shapes, init, loss_scale=loss_scale)
    del init
    n = sum(p.numel() for p in ref.params)
    times = []
    for k in range(warmup + steps):
        ref.set_grads(grads)
        t0 = time.perf_counter()
        ref.step()
        dt = time.perf_counter() - t0
        if k >= warmup:
            times.append(dt)
    times.sort()
    return {"seconds_per_step": times[len(times) // 2], "params": n, "threads": torch.get_num_threads(),
            "steps": steps}
