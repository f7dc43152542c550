"""Generates the golden fixtures in this directory by running the REFERENCE's own
PyTorch path. Needs the reference checkout; run by hand where it is mounted:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/cuda-transformer

The tests never import the reference: they read the .npz/.json files written here.

What is run, and where it comes from in the reference:
  * the model and its initial weights: reference.model.GPT(tiny_model_config(4098))
    after torch.manual_seed(0) (reference/model.py:190-211, reference/config.py:103-105);
  * the optimizer: GPT.optimizer(TrainConfig) (reference/model.py:246-260);
  * one step: the calls of reference.train.train_step after backward
    (reference/train.py:147-153), through oracle/torch_ref.py for the AMP fixture so the
    accurate-norm variant can be selected;
  * the answer-key records params / grad.* / step1.* / grad_norm:
    reference.dump.build_records (reference/dump.py:104-158) on the random-token
    fallback the reference's tests use (reference/test_reference.py:40-45).
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
sys.path.insert(0, HERE)

from inputs import GradStream, flatten, inject  # noqa: E402

STRIDE = 16                 # p/m/v are stored at every 16th element (plus per-tensor fp64 sums)


def per_tensor_sums(flat: torch.Tensor, sizes) -> np.ndarray:
    out, at = [], 0
    for n in sizes:
        out.append(float(flat[at:at + n].double().sum()))
        at += n
    return np.array(out, dtype=np.float64)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from reference import dump as ref_dump
    from reference.config import DUMP_BATCH, TrainConfig, tiny_model_config
    from reference.model import GPT
    from oracle.torch_ref import TorchAmpStep

    torch.set_num_threads(1)    # one thread: reductions inside torch do not depend on the machine
    cfg = tiny_model_config(4098)
    tc = TrainConfig()

    # ---------------------------------------------------------------- initial weights
    torch.manual_seed(0)
    model = GPT(cfg)
    names = [n for n, _ in model.named_parameters()]
    shapes = [tuple(p.shape) for p in model.parameters()]
    sizes = [p.numel() for p in model.parameters()]
    init = [p.detach().clone() for p in model.parameters()]
    np.savez_compressed(os.path.join(HERE, "debug_init.npz"), params=flatten(init).numpy())
    meta = {"names": names, "shapes": [list(s) for s in shapes], "torch": torch.__version__,
            "lr": tc.lr, "beta1": tc.beta1, "beta2": tc.beta2, "eps": tc.eps, "weight_decay": tc.weight_decay,
            "grad_clip": tc.grad_clip, "stride": STRIDE}

    # ---------------------------------------------------------------- fp32 path, 10 steps, the model's own optimizer
    opt = model.optimizer(tc)
    scaler = torch.amp.GradScaler("cpu", enabled=False)
    stream = GradStream(shapes, seed=1)
    params = list(model.parameters())
    norms, first_grad_sum = [], None
    saved = {}
    for step in range(10):
        grads = stream.next_fp32()
        if first_grad_sum is None:
            first_grad_sum = float(flatten(grads).double().sum())
        for p, g in zip(params, grads):
            p.grad = g.clone()
        # reference/train.py:147-153
        scaler.unscale_(opt)
        norm = torch.nn.utils.clip_grad_norm_(model.parameters(), tc.grad_clip)
        for group in opt.param_groups:
            group["lr"] = tc.lr
        scaler.step(opt)
        scaler.update()
        norms.append(float(norm))
        if step in (0, 9):
            p_flat = flatten([p.detach() for p in params])
            m_flat = flatten([opt.state[p]["exp_avg"] for p in params])
            v_flat = flatten([opt.state[p]["exp_avg_sq"] for p in params])
            tag = f"step{step + 1}"
            saved[tag + "_p"] = p_flat[::STRIDE].numpy().copy()
            saved[tag + "_m"] = m_flat[::STRIDE].numpy().copy()
            saved[tag + "_v"] = v_flat[::STRIDE].numpy().copy()
            saved[tag + "_p_sums"] = per_tensor_sums(p_flat, sizes)
            saved[tag + "_m_sums"] = per_tensor_sums(m_flat, sizes)
            saved[tag + "_v_sums"] = per_tensor_sums(v_flat, sizes)
    saved["norms"] = np.array(norms, dtype=np.float32)
    saved["first_grad_sum"] = np.array([first_grad_sum])
    np.savez_compressed(os.path.join(HERE, "debug_fp32_10steps.npz"), **saved)

    # ---------------------------------------------------------------- AMP path, 100 steps, injected overflows
    amp = {"loss_scale": 65536.0, "growth_interval": 8, "grad_clip": 0.25, "steps": 100}
    pick = torch.Generator().manual_seed(2)
    injections = {}
    for step, value in ((3, "inf"), (17, "inf"), (40, "inf"), (55, "nan")):
        t = int(torch.randint(len(shapes), (1,), generator=pick))
        if value == "inf":
            k = max(1, sizes[t] // 1000)
            idx = torch.randperm(sizes[t], generator=pick)[:k].tolist()
        else:
            idx = [int(torch.randint(sizes[t], (1,), generator=pick))]
        injections[str(step)] = {"tensor": t, "elements": idx, "value": value}
    ref = TorchAmpStep(shapes, init, lr=tc.lr, betas=(tc.beta1, tc.beta2), eps=tc.eps, weight_decay=tc.weight_decay,
                       grad_clip=amp["grad_clip"], loss_scale=amp["loss_scale"],
                       growth_interval=amp["growth_interval"], use_scaler=True, accurate_norm=True)
    stream = GradStream(shapes, seed=1)
    traj = {"scale_after": [], "found_inf": [], "adam_t": [], "norm": [], "growth_tracker": []}
    for step in range(amp["steps"]):
        grads = stream.next_fp16_scaled(ref.loss_scale())
        inj = injections.get(str(step))
        if inj:
            inject(grads, inj["tensor"], inj["elements"], float(inj["value"]))
        ref.set_grads(grads)
        before = ref.adam_steps()
        ref.step()
        traj["scale_after"].append(ref.loss_scale())
        traj["found_inf"].append(0 if ref.adam_steps() > before else 1)
        traj["adam_t"].append(ref.adam_steps())
        traj["norm"].append(ref.last_norm if np.isfinite(ref.last_norm) else None)
        traj["growth_tracker"].append(int(ref.scaler._growth_tracker.item()))
    p_flat, m_flat, v_flat = ref.flat("p"), ref.flat("m"), ref.flat("v")
    np.savez_compressed(os.path.join(HERE, "debug_amp_100steps.npz"),
                        p=p_flat[::STRIDE].numpy(), m=m_flat[::STRIDE].numpy(), v=v_flat[::STRIDE].numpy(),
                        p_sums=per_tensor_sums(p_flat, sizes), m_sums=per_tensor_sums(m_flat, sizes),
                        v_sums=per_tensor_sums(v_flat, sizes),
                        w16=p_flat[::STRIDE].half().numpy().view(np.uint16))
    meta["amp"] = dict(amp, injections=injections, trajectory=traj)

    # ---------------------------------------------------------------- the reference's answer key: step1.* records
    rng = np.random.default_rng(0)
    tokens = rng.integers(0, 4100, size=100_000).astype(np.uint16)      # reference/test_reference.py:31,40-45
    tokens = np.minimum(tokens, 4097).astype(np.uint16)                 # ids must be < vocab_size 4098
    header, records = ref_dump.build_records(cfg, tc, tokens, DUMP_BATCH, "cpu", perturb=True)
    torch.use_deterministic_algorithms(False)
    keep_rows = {"wte": 128}    # the embedding table is cut to its first rows to keep the file small
    dump = {"grad_norm": records["grad_norm"].numpy().reshape(1)}
    dump_names = []
    for name in names:
        p, g, s1 = records[name], records["grad." + name], records["step1." + name]
        if name in keep_rows:
            r = keep_rows[name]
            p, g, s1 = p[:r], g[:r], s1[:r]
        dump_names.append(name)
        dump["param." + name] = p.numpy().reshape(-1)
        dump["grad." + name] = g.numpy().reshape(-1)
        dump["step1." + name] = s1.numpy().reshape(-1)
    np.savez_compressed(os.path.join(HERE, "dump_step1.npz"), **dump)
    meta["dump"] = {"names": dump_names, "lr": header["lr"], "beta1": header["beta1"], "beta2": header["beta2"],
                    "eps": header["eps"], "weight_decay": header["weight_decay"],
                    "ndim": {n: len(records[n].shape) for n in names}}

    with open(os.path.join(HERE, "golden_meta.json"), "w") as f:
        json.dump(meta, f, indent=1)
    for fn in sorted(os.listdir(HERE)):
        print(f"{os.path.getsize(os.path.join(HERE, fn)):>10d}  {fn}")


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("B200AMP_REFERENCE_DIR"):
        sys.exit("usage: make_golden.py /path/to/cuda-transformer   (or set B200AMP_REFERENCE_DIR)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["B200AMP_REFERENCE_DIR"])
