"""Pins the CPU oracle (oracle/ref_step.c) against golden vectors produced by the
reference's own PyTorch path (tests/golden/make_golden.py). CPU only."""
import math

import numpy as np
import pytest
import torch

import helpers as H
from inputs import GradStream, inject
from oracle import ref_step as O


def test_struct_sizes_match_reference_abi():
    lib = O.load()
    assert lib.oracle_sizeof_state() == 60          # cuda/kernels/fast.h:104-121, 15 x 4 bytes
    assert lib.oracle_sizeof_schedule() == 44       # cuda/kernels/fast.h:123-133
    assert lib.oracle_sizeof_tensor_info() == 24    # cuda/kernels/fast.h:153-158


def test_half_to_float_every_bit_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.empty(65536, dtype=np.float32)
    O.load().oracle_unscale_f16(O._p(bits), 65536, 1.0, O._p(got))
    finite = np.isfinite(want)
    assert np.array_equal(want[finite].view(np.uint32), got[finite].view(np.uint32))
    assert np.array_equal(np.isnan(want), np.isnan(got))
    assert np.array_equal(np.isinf(want), np.isinf(got))


def test_float_to_half_round_to_nearest_even():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(200_000).astype(np.float32) * np.float32(0.02),
        rng.standard_normal(100_000).astype(np.float32) * np.float32(1e-6),       # subnormal halves
        rng.standard_normal(100_000).astype(np.float32) * np.float32(3e4),        # near overflow
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                  2.0 ** -14, 2.0 ** -14 * 0.9999, np.inf, -np.inf, 1.0009765625 + 2.0 ** -11], dtype=np.float32),
        np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)[:0x7C00],
    ])
    with np.errstate(over="ignore"):                    # values beyond 65504 are meant to become inf
        want = x.astype(np.float16).view(np.uint16)
    got = O.float_to_half(x)
    assert np.array_equal(want, got)
    assert O.float_to_half(np.array([np.nan], dtype=np.float32))[0] & 0x7C00 == 0x7C00


@pytest.mark.parametrize("kind", ["cosine", "wsd"])
def test_lr_schedule_matches_host_formula(kind):
    """Same numbers as lr_at() (reference/train.py:79-96); the reference's own bar is 1e-12
    (cuda/tests/test_checkpoint.cu:355-437)."""
    decay_steps = 40 if kind == "wsd" else 0
    cfg = O.make_schedule(lr=6e-4, min_lr=6e-5, warmup_steps=20, max_steps=200, decay_steps=decay_steps)
    lr, min_lr = float(np.float32(6e-4)), float(np.float32(6e-5))

    def lr_at(step):
        if step < 20:
            return lr * (step + 1) / 20
        if step >= 200:
            return min_lr
        if decay_steps > 0:
            start = 200 - decay_steps
            if step < start:
                return lr
            p = (step - start) / decay_steps
            return min_lr + (lr - min_lr) * (1.0 - math.sqrt(p))
        progress = (step - 20) / max(1, 200 - 20)
        return min_lr + 0.5 * (1.0 + math.cos(math.pi * progress)) * (lr - min_lr)

    for step in list(range(0, 230)):
        assert abs(O.lr_at(step, cfg) - lr_at(step)) <= 1e-12


def test_adamw_step1_matches_reference_dump_records():
    """The reference's own AdamW check (cuda/tests/test_kernels.cu:413-467, test_fast.cu:241-254):
    params + grad.* -> step1.* after one un-clipped step at lr 6e-4."""
    meta = H.golden_meta()["dump"]
    d = H.golden("dump_step1.npz")
    for contract in (0, 1):
        worst = 0.0
        for name in meta["names"]:
            p0, g, want = d["param." + name], d["grad." + name], d["step1." + name]
            decay = 1 if meta["ndim"][name] >= 2 else 0
            cfg = O.make_schedule(lr=meta["lr"], min_lr=meta["lr"], beta1=meta["beta1"], beta2=meta["beta2"],
                                  weight_decay=meta["weight_decay"], grad_clip=1e30)
            step = O.OracleStep(p0, [(0, p0.size, decay)], cfg, eps=meta["eps"], loss_scale=1.0, contract=contract)
            step.step_f32(g)
            assert step.state.adam_t == 1 and step.state.found_inf == 0 and step.state.clip_coef == 1.0
            if name.endswith("attn.c_attn.b"):
                # the key-bias slice has a true gradient of 0: its update is rounding noise / (noise + eps)
                # and differs between machines (reference/dump.py:54-65); the reference compares it at 1e-6 abs
                assert np.abs(step.master - want).max() <= 2e-6
                continue
            worst = max(worst, H.rel_err(want, step.master))
        assert worst <= H.STATE_TOL, worst


def test_grad_norm_of_dump_grads():
    """grad_norm record = sqrt(sum of squares in fp64) (reference/dump.py:144-145)."""
    d = H.golden("dump_step1.npz")
    meta = H.golden_meta()["dump"]
    g = np.concatenate([d["grad." + n] for n in meta["names"]])
    pad = (-g.size) % 4
    g = np.concatenate([g, np.zeros(pad, dtype=np.float32)])
    st = O.initial_state(1.0)
    partial = np.zeros(512, dtype=np.float32)
    O.load().oracle_unscale_and_norm_f32(O._p(g.copy()), g.size, st, O._p(partial), 1)
    got = math.sqrt(O.load().oracle_tree_sum(O._p(partial)))
    # the fixture holds only the first 128 rows of wte, so compare with the fp64 norm of what is there
    want = math.sqrt(float((g.astype(np.float64) ** 2).sum()))
    assert abs(got - want) <= 1e-6 * want


@pytest.mark.parametrize("contract", [0, 1])
def test_fp32_path_10_steps_matches_reference_optimizer(contract):
    """Debug model, the model's own AdamW groups, fp32 gradients, clip 1.0 (inactive: norm 0.61)."""
    meta = H.golden_meta()
    gold = H.golden("debug_fp32_10steps.npz")
    slots = H.debug_slots()
    assert [s.name for s in slots] == meta["names"]
    assert [list(s.shape) for s in slots] == meta["shapes"]
    cfg = O.make_schedule(lr=meta["lr"], min_lr=meta["lr"], beta1=meta["beta1"], beta2=meta["beta2"],
                          weight_decay=meta["weight_decay"], grad_clip=meta["grad_clip"], dynamic_scale=0)
    step = O.OracleStep(H.debug_init(), H.table_of(slots), cfg, eps=meta["eps"], loss_scale=1.0, contract=contract)
    stream = GradStream(H.debug_shapes(), seed=1)
    stride = meta["stride"]
    sizes = [s.count for s in slots]
    for k in range(10):
        grads = stream.next_fp32()
        flat = H.flat_np(grads)
        if k == 0:
            assert abs(float(flat.astype(np.float64).sum()) - float(gold["first_grad_sum"][0])) < 1e-9, \
                "torch's CPU generator gives a different stream than when the fixture was made"
        step.step_f32(flat)
        assert abs(step.state.grad_norm - gold["norms"][k]) <= 1e-5 * gold["norms"][k]
        assert step.state.clip_coef == 1.0
        if k in (0, 9):
            tag = f"step{k + 1}"
            for what, arr in (("p", step.master), ("m", step.m), ("v", step.v)):
                assert H.rel_err(gold[f"{tag}_{what}"], arr[::stride]) <= H.STATE_TOL, (tag, what)
                at = 0
                sums = []
                for n in sizes:
                    sums.append(arr[at:at + n].astype(np.float64).sum())
                    at += n
                want = gold[f"{tag}_{what}_sums"]
                assert np.abs(np.array(sums) - want).max() <= 1e-6 * max(1e-30, np.abs(want).max())
    assert step.state.step == 10 and step.state.adam_t == 10 and step.state.skipped == 0


@pytest.mark.parametrize("contract", [0, 1])
def test_amp_path_100_steps_trajectory_and_state(contract):
    """GradScaler semantics: inf at steps 3, 17, 40, NaN at 55, growth every 8 clean steps.
    Skip decisions, loss scale, adam_t and the growth counter are bit-exact; p/m/v to 1e-6."""
    meta = H.golden_meta()
    amp = meta["amp"]
    gold = H.golden("debug_amp_100steps.npz")
    slots = H.debug_slots()
    cfg = O.make_schedule(lr=meta["lr"], min_lr=meta["lr"], beta1=meta["beta1"], beta2=meta["beta2"],
                          weight_decay=meta["weight_decay"], grad_clip=amp["grad_clip"],
                          growth_interval=amp["growth_interval"], dynamic_scale=1)
    step = O.OracleStep(H.debug_init(), H.table_of(slots), cfg, eps=meta["eps"], loss_scale=amp["loss_scale"],
                        contract=contract)
    stream = GradStream(H.debug_shapes(), seed=1)
    traj = amp["trajectory"]
    for k in range(amp["steps"]):
        grads = stream.next_fp16_scaled(step.state.loss_scale)
        inj = amp["injections"].get(str(k))
        if inj:
            inject(grads, inj["tensor"], inj["elements"], float(inj["value"]))
        g16 = H.f16_bits(torch.cat([g.reshape(-1) for g in grads]))
        before = (step.master.copy(), step.m.copy(), step.v.copy(), step.weights16.copy())
        step.step_f16(g16)
        assert step.state.loss_scale == traj["scale_after"][k], k
        assert step.state.found_inf == traj["found_inf"][k], k
        assert step.state.adam_t == traj["adam_t"][k], k
        assert step.state.good_steps == traj["growth_tracker"][k], k
        assert step.state.step == k + 1
        if traj["found_inf"][k]:
            after = (step.master, step.m, step.v, step.weights16)
            assert all(np.array_equal(a, b) for a, b in zip(before, after)), "a skipped step moved state"
        else:
            assert abs(step.state.grad_norm - traj["norm"][k]) <= 1e-6 * traj["norm"][k]
    assert step.state.skipped == 4
    stride = meta["stride"]
    for what, arr in (("p", step.master), ("m", step.m), ("v", step.v)):
        assert H.rel_err(gold[what], arr[::stride]) <= H.STATE_TOL, what
    assert H.half_ulp_distance(gold["w16"], step.weights16[::stride]) <= 1


def test_zero_rows_with_zero_gradient_stay_zero():
    """The optimizer half of padded_rows (reference/test_reference.py:113-116): vocabulary padding
    rows start at 0, get no gradient, and an optimizer step with weight decay must leave them at
    +0.0 exactly (and their m, v, fp16 copy too)."""
    n = 8 * 256
    rng = np.random.default_rng(4)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    pad = slice(8 * 100, 8 * 140)                       # rows of a decayed 2-D tensor that are padding
    init[pad] = 0.0
    table = [(0, 8 * 200, 1), (8 * 200, n - 8 * 200, 0)]
    ora = O.OracleStep(init, table, O.make_schedule(), loss_scale=65536.0)
    for k in range(5):
        g = (rng.standard_normal(n) * 1e-3 * ora.state.loss_scale).astype(np.float16)
        g[pad] = 0.0
        ora.step_f16(g.view(np.uint16))
    for arr in (ora.master, ora.m, ora.v):
        assert np.all(arr[pad].view(np.uint32) == 0), "a padded row moved (or turned into -0.0)"
    assert np.all(ora.weights16[pad] == 0)
    assert np.all(ora.master[:8 * 100] != init[:8 * 100])      # the rest did move
