"""Config 4 at its full size (1,315,819,520 parameters, 292 tensors, 23.7 GB resident) through
size-independent properties, plus spot checks of random slices against the oracle.

The oracle cannot step 1.3 B elements in test time, so the whole-arena claims are properties
that hold for any correct step: the fp16 copy is exactly fp16(master) everywhere; the norm
equals an independent fp64 reduction; a skipped step leaves every byte of state alone; the
8-way range form gives the bits of the whole-arena launch. Element arithmetic is then checked
against the oracle on 48 random 8,192-element windows (windows that straddle tensor edges
included), with the GPU's own step scalars."""
import ctypes as C

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def _fill(t, std, seed):
    gen = torch.Generator(device=t.device).manual_seed(seed)
    chunk = 1 << 27
    for at in range(0, t.numel(), chunk):
        sl = t[at:at + chunk]
        sl.copy_((torch.randn(sl.numel(), generator=gen, device=t.device, dtype=torch.float32) * std).to(t.dtype))


def test_config4_full_size_properties_and_spot_checks():
    from cuda_transformer_b200 import amp
    from cuda_transformer_b200.layout import CONFIGS, param_layout
    from oracle import ref_step as O
    free, _ = torch.cuda.mem_get_info()
    if free < 60 * (1 << 30):
        pytest.skip("needs about 60 GB of free device memory")
    slots = param_layout(CONFIGS["1.3b"])
    cfg = amp.make_schedule()
    opt = amp.AmpOptimizer(slots, cfg, loss_scale=32768.0, history_len=8)
    n = opt.n
    assert n == 1_315_819_520 and opt.ntensors == 292
    _fill(opt.master, 0.02, 0)
    amp.cast_to_x(opt.weights16, opt.master, n)
    for k in range(2):                                  # warm m and v
        _fill(opt.grads16, 1e-3 * 32768.0, 10 + k)
        opt.optimizer_step()
    _fill(opt.grads16, 1e-3 * 32768.0, 1)
    torch.cuda.synchronize()

    # windows to check against the oracle: random ones + one across every 40th tensor edge
    rng = np.random.default_rng(0)
    W = 8192
    starts = [int(x) * 8 for x in rng.integers(0, (n - W) // 8, size=40)]
    starts += [max(0, slots[i].offset - W // 2) // 8 * 8 for i in range(1, len(slots), 40)]
    before = {s: [t[s:s + W].cpu().numpy().copy() for t in (opt.master, opt.m, opt.v)] for s in starts}
    grads = {s: H.f16_bits(opt.grads16[s:s + W].cpu()) for s in starts}

    opt.optimizer_step()
    torch.cuda.synchronize()
    st = opt.read_state()
    assert st.found_inf == 0 and st.adam_t == 3 and st.step == 3

    # (1) fp16 copy == fp16(master), everywhere
    chunk = 1 << 27
    for at in range(0, n, chunk):
        assert torch.equal(opt.master[at:at + chunk].half(), opt.weights16[at:at + chunk])
    # (2) the norm against an independent fp64 reduction
    sumsq = 0.0
    for at in range(0, n, chunk):
        g = opt.grads16[at:at + chunk].double() / 32768.0
        sumsq += float((g * g).sum())
    assert abs(st.grad_norm - sumsq ** 0.5) <= 1e-6 * sumsq ** 0.5
    assert abs(st.clip_coef - 1.0 / (sumsq ** 0.5 + 1e-6)) <= 1e-6 * st.clip_coef
    # (3) spot checks against the oracle with the GPU's scalars
    table = H.table_of(slots)
    worst = 0.0
    for s in starts:
        p0, m0, v0 = before[s]
        o = O.OracleStep(p0, table, O.make_schedule(), loss_scale=32768.0, arena_offset=s)
        o.m, o.v = m0.copy(), v0.copy()
        o.state = O.StepState.from_buffer_copy(bytes(st))
        o.pass2_f16(grads[s])
        for want, got in ((o.master, opt.master), (o.m, opt.m), (o.v, opt.v)):
            worst = max(worst, H.rel_err(want, got[s:s + W].cpu().numpy()))
        assert H.half_ulp_distance(o.weights16, H.f16_bits(opt.weights16[s:s + W].cpu())) <= 1
    assert worst <= H.STATE_TOL, worst

    # (4) the 8-way range form on the same inputs gives the bits of the whole-arena launch
    snap = [t.clone() for t in (opt.master, opt.m, opt.v, opt.weights16)]
    state_before = opt.state.clone()
    opt.optimizer_step()                                # whole arena, step 4
    whole = [t.clone() for t in (opt.master, opt.m, opt.v, opt.weights16)]
    whole_state = bytes(opt.read_state())
    for dst, src in zip((opt.master, opt.m, opt.v, opt.weights16), snap):
        dst.copy_(src)
    opt.state.copy_(state_before)
    del snap
    world, per = 8, n // 8
    ws = [torch.zeros_like(opt.workspace) for _ in range(world)]
    pairs = torch.zeros(2 * world, dtype=torch.float64, device="cuda")
    for r in range(world):
        amp.pass1_f16(opt.grads16[r * per:(r + 1) * per], per, opt.state, ws[r])
        pairs[2 * r:2 * r + 2] = ws[r][:16].view(torch.float64)
    amp.finalize_sums(opt.state, pairs, world, cfg, opt.history, opt.history_len)
    for r in range(world):
        sl = slice(r * per, (r + 1) * per)
        amp.pass2_f16(opt.master[sl], opt.m[sl], opt.v[sl], opt.grads16[sl], opt.weights16[sl], per, r * per,
                      opt.tensors, opt.ntensors, opt.state, cfg.beta1, cfg.beta2, opt.eps)
    torch.cuda.synchronize()
    a = opt.read_state()
    b = type(a).from_buffer_copy(whole_state)
    assert (a.step, a.adam_t, a.skipped, a.loss_scale) == (b.step, b.adam_t, b.skipped, b.loss_scale)
    assert abs(a.grad_norm - b.grad_norm) <= 1e-6 * b.grad_norm
    if a.clip_coef == b.clip_coef:
        for x, y in zip((opt.master, opt.m, opt.v, opt.weights16), whole):
            assert torch.equal(x, y)
    del whole

    # (5) a skipped step: one inf among 1.3 G gradients, nothing else moves
    sums_before = [float(t.double().sum()) for t in (opt.master, opt.m, opt.v)]
    keep = opt.weights16.clone()
    opt.grads16[n - 3] = float("inf")
    opt.optimizer_step()
    torch.cuda.synchronize()
    st = opt.read_state()
    assert st.found_inf == 1 and st.skipped == 1 and st.loss_scale == 16384.0 and st.adam_t == a.adam_t
    assert [float(t.double().sum()) for t in (opt.master, opt.m, opt.v)] == sums_before
    assert torch.equal(keep, opt.weights16)
