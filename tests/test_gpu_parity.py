"""Parity of the CUDA path with the oracle, the golden vectors and (when built) the
reference's own CUDA kernels. Every call goes through the C ABI of libb200amp.so."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import helpers as H
from inputs import GradStream, inject

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import gpu_helpers
    from cuda_transformer_b200 import _lib
    _lib.check(_lib.load().b200amp_device_check())
    return gpu_helpers


@pytest.fixture(scope="module")
def O():
    from oracle import ref_step
    ref_step.load()
    return ref_step


def sched(amp_or_oracle, **kw):
    return amp_or_oracle.make_schedule(**kw)


def compare_arrays(gpu, oracle, tol=H.STATE_TOL):
    gm, gmm, gv, gw = gpu.host()
    assert H.rel_err(oracle.master, gm) <= tol
    assert H.rel_err(oracle.m, gmm) <= tol
    assert H.rel_err(oracle.v, gv) <= tol
    assert H.half_ulp_distance(oracle.weights16, gw) <= 1
    # the fp16 copy is exactly fp16(master) (cuda/tests/test_fast.cu:255-267)
    assert np.array_equal(gm.astype(np.float16).view(np.uint16), gw)


# ---------------------------------------------------------------- debug model (config 0 sizes)

def test_compat_fp32_10_steps_match_reference_optimizer(G, O):
    """Config 0: the reference's entry points, fp32 gradients, against the golden vectors the
    reference's PyTorch path produced and against the oracle."""
    from cuda_transformer_b200 import amp
    meta = H.golden_meta()
    gold = H.golden("debug_fp32_10steps.npz")
    slots = H.debug_slots()
    kw = dict(lr=meta["lr"], min_lr=meta["lr"], beta1=meta["beta1"], beta2=meta["beta2"],
              weight_decay=meta["weight_decay"], grad_clip=meta["grad_clip"], dynamic_scale=0)
    table = H.table_of(slots)
    gpu = G.GpuStep(H.debug_init(), table, sched(amp, **kw), eps=meta["eps"], loss_scale=1.0)
    ora = O.OracleStep(H.debug_init(), table, sched(O, **kw), eps=meta["eps"], loss_scale=1.0, contract=1)
    stream = GradStream(H.debug_shapes(), seed=1)
    stride = meta["stride"]
    for k in range(10):
        flat = H.flat_np(stream.next_fp32())
        g_dev = gpu.step_f32(flat)
        g_ora = ora.step_f32(flat)
        assert np.array_equal(g_dev.cpu().numpy(), g_ora), "in-place unscale differs"
        st = gpu.read_state()
        G.assert_states_equal(st, ora.state)
        assert abs(st.grad_norm - gold["norms"][k]) <= 1e-5 * gold["norms"][k]
        if k in (0, 9):
            gm, gmm, gv, _ = gpu.host()
            tag = f"step{k + 1}"
            for what, arr in (("p", gm), ("m", gmm), ("v", gv)):
                assert H.rel_err(gold[f"{tag}_{what}"], arr[::stride]) <= H.STATE_TOL, (tag, what)
    compare_arrays(gpu, ora)
    st = gpu.read_state()
    assert st.step == 10 and st.adam_t == 10 and st.skipped == 0 and st.loss_scale == 1.0


def test_native_amp_100_steps_trajectory_matches_reference_scaler(G, O):
    """fp16 gradient arena, inf at steps 3/17/40, NaN at 55, growth every 8 clean steps: skip
    decisions, loss scale, adam_t and the growth counter bit-exact against torch's GradScaler
    (golden), state arrays against golden and oracle."""
    from cuda_transformer_b200 import amp
    meta = H.golden_meta()
    a = meta["amp"]
    gold = H.golden("debug_amp_100steps.npz")
    slots = H.debug_slots()
    kw = dict(lr=meta["lr"], min_lr=meta["lr"], beta1=meta["beta1"], beta2=meta["beta2"],
              weight_decay=meta["weight_decay"], grad_clip=a["grad_clip"], growth_interval=a["growth_interval"],
              dynamic_scale=1)
    n = slots[-1].offset + slots[-1].count
    n_pad = (n + 7) // 8 * 8
    table = H.table_of(slots)
    init = np.zeros(n_pad, dtype=np.float32)
    init[:n] = H.debug_init()
    gpu = G.GpuStep(init, table, sched(amp, **kw), eps=meta["eps"], loss_scale=a["loss_scale"])
    ora = O.OracleStep(init, table, sched(O, **kw), eps=meta["eps"], loss_scale=a["loss_scale"], contract=1)
    stream = GradStream(H.debug_shapes(), seed=1)
    traj = a["trajectory"]
    for k in range(a["steps"]):
        scale = gpu.read_state().loss_scale
        grads = stream.next_fp16_scaled(scale)
        inj = a["injections"].get(str(k))
        if inj:
            inject(grads, inj["tensor"], inj["elements"], float(inj["value"]))
        bits = np.zeros(n_pad, dtype=np.uint16)
        bits[:n] = H.f16_bits(torch.cat([g.reshape(-1) for g in grads]))
        before = gpu.host() if traj["found_inf"][k] else None
        gpu.set_grads16(bits)
        gpu.step_f16()
        ora.step_f16(bits)
        st = gpu.read_state()
        assert st.loss_scale == traj["scale_after"][k], k
        assert st.found_inf == traj["found_inf"][k], k
        assert st.adam_t == traj["adam_t"][k], k
        assert st.good_steps == traj["growth_tracker"][k], k
        assert st.step == k + 1
        G.assert_states_equal(st, ora.state)
        if before is not None:
            after = gpu.host()
            assert all(np.array_equal(x, y) for x, y in zip(before, after)), "a skipped step moved state"
        else:
            assert abs(st.grad_norm - traj["norm"][k]) <= 1e-6 * traj["norm"][k]
    assert gpu.read_state().skipped == 4
    compare_arrays(gpu, ora)
    gm, gmm, gv, gw = gpu.host()
    stride = meta["stride"]
    for what, arr in (("p", gm[:n]), ("m", gmm[:n]), ("v", gv[:n])):
        assert H.rel_err(gold[what], arr[::stride]) <= H.STATE_TOL, what
    assert H.half_ulp_distance(gold["w16"], gw[:n][::stride]) <= 1
    # the history ring holds every finished step (cuda/kernels/scaler.cu:165-168)
    for k in (0, 3, 55, 99):
        h = G.read_struct(gpu.history, k)
        assert h.step == k and h.found_inf == traj["found_inf"][k]


# ---------------------------------------------------------------- README model (configs 1 and 2)

def _readme_run(G, O, steps, injections, growth_interval, check_every):
    from cuda_transformer_b200 import amp
    from cuda_transformer_b200.layout import CONFIGS, param_layout
    slots = param_layout(CONFIGS["readme"])
    n = slots[-1].offset + slots[-1].count
    assert n == 12_343_296
    shapes = [s.shape for s in slots]
    table = H.table_of(slots)
    gen = torch.Generator().manual_seed(0)
    init = (torch.randn(n, generator=gen) * 0.02).numpy()
    kw = dict(lr=6e-4, min_lr=6e-4, beta1=0.9, beta2=0.95, weight_decay=0.1, grad_clip=1.0,
              growth_interval=growth_interval, dynamic_scale=1)
    gpu = G.GpuStep(init, table, sched(amp, **kw), loss_scale=65536.0)
    ora = O.OracleStep(init, table, sched(O, **kw), loss_scale=65536.0, contract=1)
    stream = GradStream(shapes, seed=1)
    scales = []
    for k in range(steps):
        grads = stream.next_fp16_scaled(ora.state.loss_scale)
        if k in injections:
            t, idx, val = injections[k]
            inject(grads, t, idx, val)
        bits = H.f16_bits(torch.cat([g.reshape(-1) for g in grads]))
        gpu.set_grads16(bits)
        gpu.step_f16()
        ora.step_f16(bits)
        st = gpu.read_state()
        G.assert_states_equal(st, ora.state)
        scales.append(st.loss_scale)
        if (k + 1) % check_every == 0 or k in injections:
            compare_arrays(gpu, ora)
    compare_arrays(gpu, ora)
    return gpu.read_state(), scales, ora


def test_readme_model_amp_steps_match_oracle(G, O):
    """Config 1 (12.3 M parameters, 76 tensors, clip active: norm 3.5 -> coef 0.285), with growth
    every 8 steps so the scale moves too."""
    st, scales, ora = _readme_run(G, O, steps=24, injections={}, growth_interval=8, check_every=8)
    assert st.adam_t == 24 and st.skipped == 0
    assert scales[7] == 131072.0 and scales[15] == 262144.0 and scales[23] == 524288.0
    assert 0.28 < ora.state.clip_coef < 0.29


def test_readme_model_overflow_trajectory(G, O):
    """Config 2: +inf into 0.1 % of one tensor at steps 3, 17, 40 and one NaN at step 55; 100 steps."""
    from cuda_transformer_b200.layout import CONFIGS, param_layout
    slots = param_layout(CONFIGS["readme"])
    pick = torch.Generator().manual_seed(2)
    injections = {}
    for step, val in ((3, float("inf")), (17, float("inf")), (40, float("inf")), (55, float("nan"))):
        t = int(torch.randint(len(slots), (1,), generator=pick))
        if math.isinf(val):
            k = max(1, slots[t].count // 1000)
            idx = torch.randperm(slots[t].count, generator=pick)[:k].tolist()
        else:
            idx = [int(torch.randint(slots[t].count, (1,), generator=pick))]
        injections[step] = (t, idx, val)
    st, scales, _ = _readme_run(G, O, steps=100, injections=injections, growth_interval=2000, check_every=50)
    assert st.skipped == 4 and st.adam_t == 96 and st.step == 100
    expect = 65536.0
    for k in range(100):
        if k in injections:
            expect *= 0.5
        assert scales[k] == expect, k
    assert scales[-1] == 4096.0


# ---------------------------------------------------------------- edge cases

@pytest.mark.parametrize("n", [8, 64, 2048, 8192 + 8, (1 << 20) + 24])
def test_small_and_ragged_sizes(G, O, n):
    from cuda_transformer_b200 import amp
    rng = np.random.default_rng(n)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    table = [(0, n, 1)]
    kw = dict(grad_clip=1.0)
    gpu = G.GpuStep(init, table, sched(amp, **kw), loss_scale=1024.0)
    ora = O.OracleStep(init, table, sched(O, **kw), loss_scale=1024.0)
    for _ in range(3):
        bits = (rng.standard_normal(n) * 1e-2 * 1024.0).astype(np.float16).view(np.uint16)
        gpu.set_grads16(bits)
        gpu.step_f16()
        ora.step_f16(bits)
        G.assert_states_equal(gpu.read_state(), ora.state)
    compare_arrays(gpu, ora)


def test_1024_tensors_and_boundaries_inside_a_group(G, O):
    """The longest table the ABI allows; tensor edges at multiples of 4 that are not multiples of
    8, so a decayed and an undecayed tensor share one 8-element group."""
    from cuda_transformer_b200 import amp
    rng = np.random.default_rng(7)
    counts = rng.choice([4, 12, 20, 36, 260, 1028], size=1024)
    table, at = [], 0
    for i, c in enumerate(counts):
        table.append((at, int(c), int(i % 2)))
        at += int(c)
    n = (at + 7) // 8 * 8
    init = (rng.standard_normal(n) * 0.5).astype(np.float32)
    kw = dict(weight_decay=0.5, lr=1e-2, min_lr=1e-2)       # a decay large enough that a wrong flag shows
    gpu = G.GpuStep(init, table, sched(amp, **kw), loss_scale=256.0)
    ora = O.OracleStep(init, table, sched(O, **kw), loss_scale=256.0)
    for _ in range(2):
        bits = (rng.standard_normal(n) * 1e-3 * 256.0).astype(np.float16).view(np.uint16)
        gpu.set_grads16(bits)
        gpu.step_f16()
        ora.step_f16(bits)
    compare_arrays(gpu, ora)
    # and the compat kernel, whose granularity is 4
    gpu2 = G.GpuStep(init, table, sched(amp, **kw), loss_scale=256.0)
    ora2 = O.OracleStep(init, table, sched(O, **kw), loss_scale=256.0)
    g = (rng.standard_normal(n) * 1e-3 * 256.0).astype(np.float32)
    gpu2.step_f32(g)
    ora2.step_f32(g)
    compare_arrays(gpu2, ora2)


@pytest.mark.parametrize("world", [1, 4])
def test_decay_runs_as_a_kernel_parameter_give_the_bits_of_the_table_in_memory(G, world):
    """b200amp_pass2_f16_runs against b200amp_pass2_f16: 400 tensors that merge into 256 runs (the
    most the parameter form takes), edges at multiples of 4 inside 8-element groups, gaps between
    tensors, whole arena and 4 shards addressed by their offsets; and a table of 258 runs is
    refused by the builder, not truncated."""
    from cuda_transformer_b200 import _lib, amp
    rng = np.random.default_rng(11)
    counts = rng.choice([4, 12, 20, 36, 260, 1028, 5000], size=400)
    flags = []
    for i in range(400):                                # the flag changes at two tensors out of three
        flags.append((flags[-1] ^ 1) if i and i % 3 != 0 else (flags[-1] if i else 1))
    changes = sum(1 for a, b in zip(flags, flags[1:]) if a != b)
    for i in range(len(flags) - 1, 0, -1):              # 266 changes: undo the last ones until 255 are left (256 runs)
        if changes <= 255:
            break
        if flags[i] != flags[i - 1]:
            for j in range(i, len(flags)):
                flags[j] ^= 1
            changes -= 1
    table, at = [], 0
    for i, c in enumerate(counts):
        table.append((at, int(c), int(flags[i])))
        at += int(c) + (8 if i % 50 == 49 else 0)       # a gap now and then: it belongs to the run before it
    runs = amp.decay_runs_build(table)
    assert runs.nruns == 256
    n = (at + 8 * world - 1) // (8 * world) * (8 * world)
    init = (rng.standard_normal(n) * 0.5).astype(np.float32)
    kw = dict(weight_decay=0.5, lr=1e-2, min_lr=1e-2)
    a = G.GpuStep(init, table, sched(amp, **kw), loss_scale=256.0)
    b = G.GpuStep(init, table, sched(amp, **kw), loss_scale=256.0)
    per = n // world
    for _ in range(2):
        bits = (rng.standard_normal(n) * 1e-3 * 256.0).astype(np.float16).view(np.uint16)
        for g in (a, b):
            g.set_grads16(bits)
            amp.pass1_finalize_f16(g.grads16, n, g.state, g.workspace, g.cfg, g.history, g.history_len)
        for r in range(world):
            sl = slice(r * per, (r + 1) * per)
            amp.pass2_f16(a.master[sl], a.m[sl], a.v[sl], a.grads16[sl], a.weights16[sl], per, r * per, a.tensors,
                          a.ntensors, a.state, a.cfg.beta1, a.cfg.beta2, a.eps)
            amp.pass2_f16_runs(b.master[sl], b.m[sl], b.v[sl], b.grads16[sl], b.weights16[sl], per, r * per, runs,
                               b.state, b.cfg.beta1, b.cfg.beta2, b.eps)
    for x, y in zip(a.host(), b.host()):
        assert np.array_equal(x, y)
    assert bytes(a.read_state()) == bytes(b.read_state())
    too_many = [(4 * i, 4, i % 2) for i in range(258)]
    with pytest.raises(amp.B200AmpError, match="runs") as err:
        amp.decay_runs_build(too_many)
    assert err.value.status == _lib.ERR_LIMIT


def test_zero_gradients_are_not_an_overflow(G, O):
    """An empty batch: grad_norm == 0.0 and the step is taken (cuda/tests/test_fast.cu:459-471)."""
    from cuda_transformer_b200 import amp
    n = 4096
    init = np.full(n, 0.25, dtype=np.float32)
    gpu = G.GpuStep(init, [(0, n, 1)], sched(amp), loss_scale=65536.0)
    gpu.set_grads16(np.zeros(n, dtype=np.uint16))
    gpu.step_f16()
    st = gpu.read_state()
    assert st.grad_norm == 0.0 and st.found_inf == 0 and st.skipped == 0 and st.adam_t == 1
    assert st.clip_coef == 1.0


def test_scaler_checks_of_the_reference(G, O):
    """The expectations of scaler_checks (cuda/tests/test_fast.cu:272-326): an inf gradient skips
    the step and halves S; the next step runs; growth_interval 2 doubles S back; S = 2^30 halves
    to 2^29; with dynamic_scale 0 the scale stays."""
    from cuda_transformer_b200 import amp
    n = 1 << 16
    rng = np.random.default_rng(3)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    cfg = sched(amp, growth_interval=2000)
    gpu = G.GpuStep(init, [(0, n, 1)], cfg, loss_scale=65536.0)
    before = gpu.host()
    bits = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16).view(np.uint16)
    bad = bits.copy()
    bad[12345 % n] = 0x7C00                                   # +inf
    gpu.set_grads16(bad)
    gpu.step_f16()
    st = gpu.read_state()
    assert st.found_inf == 1 and st.skipped == 1 and st.adam_t == 0 and st.step == 1
    assert st.loss_scale == 32768.0 and st.good_steps == 0
    after = gpu.host()
    assert all(np.array_equal(a, b) for a, b in zip(before, after))
    assert not after[1].any()                                 # m did not move
    gpu.set_grads16((rng.standard_normal(n) * 1e-3 * 32768.0).astype(np.float16).view(np.uint16))
    gpu.step_f16()
    st = gpu.read_state()
    assert st.found_inf == 0 and st.adam_t == 1 and st.step == 2 and st.skipped == 1
    assert not np.array_equal(gpu.host()[0], before[0])
    gpu.cfg.growth_interval = 2
    gpu.step_f16()
    st = gpu.read_state()
    assert st.loss_scale == 65536.0 and st.good_steps == 0
    big = G.GpuStep(init, [(0, n, 1)], cfg, loss_scale=float(2 ** 30))
    big.set_grads16(bad)
    big.step_f16()
    st = big.read_state()
    assert st.found_inf == 1 and st.skipped == 1 and st.loss_scale == float(2 ** 29)
    fixed = G.GpuStep(init, [(0, n, 1)], sched(amp, dynamic_scale=0), loss_scale=65536.0)
    fixed.set_grads16(bad)
    fixed.step_f16()
    assert fixed.read_state().loss_scale == 65536.0 and fixed.read_state().skipped == 1
    # negative infinity and NaN are found too, wherever they sit
    for pattern, where in ((0xFC00, 0), (0x7E00, n - 1), (0xFFFF, n // 2 + 3)):
        g = G.GpuStep(init, [(0, n, 1)], cfg, loss_scale=65536.0)
        b = bits.copy()
        b[where] = pattern
        g.set_grads16(b)
        g.step_f16()
        assert g.read_state().found_inf == 1, hex(pattern)
    # the largest finite fp16 is not an overflow
    g = G.GpuStep(init, [(0, n, 1)], cfg, loss_scale=65536.0)
    b = bits.copy()
    b[5] = 0x7BFF
    b[6] = 0xFBFF
    g.set_grads16(b)
    g.step_f16()
    assert g.read_state().found_inf == 0


def test_graph_replay_equals_eager(G):
    """graph_checks (cuda/tests/test_fast.cu:330-371): capturing runs nothing; 4 replays give the
    bits of 4 eager steps."""
    from cuda_transformer_b200 import amp
    n = 1 << 18
    rng = np.random.default_rng(11)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    bits = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16).view(np.uint16)
    table = [(0, n // 2, 1), (n // 2, n // 2, 0)]
    eager = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
    graphed = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
    eager.set_grads16(bits)
    graphed.set_grads16(bits)
    for _ in range(4):
        eager.step_f16()
    stream = torch.cuda.Stream()
    graph = amp.CudaGraph()
    assert not graph.ready()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        graph.capture(stream, lambda: graphed.step_f16())
    assert graph.ready()
    stream.synchronize()
    assert graphed.read_state().step == 0, "capturing must not run the step"
    for _ in range(4):
        graph.launch(stream)
    stream.synchronize()
    a, b = eager.read_state(), graphed.read_state()
    assert a.step == 4 and b.step == 4 and b.adam_t == 4
    assert bytes(a) == bytes(b)
    assert all(np.array_equal(x, y) for x, y in zip(eager.host(), graphed.host()))
    assert eager.history.cpu().numpy().tobytes() == graphed.history.cpu().numpy().tobytes()


def test_result_does_not_depend_on_launch_shape(G):
    from cuda_transformer_b200 import _lib, amp
    lib = _lib.load()
    n = (1 << 22) + 8 * 37
    rng = np.random.default_rng(5)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    bits = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16).view(np.uint16)
    table = [(0, 1000, 0), (1000, n - 1000, 1)]
    results = []
    base = dict(pass1_blocks_per_sm=8, pass2_blocks_per_sm=4, pass2_store_hint=0, pass2_threads=256,
                pass2_variant=0, pass2_stages=6)
    knobs = [base,
             dict(base, pass1_blocks_per_sm=1, pass2_blocks_per_sm=1, pass2_store_hint=1),
             dict(base, pass1_blocks_per_sm=3, pass2_blocks_per_sm=7),
             dict(base, pass2_threads=512, pass2_blocks_per_sm=1, pass2_store_hint=1),
             dict(base, pass2_threads=1024, pass2_blocks_per_sm=1),
             dict(base, pass2_variant=1, pass2_stages=6),
             dict(base, pass2_variant=1, pass2_stages=3)]
    defaults = {}
    for key in knobs[0]:
        v = C.c_int()
        _lib.check(lib.b200amp_tune_get(key.encode(), C.byref(v)))
        defaults[key] = v.value
    try:
        for kn in knobs:
            for key, val in kn.items():
                _lib.check(lib.b200amp_tune_set(key.encode(), val))
            g = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
            g.set_grads16(bits)
            g.step_f16()
            g.step_f16()
            results.append((bytes(g.read_state()), g.host()))
    finally:
        for key, val in defaults.items():
            lib.b200amp_tune_set(key.encode(), val)
    different = []
    for idx, (st, arrays) in enumerate(results[1:], start=1):
        if st != results[0][0]:
            different.append((idx, "state"))
        for name, x, y in zip(("master", "m", "v", "weights16"), arrays, results[0][1]):
            if not np.array_equal(x, y):
                bad = np.flatnonzero(x != y)
                different.append((idx, name, int(bad.size), int(bad[0]), int(bad[-1])))
    assert not different, f"launch shapes (index into knobs) that changed the result: {different}"
    flag = C.c_int(-1)
    _lib.check(lib.b200amp_device_error(C.byref(flag)))
    assert flag.value == 0, "a staged launch gave up waiting for a bulk copy"


def test_sharded_passes_equal_the_whole_arena(G, O):
    """Pass 2 run as 8 ranges with their arena offsets gives the bits of one launch over the
    arena; pass 1 partial sums of the ranges, added in rank order, give the same state."""
    from cuda_transformer_b200 import amp
    n = 8 * 128 * 523
    rng = np.random.default_rng(9)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    bits = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16).view(np.uint16)
    edges = sorted(set([0] + [int(x) * 4 for x in rng.integers(1, n // 4, size=40)]))
    table = [(a, b - a, i % 2) for i, (a, b) in enumerate(zip(edges, edges[1:] + [n]))]
    whole = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
    whole.set_grads16(bits)
    whole.step_f16()
    parts = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
    parts.set_grads16(bits)
    world = 8
    per = n // world
    lib_ws = [torch.zeros_like(parts.workspace) for _ in range(world)]
    sums = torch.zeros(2 * world, dtype=torch.float64, device="cuda")
    for r in range(world):
        amp.pass1_f16(parts.grads16[r * per:(r + 1) * per], per, parts.state, lib_ws[r])
        sums[2 * r:2 * r + 2] = lib_ws[r][:16].view(torch.float64)
    amp.finalize_sums(parts.state, sums, world, parts.cfg, parts.history, parts.history_len)
    for r in range(world):
        sl = slice(r * per, (r + 1) * per)
        amp.pass2_f16(parts.master[sl], parts.m[sl], parts.v[sl], parts.grads16[sl], parts.weights16[sl], per,
                      r * per, parts.tensors, parts.ntensors, parts.state, parts.cfg.beta1, parts.cfg.beta2,
                      parts.eps)
    a, b = whole.read_state(), parts.read_state()
    G.assert_states_equal(b, a, tol=1e-6)
    if a.clip_coef == b.clip_coef:
        assert all(np.array_equal(x, y) for x, y in zip(whole.host(), parts.host()))
    else:
        for x, y in zip(whole.host()[:3], parts.host()[:3]):
            assert H.rel_err(x, y) <= H.STATE_TOL
    # an inf in one range only must skip every range
    bad = bits.copy()
    bad[5 * per + 17] = 0x7C00
    parts.set_grads16(bad)
    for r in range(world):
        amp.pass1_f16(parts.grads16[r * per:(r + 1) * per], per, parts.state, lib_ws[r])
        sums[2 * r:2 * r + 2] = lib_ws[r][:16].view(torch.float64)
    assert [float(sums[2 * r + 1]) for r in range(world)] == [0, 0, 0, 0, 0, 1, 0, 0]
    amp.finalize_sums(parts.state, sums, world, parts.cfg, parts.history, parts.history_len)
    assert parts.read_state().found_inf == 1 and parts.read_state().skipped == 1


@pytest.mark.parametrize("kind", ["cosine", "wsd"])
def test_lr_on_gpu_matches_host_schedule(G, O, kind):
    """GPU lr == host lr_at to 1e-12 (cuda/tests/test_checkpoint.cu:355-437)."""
    from cuda_transformer_b200 import amp
    decay_steps = 40 if kind == "wsd" else 0
    kw = dict(lr=6e-4, min_lr=6e-5, warmup_steps=20, max_steps=200, decay_steps=decay_steps)
    for step in (0, 1, 19, 20, 21, 100, 159, 160, 161, 199, 200, 5000):
        assert abs(amp.lr_on_gpu(step, sched(amp, **kw)) - O.lr_at(step, sched(O, **kw))) <= 1e-12


def test_bad_arguments_are_errors_not_crashes(G):
    from cuda_transformer_b200 import _lib, amp
    g = G.GpuStep(np.zeros(64, dtype=np.float32), [(0, 64, 1)], sched(amp))
    with pytest.raises(amp.B200AmpError) as e:
        amp.pass1_finalize_f16(g.grads16, 60, g.state, g.workspace, g.cfg)          # n % 8 != 0
    assert e.value.status == _lib.ERR_ARG and "multiple of 8" in str(e.value)
    with pytest.raises(amp.B200AmpError):
        amp.pass1_finalize_f16(g.grads16.data_ptr() + 2, 56, g.state, g.workspace, g.cfg)   # misaligned
    with pytest.raises(amp.B200AmpError):
        amp.pass2_f16(g.master, g.m, g.v, g.grads16, g.weights16, 64, 0, g.tensors, 1025, g.state, 0.9, 0.95, 1e-8)
    with pytest.raises(amp.B200AmpError):
        amp.pass2_f16(g.master.data_ptr() + 16, g.m, g.v, g.grads16, g.weights16, 56, 0, g.tensors, 1, g.state,
                      0.9, 0.95, 1e-8)
    with pytest.raises(amp.B200AmpError):
        amp.finalize_step(g.state, g.partial, g.cfg, g.history, 0)                  # history without a length
    with pytest.raises(amp.B200AmpError):
        amp.unscale_and_norm(g.master, 0, g.state, g.partial)
    # the context is still usable
    g.step_f16()
    assert g.read_state().step == 1


def test_one_oracle_rounding_variant_gives_the_kernel_bits(G, O):
    """With the clip inactive (coef exactly 1) the step is purely elementwise, so the oracle
    variant that fuses the same multiply-adds as the compiled kernel must reproduce master, m,
    v and the fp16 copy bit for bit. Exactly which variant that is gets printed."""
    from cuda_transformer_b200 import amp
    n = 1 << 20
    rng = np.random.default_rng(21)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    table = [(0, n // 2, 1), (n // 2, n // 2, 0)]
    kw = dict(grad_clip=1e30)
    gpu = G.GpuStep(init, table, sched(amp, **kw), loss_scale=65536.0)
    variants = {c: O.OracleStep(init, table, sched(O, **kw), loss_scale=65536.0, contract=c) for c in (0, 1, 3, 5, 7)}
    for _ in range(4):
        bits = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16).view(np.uint16)
        gpu.set_grads16(bits)
        gpu.step_f16()
        for o in variants.values():
            o.step_f16(bits)
    st = gpu.read_state()
    hm = gpu.host()
    matches = []
    for c, o in variants.items():
        assert st.clip_coef == 1.0 and o.state.clip_coef == 1.0
        same_scalars = (st.step_size == o.state.step_size and st.bc2_sqrt == o.state.bc2_sqrt
                        and st.decay == o.state.decay)
        same = all(np.array_equal(a, b) for a, b in zip(hm, (o.master, o.m, o.v, o.weights16)))
        if same and same_scalars:
            matches.append(c)
        assert H.rel_err(o.master, hm[0]) <= H.STATE_TOL and H.rel_err(o.m, hm[1]) <= H.STATE_TOL
        assert H.rel_err(o.v, hm[2]) <= H.STATE_TOL
    print("oracle contract variants that reproduce the kernel's bits:", matches)
    assert matches, "no rounding variant of the oracle reproduces the kernel bit for bit"
    assert 0 not in matches, "the kernel was expected to use fused multiply-adds"


# ---------------------------------------------------------------- the reference's own CUDA kernels

def _ref():
    from oracle import ref_cuda
    if not ref_cuda.available():
        pytest.skip("oracle/_ref/libref_amp.so was not built (no reference checkout at build time)")
    return ref_cuda, ref_cuda.load()


def test_compat_path_is_bit_identical_to_the_reference_kernels(G):
    """Same fp32 gradients through the reference's kernels (built from its sources for sm_100a)
    and through the compat entry points: partial[512], the 60 state bytes, the unscaled gradients,
    params, m, v and the fp16 copy must carry the same bits, step after step, skip included."""
    from cuda_transformer_b200 import amp
    from cuda_transformer_b200.layout import CONFIGS, param_layout
    ref_cuda, ref = _ref()
    slots = param_layout(CONFIGS["readme"])
    n = slots[-1].offset + slots[-1].count
    table = H.table_of(slots)
    gen = torch.Generator().manual_seed(0)
    init = (torch.randn(n, generator=gen) * 0.02).numpy()
    cfg = sched(amp, growth_interval=3)
    mine = G.GpuStep(init, table, cfg, loss_scale=65536.0)
    theirs = G.GpuStep(init, table, cfg, loss_scale=65536.0)
    s = torch.cuda.current_stream().cuda_stream
    for k in range(6):
        g = torch.randn(n, generator=gen) * 1e-3 * mine.read_state().loss_scale
        if k == 2:
            g[777] = float("inf")
        g_np = g.numpy()
        g_mine = mine.step_f32(g_np)
        g_theirs = G.to_dev(g_np)
        ref.refamp_begin_step(theirs.state.data_ptr(), s)
        ref_cuda.optimizer_step(ref, g_theirs.data_ptr(), n, theirs.state.data_ptr(), theirs.partial.data_ptr(),
                                C.addressof(cfg), theirs.history.data_ptr(), theirs.history_len,
                                theirs.master.data_ptr(), theirs.weights16.data_ptr(), theirs.m.data_ptr(),
                                theirs.v.data_ptr(), theirs.tensors.data_ptr(), theirs.ntensors, cfg.beta1,
                                cfg.beta2, theirs.eps, s)
        torch.cuda.synchronize()
        assert torch.equal(mine.partial, theirs.partial) or k == 2, k      # NaN partials never compare equal
        assert bytes(mine.read_state())[:32] == bytes(theirs.read_state())[:32], k
        G.assert_states_equal(mine.read_state(), theirs.read_state(), tol=0.0 if k != 2 else 1e-6)
        if k != 2:
            assert torch.equal(g_mine, g_theirs), k
        for a, b in zip(mine.host(), theirs.host()):
            assert np.array_equal(a, b), k
    assert mine.read_state().skipped == 1


def test_native_path_matches_the_reference_kernels(G):
    """fp16 gradient arena through the native kernels against the reference's kernels fed
    float(fp16 gradient): control flow bit-exact, state arrays within 1e-6, fp16 weights 1 ulp."""
    from cuda_transformer_b200 import amp
    from cuda_transformer_b200.layout import CONFIGS, param_layout
    ref_cuda, ref = _ref()
    slots = param_layout(CONFIGS["readme"])
    n = slots[-1].offset + slots[-1].count
    table = H.table_of(slots)
    gen = torch.Generator().manual_seed(0)
    init = (torch.randn(n, generator=gen) * 0.02).numpy()
    cfg = sched(amp, growth_interval=4)
    mine = G.GpuStep(init, table, cfg, loss_scale=65536.0)
    theirs = G.GpuStep(init, table, cfg, loss_scale=65536.0)
    s = torch.cuda.current_stream().cuda_stream
    identical = 0
    for k in range(10):
        g16 = (torch.randn(n, generator=gen) * 1e-3 * mine.read_state().loss_scale).half()
        if k == 5:
            g16[123456] = float("nan")
        mine.grads16.copy_(g16)
        mine.step_f16()
        g32 = g16.float().cuda()
        ref.refamp_begin_step(theirs.state.data_ptr(), s)
        ref_cuda.optimizer_step(ref, g32.data_ptr(), n, theirs.state.data_ptr(), theirs.partial.data_ptr(),
                                C.addressof(cfg), theirs.history.data_ptr(), theirs.history_len,
                                theirs.master.data_ptr(), theirs.weights16.data_ptr(), theirs.m.data_ptr(),
                                theirs.v.data_ptr(), theirs.tensors.data_ptr(), theirs.ntensors, cfg.beta1,
                                cfg.beta2, theirs.eps, s)
        torch.cuda.synchronize()
        a, b = mine.read_state(), theirs.read_state()
        G.assert_states_equal(a, b, tol=1e-6)
        identical += int(a.clip_coef == b.clip_coef)
    hm, ht = mine.host(), theirs.host()
    for x, y in zip(hm[:3], ht[:3]):
        assert H.rel_err(y, x) <= H.STATE_TOL
    assert H.half_ulp_distance(ht[3], hm[3]) <= 1
    assert mine.read_state().skipped == 1 and mine.read_state().adam_t == 9


def test_staged_kernel_gives_up_a_starved_wait_and_reports_it(G):
    """Failure detection without a fault: the staged kernel's barrier waits are bounded. With the
    test hook one CTA announces bytes that never arrive; its wait must run out (well under a
    second), the kernel must return, b200amp_device_error must report it once, and the context
    must stay usable."""
    import time
    from cuda_transformer_b200 import _lib, amp
    lib = _lib.load()
    n = 148 * 2048 * 6
    rng = np.random.default_rng(13)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    bits = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16).view(np.uint16)
    flag = C.c_int(-1)
    _lib.check(lib.b200amp_device_error(C.byref(flag)))                 # clear anything older
    g = G.GpuStep(init, [(0, n, 1)], sched(amp), loss_scale=65536.0)
    g.set_grads16(bits)
    try:
        _lib.check(lib.b200amp_tune_set(b"pass2_variant", 1))
        _lib.check(lib.b200amp_tune_set(b"pass2_test_starve", 1))
        t0 = time.perf_counter()
        g.step_f16()
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
    finally:
        lib.b200amp_tune_set(b"pass2_test_starve", 0)
        lib.b200amp_tune_set(b"pass2_variant", 0)
    assert waited < 10.0, f"the bounded wait took {waited:.1f} s"
    _lib.check(lib.b200amp_device_error(C.byref(flag)))
    assert flag.value == 1, "the starved wait was not reported"
    _lib.check(lib.b200amp_device_error(C.byref(flag)))
    assert flag.value == 0, "reading the flag clears it"
    # the context is intact: a fresh optimizer steps and matches the registers-only kernel
    a = G.GpuStep(init, [(0, n, 1)], sched(amp), loss_scale=65536.0)
    a.set_grads16(bits)
    a.step_f16()
    _lib.check(lib.b200amp_tune_set(b"pass2_variant", 1))
    try:
        b = G.GpuStep(init, [(0, n, 1)], sched(amp), loss_scale=65536.0)
        b.set_grads16(bits)
        b.step_f16()
        torch.cuda.synchronize()
    finally:
        lib.b200amp_tune_set(b"pass2_variant", 0)
    assert all(np.array_equal(x, y) for x, y in zip(a.host(), b.host()))
    _lib.check(lib.b200amp_device_error(C.byref(flag)))
    assert flag.value == 0


def test_fp32_gradient_bridge_matches_cast_then_pass1(G):
    """b200amp_cast_pass1_f32: the reference's fp32 loss-scaled gradient arena -> fp16 arena + pass 1
    (+ finalize) in one sweep, optionally clearing the fp32 arena. Must equal: round to fp16, then the
    native pass 1 / step on that fp16 arena, bit for bit; an fp32 value beyond the fp16 range becomes
    inf and skips the step."""
    from cuda_transformer_b200 import _lib, amp
    n = (1 << 21) + 8 * 77
    rng = np.random.default_rng(31)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    table = [(0, 4096, 0), (4096, n - 4096, 1)]
    for trial, poison in enumerate((False, True)):
        g32_host = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float32)
        if poison:
            g32_host[n // 3] = 1.0e6                      # finite in fp32, inf in fp16
        with np.errstate(over="ignore"):                # the poisoned value is meant to become inf
            want16 = g32_host.astype(np.float16)
        # (a) reference flow: fp16 arena given, native step
        a = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
        a.set_grads16(want16.view(np.uint16))
        a.step_f16()
        # (b) bridge with the finalize inside, then pass 2
        b = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
        g32 = G.to_dev(g32_host)
        amp.cast_pass1_f32(g32, b.grads16, n, True, b.state, b.workspace, b.cfg, b.history, b.history_len)
        amp.pass2_f16(b.master, b.m, b.v, b.grads16, b.weights16, n, 0, b.tensors, b.ntensors, b.state,
                      b.cfg.beta1, b.cfg.beta2, b.eps)
        torch.cuda.synchronize()
        assert np.array_equal(H.f16_bits(b.grads16.cpu()), want16.view(np.uint16))
        assert not g32.any(), "clear_source must leave zeros in the fp32 arena"
        assert bytes(a.read_state()) == bytes(b.read_state())
        assert all(np.array_equal(x, y) for x, y in zip(a.host(), b.host()))
        assert b.read_state().found_inf == (1 if poison else 0)
        # (c) without the finalize and without clearing: only {sum, flag}, source untouched
        c = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
        g32 = G.to_dev(g32_host)
        amp.cast_pass1_f32(g32, c.grads16, n, False, c.state, c.workspace)
        ws_ref = torch.zeros_like(c.workspace)
        amp.pass1_f16(c.grads16, n, c.state, ws_ref)
        torch.cuda.synchronize()
        got = c.workspace[:16].view(torch.float64).cpu().numpy()
        ref = ws_ref[:16].view(torch.float64).cpu().numpy()
        assert got[1] == ref[1] == (1.0 if poison else 0.0)
        assert (got[0] == ref[0]) or (np.isinf(got[0]) and np.isinf(ref[0]))
        assert np.array_equal(g32.cpu().numpy(), g32_host)
        assert c.read_state().step == 0
    with pytest.raises(amp.B200AmpError):
        amp.cast_pass1_f32(g32, c.grads16, n - 4, False, c.state, c.workspace)


def test_compat_adamw_wide_and_narrow_forms_agree(G, O):
    """b200amp_adamw_multi_f32 uses 256-bit accesses when n % 8 == 0 and the arrays are 32-byte
    aligned, and the reference's 4-element granularity otherwise. Same arena through both forms
    (the narrow one by starting 4 elements in): same bits, and both match the oracle."""
    from cuda_transformer_b200 import amp
    n = 8 * 4099
    rng = np.random.default_rng(41)
    init = (rng.standard_normal(n + 8) * 0.5).astype(np.float32)
    g = (rng.standard_normal(n + 8) * 1e-3).astype(np.float32)
    table = [(0, 1028, 1), (1028, 2052, 0), (3080, n + 8 - 3080, 1)]
    kw = dict(weight_decay=0.3, lr=1e-2, min_lr=1e-2, grad_clip=1e30)
    wide = G.GpuStep(init[:n], table, sched(amp, **kw), loss_scale=1.0)
    wide.step_f32(g[:n])
    ora = O.OracleStep(init[:n], table, sched(O, **kw), loss_scale=1.0)
    ora.step_f32(g[:n])
    compare_arrays(wide, ora)
    # the narrow form: n - 4 elements starting at element 4 (16-byte aligned only), table shifted by 4
    full = G.GpuStep(init[:n], table, sched(amp, **kw), loss_scale=1.0)
    shifted = [(0, 1024, 1), (1024, 2052, 0), (3076, n - 4 - 3076, 1)]
    tab_dev = G.table_dev(shifted)
    g_dev = G.to_dev(g[:n])
    amp.begin_step(full.state)
    amp.unscale_and_norm(g_dev, n, full.state, full.partial)
    amp.finalize_step(full.state, full.partial, full.cfg, full.history, full.history_len)
    m4 = n - 4
    amp.adamw_multi(full.master.data_ptr() + 16, full.weights16.data_ptr() + 8, g_dev.data_ptr() + 16,
                    full.m.data_ptr() + 16, full.v.data_ptr() + 16, m4, tab_dev, len(shifted), full.state,
                    full.cfg.beta1, full.cfg.beta2, full.eps)
    torch.cuda.synchronize()
    for a, b in zip(wide.host(), full.host()):
        assert np.array_equal(a[4:], b[4:])
    assert np.array_equal(full.host()[0][:4], init[:4])         # the first quad was outside the narrow call


def test_growth_after_2000_clean_steps_as_the_reference_run(G, O):
    """The reference's production setting (growth_interval 2000, cuda/gpt_fast.cu:142-143; its
    training log shows S going 65,536 -> 131,072 at step 2000): 2001 graph replays of the step on
    a small arena against the oracle, with the whole history ring compared at the end."""
    from cuda_transformer_b200 import amp
    n = 8 * 512
    rng = np.random.default_rng(2000)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    bits = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16).view(np.uint16)
    table = [(0, n // 4, 0), (n // 4, n - n // 4, 1)]
    cfg = amp.make_schedule(lr=6e-4, min_lr=6e-5, warmup_steps=100, max_steps=2500, growth_interval=2000)
    ocfg = O.make_schedule(lr=6e-4, min_lr=6e-5, warmup_steps=100, max_steps=2500, growth_interval=2000)
    g = G.GpuStep(init, table, cfg, loss_scale=65536.0, history_len=4096)
    g.set_grads16(bits)
    ora = O.OracleStep(init, table, ocfg, loss_scale=65536.0, history_len=4096)
    stream = torch.cuda.Stream()
    graph = amp.CudaGraph()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        graph.capture(stream, lambda: g.step_f16())
    for _ in range(2001):
        graph.launch(stream)
    stream.synchronize()
    for _ in range(2001):
        ora.step_f16(bits)          # the same scaled gradients every step: step 2000 sees them at S = 131072
    st = g.read_state()
    assert st.step == 2001 and st.adam_t == 2001 and st.skipped == 0
    assert st.loss_scale == 131072.0 and st.good_steps == 1
    G.assert_states_equal(st, ora.state, tol=1e-6)
    hist = np.frombuffer(g.history.cpu().numpy().tobytes(), dtype=np.float32).reshape(4096, 15)
    scales = hist[:2001, 0]
    assert np.all(scales[:1999] == 65536.0) and scales[1999] == 131072.0 and scales[2000] == 131072.0
    lrs = hist[:2001, 7].astype(np.float64)
    want = np.array([O.lr_at(k, ocfg) for k in range(2001)])
    assert np.max(np.abs(lrs - want) / want) <= 1e-6
    gm, gmm, gv, gw = g.host()
    for got, ref in ((gm, ora.master), (gmm, ora.m), (gv, ora.v)):
        assert H.rel_err(ref, got) <= 2e-6, "2001 steps of one-ulp differences may add up to a little over 1e-6"
    assert H.half_ulp_distance(ora.weights16, gw) <= 1


def test_zero_rows_with_zero_gradient_stay_zero(G):
    """The optimizer half of padded_rows (reference/test_reference.py:113-116) on the GPU, native
    and compat path: zero parameter + zero gradient stays +0.0 exactly under weight decay, and so
    does the arena's alignment padding in AmpOptimizer."""
    from cuda_transformer_b200 import amp
    n = 8 * 256
    rng = np.random.default_rng(4)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    pad = slice(8 * 100, 8 * 140)
    init[pad] = 0.0
    table = [(0, 8 * 200, 1), (8 * 200, n - 8 * 200, 0)]
    native = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
    compat = G.GpuStep(init, table, sched(amp), loss_scale=65536.0)
    for k in range(5):
        g = (rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16)
        g[pad] = 0.0
        native.set_grads16(g.view(np.uint16))
        native.step_f16()
        compat.step_f32(g.astype(np.float32))
    for step in (native, compat):
        master, m, v, w16 = step.host()
        for arr in (master, m, v):
            assert np.all(arr[pad].view(np.uint32) == 0), "a padded row moved (or turned into -0.0)"
        assert np.all(w16[pad] == 0)
        assert np.all(master[:8 * 100] != init[:8 * 100])
    slots = H.debug_slots()
    opt = amp.AmpOptimizer(slots, sched(amp), loss_scale=65536.0)
    opt.set_params(torch.from_numpy(H.debug_init()))
    assert opt.n > opt.n_params or opt.n % 1024 == 0
    opt.grads16[: opt.n_params].copy_((torch.randn(opt.n_params) * 1e-3 * 65536.0).half())
    for _ in range(3):
        opt.optimizer_step()
    tail = slice(opt.n_params, opt.n)
    for t in (opt.master, opt.m, opt.v, opt.weights16):
        assert not torch.any(t[tail] != 0)


def test_steps_fed_from_pinned_host_memory_equal_the_serial_steps(G):
    """HostGradientFeed on AmpOptimizer: five steps whose gradients come from pinned host memory
    through two device arenas taking turns (one with an inf), against the same optimizer stepped
    serially on the same gradients: every state and every array bit for bit, tickets collected
    late, early and by the submission of a later step."""
    from cuda_transformer_b200 import amp
    from cuda_transformer_b200.layout import CONFIGS, param_layout
    slots = param_layout(CONFIGS["debug"])
    cfg = amp.make_schedule(grad_clip=0.5, growth_interval=2)
    fed = amp.AmpOptimizer(slots, cfg, loss_scale=4096.0, history_len=8)
    serial = amp.AmpOptimizer(slots, cfg, loss_scale=4096.0, history_len=8)
    gen = torch.Generator().manual_seed(5)
    init = torch.randn(fed.n_params, generator=gen) * 0.02
    fed.set_params(init)
    serial.set_params(init)
    batches = []
    for k in range(5):
        g = (torch.randn(fed.n, generator=gen) * 1e-3 * 4096.0).half()
        g[fed.n_params:] = 0
        if k == 2:
            g[77] = float("inf")
        batches.append(g.pin_memory())
    want = []
    for g in batches:
        serial.grads16.copy_(g)
        serial.optimizer_step()
        want.append(bytes(serial.read_state()))
    tickets = [fed.submit_host_gradients(g) for g in batches]       # submitting 2, 3, 4 collects 0, 1, 2 internally
    assert tickets == [0, 1, 2, 3, 4]
    got = [bytes(fed.collect(t)) for t in (4, 3)]                   # out of order is fine
    fed.drain_host_feed()
    got = [bytes(fed.collect(t)) for t in (0, 1, 2)] + got[::-1]
    assert got == want
    with pytest.raises(ValueError):
        fed.collect(3)
    assert bytes(fed.read_state()) == want[-1]
    for a, b in ((fed.master, serial.master), (fed.m, serial.m), (fed.v, serial.v), (fed.weights16, serial.weights16)):
        assert torch.equal(a, b)
    st = fed.read_state()
    assert st.skipped == 1 and st.adam_t == 4
