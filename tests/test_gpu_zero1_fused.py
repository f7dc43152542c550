"""The fused ZeRO-1 kernels (reduce-scatter + pass 1, pass 2 + all-gather).

On one GPU the R ranks are emulated: R gradient arenas, R weight arenas and R pair tables all
live on the same device and each emulated rank's launch gets the same pointer lists a real
rank would get. The kernels never wait on each other, so running the ranks' launches one after
the other on one stream is the same computation. With two or more GPUs a second test runs the
real thing (one process per GPU, symmetric memory, barriers)."""
import os
import socket

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def _average_fp16(arenas_bits, world):
    """fp32 sum in rank order, * 1/world, one rounding to fp16: what rs_pass1 stores."""
    acc = np.zeros(arenas_bits[0].size, dtype=np.float32)
    for bits in arenas_bits:
        acc += bits.view(np.float16).astype(np.float32)
    return (acc * np.float32(1.0 / world)).astype(np.float16).view(np.uint16)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_emulated_ranks_match_single_arena_step(world):
    import gpu_helpers as G
    from cuda_transformer_b200 import _lib, amp
    from oracle import ref_step as O
    lib = _lib.load()
    n = 8 * 128 * 97 * world                    # every slice a multiple of 128 elements
    per = n // world
    rng = np.random.default_rng(100 + world)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    edges = sorted(set([0] + [int(x) * 4 for x in rng.integers(1, n // 4, size=23)]))
    table = [(a, b - a, i % 2) for i, (a, b) in enumerate(zip(edges, edges[1:] + [n]))]
    cfg = amp.make_schedule(grad_clip=0.5)
    scale = 4096.0

    def rank_grads(seed, poison=None):
        g = (np.random.default_rng(1000 * world + seed).standard_normal(n) * 1e-3 * scale).astype(np.float16)
        if poison is not None:
            g[poison] = np.float16(np.inf)
        return g.view(np.uint16)

    for trial, poison in enumerate((None, (world - 1, per * (world // 2) + 17))):
        arenas_bits = [rank_grads(10 * trial + r, poison[1] if poison and poison[0] == r else None)
                       for r in range(world)]
        arenas = [torch.from_numpy(b.copy()).view(torch.float16).cuda() for b in arenas_bits]
        weights = [torch.zeros(n, dtype=torch.float16, device="cuda") for _ in range(world)]
        for w in weights:
            amp.cast_to_x(w, G.to_dev(init), n)
        tables = [torch.full((2 * world,), -1.0, dtype=torch.float64, device="cuda") for _ in range(world)]
        ranks = []
        for r in range(world):
            sl = slice(r * per, (r + 1) * per)
            g = G.GpuStep(init[sl], table, cfg, loss_scale=scale)       # master/m/v/state/workspace of rank r
            ranks.append(g)
        reduced = [torch.zeros(per, dtype=torch.float16, device="cuda") for _ in range(world)]
        # --- reduce-scatter + pass 1, every emulated rank
        for r, g in enumerate(ranks):
            src = [a.data_ptr() + 2 * r * per for a in arenas]
            amp.rs_pass1_f16(src, r, reduced[r], per, g.state, g.workspace, [t.data_ptr() for t in tables])
        torch.cuda.synchronize()
        want_bits = _average_fp16(arenas_bits, world)
        got_bits = np.concatenate([H.f16_bits(x.cpu()) for x in reduced])
        assert np.array_equal(got_bits, want_bits), "averaged slice is not fp16(fp32 sum / world)"
        for t in tables[1:]:
            assert torch.equal(t, tables[0]), "pair tables differ between ranks"
        pairs = tables[0].cpu().numpy().reshape(world, 2)
        ws_check = torch.zeros(lib.b200amp_workspace_bytes(), dtype=torch.uint8, device="cuda")
        for r in range(world):
            amp.pass1_f16(reduced[r], per, ranks[r].state, ws_check)    # pass 1 alone on the averaged slice
            alone = ws_check[:16].view(torch.float64).cpu().numpy()
            if poison is None:
                assert pairs[r, 0] == alone[0] and pairs[r, 1] == alone[1] == 0.0
        if poison is not None:
            assert [p[1] for p in pairs] == [1.0 if r == world // 2 else 0.0 for r in range(world)]
        # --- finalize on every rank from the same table, then pass 2 + all-gather
        before = [w.clone() for w in weights]
        for r, g in enumerate(ranks):
            amp.finalize_sums(g.state, tables[r], world, cfg, g.history, g.history_len)
        for r, g in enumerate(ranks):
            dst = [w.data_ptr() + 2 * r * per for w in weights]
            amp.pass2_ag_f16(g.master, g.m, g.v, reduced[r], dst, per, r * per, g.tensors, g.ntensors, g.state,
                             cfg.beta1, cfg.beta2, g.eps)
        torch.cuda.synchronize()
        states = [bytes(g.read_state()) for g in ranks]
        assert all(s == states[0] for s in states), "ranks disagree on the step state"
        st = ranks[0].read_state()
        for w in weights[1:]:
            assert torch.equal(w, weights[0]), "weight arenas differ between ranks"
        if poison is not None:
            assert st.found_inf == 1 and st.skipped == 1
            assert all(torch.equal(a, b) for a, b in zip(before, weights)), "a skipped step wrote weights"
            continue
        # --- against one arena stepped on the averaged gradients (library) and the oracle
        whole = G.GpuStep(init, table, cfg, loss_scale=scale)
        whole.set_grads16(want_bits)
        whole.step_f16()
        ora = O.OracleStep(init, table, O.make_schedule(grad_clip=0.5), loss_scale=scale)
        ora.step_f16(want_bits)
        G.assert_states_equal(st, whole.read_state(), tol=1e-6)
        G.assert_states_equal(st, ora.state, tol=1e-6)
        wm, wmm, wv, ww = whole.host()
        gm = np.concatenate([g.host()[0] for g in ranks])
        gmm = np.concatenate([g.host()[1] for g in ranks])
        gv = np.concatenate([g.host()[2] for g in ranks])
        gw = H.f16_bits(weights[0].cpu())
        if st.clip_coef == whole.read_state().clip_coef:
            assert np.array_equal(gm, wm) and np.array_equal(gmm, wmm) and np.array_equal(gv, wv)
            assert np.array_equal(gw, ww)
        for got, want in ((gm, ora.master), (gmm, ora.m), (gv, ora.v)):
            assert H.rel_err(want, got) <= H.STATE_TOL
        assert H.half_ulp_distance(ora.weights16, gw) <= 1
        assert np.array_equal(gm.astype(np.float16).view(np.uint16), gw)


def _emulated_setup(world, per, seed, scale=4096.0, clip=0.5, poison=False, ntable=31):
    """R emulated ranks on one GPU: gradient arenas, weight arenas, pair tables, flag blocks, and
    one GpuStep (master / m / v / state / workspace of the slice) per rank."""
    import gpu_helpers as G
    from cuda_transformer_b200 import _lib, amp
    n = per * world
    rng = np.random.default_rng(seed)
    init = (rng.standard_normal(n) * 0.02).astype(np.float32)
    edges = sorted(set([0] + [int(x) * 4 for x in rng.integers(1, n // 4, size=ntable)]))
    table = [(a, b - a, i % 2) for i, (a, b) in enumerate(zip(edges, edges[1:] + [n]))]
    cfg = amp.make_schedule(grad_clip=clip)
    arenas = []
    for r in range(world):
        g = (rng.standard_normal(n) * 1e-3 * scale).astype(np.float16)
        if poison and r == world - 1:
            g[per * (world // 2) + per // 3 + 5] = np.float16(np.nan)
        arenas.append(torch.from_numpy(g).cuda())

    def fresh():
        w = [torch.zeros(n, dtype=torch.float16, device="cuda") for _ in range(world)]
        for t in w:
            amp.cast_to_x(t, G.to_dev(init), n)
        return dict(
            weights=w,
            tables=[torch.full((2 * world,), -1.0, dtype=torch.float64, device="cuda") for _ in range(world)],
            blocks=[torch.zeros(_lib.ZERO1_SYNC_BYTES // 4, dtype=torch.int32, device="cuda") for _ in range(world)],
            ranks=[G.GpuStep(init[r * per:(r + 1) * per], table, cfg, loss_scale=scale) for r in range(world)],
            reduced=[torch.full((per,), 7.0, dtype=torch.float16, device="cuda") for _ in range(world)])
    return n, init, table, cfg, arenas, fresh


def _snapshot(run):
    torch.cuda.synchronize()
    return dict(state=[bytes(g.read_state()) for g in run["ranks"]],
                pairs=[t.cpu().numpy().tobytes() for t in run["tables"]],
                reduced=[H.f16_bits(x.cpu()) for x in run["reduced"]],
                weights=[H.f16_bits(w.cpu()) for w in run["weights"]],
                arrays=[g.host()[:3] for g in run["ranks"]],
                ws=[g.workspace[:32].cpu().numpy().tobytes() for g in run["ranks"]])


def _assert_same(got, base, what):
    assert got["state"] == base["state"] and got["pairs"] == base["pairs"], what
    assert got["ws"] == base["ws"], f"{what}: sums, ticket and flag of the workspace"
    for a, b in zip(got["reduced"] + got["weights"], base["reduced"] + base["weights"]):
        assert np.array_equal(a, b), what
    for ra, rb in zip(got["arrays"], base["arrays"]):
        assert all(np.array_equal(x, y) for x, y in zip(ra, rb)), what


def _plain_step(run, arenas, world, per, cfg):
    """The caller-ordered entry points, rank after rank."""
    from cuda_transformer_b200 import amp
    tptrs = [t.data_ptr() for t in run["tables"]]
    for r, g in enumerate(run["ranks"]):
        src = [a.data_ptr() + 2 * r * per for a in arenas]
        amp.rs_pass1_f16(src, r, run["reduced"][r], per, g.state, g.workspace, tptrs)
    for r, g in enumerate(run["ranks"]):
        amp.finalize_sums(g.state, run["tables"][r], world, cfg, g.history, g.history_len)
    for r, g in enumerate(run["ranks"]):
        dst = [w.data_ptr() + 2 * r * per for w in run["weights"]]
        amp.pass2_ag_f16(g.master, g.m, g.v, run["reduced"][r], dst, per, r * per, g.tensors, g.ntensors, g.state,
                         cfg.beta1, cfg.beta2, g.eps)


def _self_ordered_step(run, arenas, world, per, cfg, form="sm", pieces=3, limit=0):
    """The library-ordered entry points. Emulated ranks run one after the other on one stream,
    so the announcements a real rank's kernel would make while the others wait are made for all
    ranks first (a kernel that waited for a launch still queued behind it would only time out)."""
    from cuda_transformer_b200 import _lib, amp
    bptrs = [b.data_ptr() for b in run["blocks"]]
    sync = amp.make_sync(bptrs, limit)
    tptrs = [t.data_ptr() for t in run["tables"]]
    if form == "push":
        # every emulated rank pushes first (copies and piece flags), then every owner reduces
        rows = run.setdefault("push_rows", [torch.full((world * per,), 55.0, dtype=torch.float16, device="cuda")
                                            for _ in range(world)])
        for r in range(world):
            amp.rs_push_f16_ce(arenas[r], [x.data_ptr() for x in rows], r, per, pieces, sync)
        torch.cuda.synchronize()                # the lanes' copies have landed; a real owner's kernels wait instead
    else:
        for r in range(world):
            amp.zero1_barrier(sync, world, r, _lib.PHASE_GRADS, _lib.SYNC_SIGNAL)
    for r, g in enumerate(run["ranks"]):
        src = [a.data_ptr() + 2 * r * per for a in arenas]
        if form == "sm":
            amp.rs_pass1_f16_sync(src, r, run["reduced"][r], per, g.state, g.workspace, tptrs, sync)
        elif form == "push":
            amp.rs_pass1_f16_pushed(src[r], run["push_rows"][r], world, r, run["reduced"][r], per, pieces, g.state,
                                    g.workspace, tptrs, sync)
        else:
            staging = torch.full((max(1, (world - 1) * per),), 77.0, dtype=torch.float16, device="cuda")
            amp.rs_pass1_f16_ce(src, r, staging, run["reduced"][r], per, pieces, g.state, g.workspace, tptrs, sync)
    for r, g in enumerate(run["ranks"]):
        amp.finalize_sums_sync(g.state, run["tables"][r], world, r, cfg, sync, g.history, g.history_len)
    for r, g in enumerate(run["ranks"]):
        dst = [w.data_ptr() + 2 * r * per for w in run["weights"]]
        if form in ("sm", "push"):
            amp.pass2_ag_f16(g.master, g.m, g.v, run["reduced"][r], dst, per, r * per, g.tensors, g.ntensors,
                             g.state, cfg.beta1, cfg.beta2, g.eps)
        else:
            amp.pass2_ag_f16_ce(g.master, g.m, g.v, run["reduced"][r], dst, r, per, r * per, g.tensors, g.ntensors,
                                g.state, cfg.beta1, cfg.beta2, g.eps, pieces)
    for r in range(world):
        amp.zero1_barrier(sync, world, r, _lib.PHASE_WEIGHTS, _lib.SYNC_SIGNAL)
    for r in range(world):
        amp.zero1_barrier(sync, world, r, _lib.PHASE_WEIGHTS, _lib.SYNC_WAIT | _lib.SYNC_ADVANCE)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_self_ordered_parts_and_copy_engine_forms_are_the_fused_kernels_bit_for_bit(world):
    """Emulated ranks on one GPU: the reduce-scatter in parts, the library-ordered (flag word)
    entry points and both copy-engine forms (the copies are then device-local) against
    b200amp_rs_pass1_f16 / b200amp_pass2_ag_f16, two steps each, the second with a NaN."""
    from cuda_transformer_b200 import amp
    vb_elems = amp.pass1_partition(8)[1]                 # 8192 elements per virtual block
    per = vb_elems * 13 + 8 * 57                        # 14 virtual blocks, the last one short
    assert amp.pass1_partition(per) == (14, vb_elems)
    for poison in (False, True):
        n, init, table, cfg, arenas, fresh = _emulated_setup(world, per, 7 + world, poison=poison)
        base_run = fresh()
        _plain_step(base_run, arenas, world, per, cfg)
        base = _snapshot(base_run)
        assert base_run["ranks"][0].read_state().found_inf == (1 if poison else 0)

        # in parts
        run = fresh()
        tptrs = [t.data_ptr() for t in run["tables"]]
        cuts = [0, 1, 4, 9, 14]
        for r, g in enumerate(run["ranks"]):
            src = [a.data_ptr() + 2 * r * per for a in arenas]
            for a, b in zip(cuts, cuts[1:]):
                amp.rs_pass1_f16_part(src, r, run["reduced"][r], per, a, b - a, b == 14, g.state, g.workspace, tptrs)
        for r, g in enumerate(run["ranks"]):
            amp.finalize_sums(g.state, run["tables"][r], world, cfg, g.history, g.history_len)
        for r, g in enumerate(run["ranks"]):
            dst = [w.data_ptr() + 2 * r * per for w in run["weights"]]
            amp.pass2_ag_f16(g.master, g.m, g.v, run["reduced"][r], dst, per, r * per, g.tensors, g.ntensors,
                             g.state, cfg.beta1, cfg.beta2, g.eps)
        _assert_same(_snapshot(run), base, "parts")

        for form in ("sm", "ce", "push"):
            run = fresh()
            _self_ordered_step(run, arenas, world, per, cfg, form=form, pieces=5)
            _assert_same(_snapshot(run), base, f"self-ordered {form}")
            for r, b in enumerate(run["blocks"]):
                assert amp.zero1_sync_read(b) == (1, 0), "one step counted, no give-up"
            assert amp.device_error() == 0
            # a second step on the same blocks: the counter advances, the flags are reused
            base2 = fresh()
            for k in range(2):
                _plain_step(base2, arenas, world, per, cfg)
            _self_ordered_step(run, arenas, world, per, cfg, form=form, pieces=2)
            _assert_same(_snapshot(run), _snapshot(base2), f"self-ordered {form}, second step")
            assert all(amp.zero1_sync_read(b) == (2, 0) for b in run["blocks"])


def test_step_counter_of_the_flag_blocks_may_wrap():
    """Step numbers are compared for equality and never take the value 0, so the 32-bit counter may
    wrap: blocks whose last completed step is 2^32 - 2 take three more steps (numbers 2^32 - 1, 1,
    2; the piece words of the pushed form still zero from the set-up) and match the caller-ordered path."""
    from cuda_transformer_b200 import amp
    world, per = 4, 8 * 128 * 33
    n, init, table, cfg, arenas, fresh = _emulated_setup(world, per, 321)
    run, base = fresh(), fresh()
    old = np.zeros(256, dtype=np.uint32)
    old[:24] = 0xFFFFFFFE                       # the three phases of every rank, as that history leaves them
    old[24] = 0xFFFFFFFE                        # the last completed step
    for b in run["blocks"]:
        b.copy_(torch.from_numpy(old.view(np.int32)).cuda())
    for k, (form, want) in enumerate((("sm", 0xFFFFFFFF), ("push", 1), ("ce", 2))):
        _self_ordered_step(run, arenas, world, per, cfg, form=form, pieces=2)
        _plain_step(base, arenas, world, per, cfg)
        assert all(amp.zero1_sync_read(b) == (want, 0) for b in run["blocks"]), (k, form)
    _assert_same(_snapshot(run), _snapshot(base), "three steps across the wrap of the step counter")
    assert amp.device_error() == 0


def test_a_rank_that_never_announces_makes_the_wait_run_out_and_the_step_is_not_applied():
    """Two emulated ranks; rank 1 never announces its gradients (nothing sets its flag). Rank 0's
    kernels give up after a short poll limit, report it, apply nothing, and the context stays
    usable: the same buffers, re-armed, then take a correct step."""
    from cuda_transformer_b200 import _lib, amp
    world, per = 2, 8 * 128 * 61
    n, init, table, cfg, arenas, fresh = _emulated_setup(world, per, 99)
    run = fresh()
    g0 = run["ranks"][0]
    before = _snapshot(run)
    sync = amp.make_sync([b.data_ptr() for b in run["blocks"]], 2000)      # a few milliseconds of polling
    tptrs = [t.data_ptr() for t in run["tables"]]
    src = [a.data_ptr() for a in arenas]
    assert amp.device_error() == 0
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    amp.rs_pass1_f16_sync(src, 0, run["reduced"][0], per, g0.state, g0.workspace, tptrs, sync)
    t1.record()
    torch.cuda.synchronize()
    gave_up_after_ms = t0.elapsed_time(t1)
    print(f"a wait of 2000 polls gave up after {gave_up_after_ms:.3f} ms ({gave_up_after_ms / 2000 * 1e3:.2f} us per poll)")
    assert gave_up_after_ms < 100.0, "2000 polls must be a matter of milliseconds"
    amp.finalize_sums_sync(g0.state, run["tables"][0], world, 0, cfg, sync, g0.history, g0.history_len)
    dst = [w.data_ptr() for w in run["weights"]]
    amp.pass2_ag_f16(g0.master, g0.m, g0.v, run["reduced"][0], dst, per, 0, g0.tensors, g0.ntensors, g0.state,
                     cfg.beta1, cfg.beta2, g0.eps)
    amp.zero1_barrier(sync, world, 0, _lib.PHASE_WEIGHTS, _lib.SYNC_SIGNAL | _lib.SYNC_WAIT | _lib.SYNC_ADVANCE)
    torch.cuda.synchronize()
    steps, error = amp.zero1_sync_read(run["blocks"][0])
    assert steps == 0, "the step counter must not advance"
    assert error == (_lib.PHASE_GRADS + 1) | (1 << 8), "phase 'gradients ready', missing rank 1"
    assert amp.device_error() == 2 and amp.device_error() == 0, "reported once, then cleared"
    st = g0.read_state()
    assert st.found_inf == 1 and st.step == 0 and st.skipped == 0 and st.adam_t == 0
    after = _snapshot(run)
    for key in ("pairs", "reduced", "weights"):
        assert all(np.array_equal(np.frombuffer(a, np.uint8) if isinstance(a, bytes) else a,
                                  np.frombuffer(b, np.uint8) if isinstance(b, bytes) else b)
                   for a, b in zip(after[key], before[key])), key
    for ra, rb in zip(after["arrays"], before["arrays"]):
        assert all(np.array_equal(x, y) for x, y in zip(ra, rb)), "master, m or v moved"
    # the copy-engine form gives up the same way (its first launch is the phase-0 exchange)
    for b in run["blocks"]:
        amp.zero1_sync_init(b)
    staging = torch.zeros(per, dtype=torch.float16, device="cuda")
    amp.rs_pass1_f16_ce(src, 0, staging, run["reduced"][0], per, 3, g0.state, g0.workspace, tptrs, sync)
    torch.cuda.synchronize()
    assert amp.zero1_sync_read(run["blocks"][0])[1] == (_lib.PHASE_GRADS + 1) | (1 << 8)
    assert amp.device_error() == 2
    assert np.array_equal(H.f16_bits(run["reduced"][0].cpu()), before["reduced"][0])
    # and so does the owner's side of the pushed form when a peer's piece never arrives
    for b in run["blocks"]:
        amp.zero1_sync_init(b)
    rows = torch.zeros(world * per, dtype=torch.float16, device="cuda")
    amp.rs_pass1_f16_pushed(src[0], rows, world, 0, run["reduced"][0], per, 2, g0.state, g0.workspace, tptrs, sync)
    torch.cuda.synchronize()
    assert amp.zero1_sync_read(run["blocks"][0])[1] == 4 | (1 << 8), "a pushed piece (code 4) of rank 1"
    assert amp.device_error() == 2
    assert np.array_equal(H.f16_bits(run["reduced"][0].cpu()), before["reduced"][0])
    # recovery: state restored by the caller, blocks zeroed; the next step is a correct one
    fresh_run = fresh()
    _self_ordered_step(fresh_run, arenas, world, per, cfg)
    base = fresh()
    _plain_step(base, arenas, world, per, cfg)
    _assert_same(_snapshot(fresh_run), _snapshot(base), "step after a give-up")
    # and the workspace of the rank that gave up was left re-armed (ticket and flag zero)
    assert g0.workspace[16:24].cpu().numpy().tobytes() == bytes(8)


def test_emulated_eight_ranks_at_the_gpt2_small_arena():
    """The GPT-2-small arena at its real size (124,475,904 parameters padded to 124,476,416, 148
    tensors + the zero padding with decay flag 0), eight emulated ranks, against the one-GPU step
    on the averaged gradients (bits), an independent average and norm, and the oracle on windows."""
    import gpu_helpers as G
    from cuda_transformer_b200 import _lib, amp
    from cuda_transformer_b200.layout import CONFIGS, padded, param_layout, tensor_table
    from oracle import ref_step as O
    world = 8
    slots = param_layout(CONFIGS["gpt2-small"])
    n_params = slots[-1].offset + slots[-1].count
    n = padded(n_params)
    assert (n_params, n) == (124_475_904, 124_476_416)
    per = n // world
    table = list(tensor_table(slots)) + [(n_params, n - n_params, 0)]
    cfg = amp.make_schedule()
    scale = 65536.0
    gen = torch.Generator(device="cuda").manual_seed(0)
    init = torch.zeros(n, dtype=torch.float32, device="cuda")
    init[:n_params] = torch.randn(n_params, generator=gen, device="cuda") * 0.02
    arenas = []
    for r in range(world):
        gen = torch.Generator(device="cuda").manual_seed(r + 1)
        g = torch.zeros(n, dtype=torch.float16, device="cuda")
        g[:n_params] = (torch.randn(n_params, generator=gen, device="cuda") * (1e-3 * scale)).half()
        arenas.append(g)
    init_host = init.cpu().numpy()
    weights = [torch.zeros(n, dtype=torch.float16, device="cuda") for _ in range(world)]
    for w in weights:
        amp.cast_to_x(w, init, n)
    tables = [torch.full((2 * world,), -1.0, dtype=torch.float64, device="cuda") for _ in range(world)]
    blocks = [torch.zeros(_lib.ZERO1_SYNC_BYTES // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    ranks = [G.GpuStep(init_host[r * per:(r + 1) * per], table, cfg, loss_scale=scale) for r in range(world)]
    reduced = [torch.zeros(per, dtype=torch.float16, device="cuda") for _ in range(world)]
    run = dict(weights=weights, tables=tables, blocks=blocks, ranks=ranks, reduced=reduced)
    for step in range(2):                               # the second step runs on warm m and v
        _self_ordered_step(run, arenas, world, per, cfg)
    torch.cuda.synchronize()
    states = [bytes(g.read_state()) for g in ranks]
    assert all(s == states[0] for s in states)
    st = ranks[0].read_state()
    assert st.found_inf == 0 and st.adam_t == 2
    assert all(torch.equal(w, weights[0]) for w in weights[1:]), "weight arenas differ between ranks"
    # the averaged slice: fp16(fp32 sum in rank order / 8)
    acc = torch.zeros(n, dtype=torch.float32, device="cuda")
    for a in arenas:
        acc += a.float()
    avg = (acc * 0.125).half()
    del acc
    assert torch.equal(torch.cat(reduced), avg)
    sumsq = float(((avg.double() / scale) ** 2).sum())
    assert abs(st.grad_norm - sumsq ** 0.5) <= 1e-6 * sumsq ** 0.5
    # the zero padding stays zero and undecayed
    tail = slice(n_params - (world - 1) * per, None)
    assert float(ranks[-1].master[tail].abs().sum()) == 0.0 and float(weights[0][n_params:].abs().sum()) == 0.0
    # one arena stepped twice on the averaged gradients by the one-GPU path: the same bits
    whole = amp.AmpOptimizer(slots, cfg, loss_scale=scale, history_len=8)
    whole.master.copy_(init)
    amp.cast_to_x(whole.weights16, whole.master, n)
    whole.grads16.copy_(avg)
    whole.optimizer_step()
    whole.optimizer_step()
    torch.cuda.synchronize()
    G.assert_states_equal(st, whole.read_state(), tol=1e-6)
    if st.clip_coef == whole.read_state().clip_coef:
        assert torch.equal(torch.cat([g.master for g in ranks]), whole.master)
        assert torch.equal(torch.cat([g.m for g in ranks]), whole.m)
        assert torch.equal(torch.cat([g.v for g in ranks]), whole.v)
        assert torch.equal(weights[3], whole.weights16)
    # the oracle, two steps, on windows (some across shard and tensor edges, one in the padding)
    W = 8192
    rng = np.random.default_rng(0)
    starts = [int(x) * 8 for x in rng.integers(0, (n - W) // 8, size=12)]
    starts += [per * r - W // 2 for r in (1, 4, 7)] + [n - W] + [slots[i].offset - W // 2 for i in (1, 50, 100)]
    gm = torch.cat([g.master for g in ranks])
    gmm = torch.cat([g.m for g in ranks])
    gv = torch.cat([g.v for g in ranks])
    history = G.read_struct(ranks[0].history, 0), G.read_struct(ranks[0].history, 1)
    for s0 in starts:
        o = O.OracleStep(init_host[s0:s0 + W], table, O.make_schedule(), loss_scale=scale, arena_offset=s0)
        bits = H.f16_bits(avg[s0:s0 + W].cpu())
        for k in range(2):
            o.state = O.StepState.from_buffer_copy(bytes(history[k]))
            o.pass2_f16(bits)
        assert H.rel_err(o.master, gm[s0:s0 + W].cpu().numpy()) <= H.STATE_TOL
        assert H.rel_err(o.m, gmm[s0:s0 + W].cpu().numpy()) <= H.STATE_TOL
        assert H.rel_err(o.v, gv[s0:s0 + W].cpu().numpy()) <= H.STATE_TOL
        assert H.half_ulp_distance(o.weights16, H.f16_bits(weights[0][s0:s0 + W].cpu())) <= 1


def test_fused_entry_points_reject_bad_arguments():
    import gpu_helpers as G
    from cuda_transformer_b200 import amp
    g = G.GpuStep(np.zeros(64, dtype=np.float32), [(0, 64, 1)], amp.make_schedule())
    red = torch.zeros(64, dtype=torch.float16, device="cuda")
    with pytest.raises(amp.B200AmpError, match="nranks"):
        amp.rs_pass1_f16([g.grads16.data_ptr()] * 3, 0, red, 64, g.state, g.workspace)
    with pytest.raises(amp.B200AmpError, match="my_rank"):
        amp.rs_pass1_f16([g.grads16.data_ptr()] * 2, 2, red, 64, g.state, g.workspace)
    with pytest.raises(amp.B200AmpError):
        amp.rs_pass1_f16([g.grads16.data_ptr(), 0], 0, red, 64, g.state, g.workspace)
    with pytest.raises(amp.B200AmpError):
        amp.pass2_ag_f16(g.master, g.m, g.v, red, [g.weights16.data_ptr() + 2], 64, 0, g.tensors, 1, g.state,
                         0.9, 0.95, 1e-8)
    # ranges longer than one launch addresses with 32-bit group indices are refused before anything runs
    from cuda_transformer_b200 import _lib
    too_long = 8 * ((1 << 31) - (1 << 23) + 1)
    for call in (lambda: amp.pass2_ag_f16(g.master, g.m, g.v, red, [g.weights16.data_ptr()], too_long, 0, g.tensors,
                                          1, g.state, 0.9, 0.95, 1e-8),
                 lambda: amp.pass2_f16(g.master, g.m, g.v, red, g.weights16, too_long, 0, g.tensors, 1, g.state,
                                       0.9, 0.95, 1e-8)):
        with pytest.raises(amp.B200AmpError, match="beyond") as err:
            call()
        assert err.value.status == _lib.ERR_LIMIT


# ---------------------------------------------------------------- two real GPUs

def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_rank(rank, world, port, out_dir):
    import traceback

    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    host = dist.new_group(backend="gloo")       # pass / fail is agreed on the host, between steps

    def agree(ok: bool, where: str) -> None:
        """Every rank learns whether any rank failed, before any of them launches the next step:
        the ranks stop together, so none is left waiting for a peer that has gone."""
        flag = torch.tensor([0 if ok else 1])
        dist.all_reduce(flag, group=host)
        if int(flag.item()) != 0:
            raise AssertionError(f"a rank failed at {where}")

    try:
        import helpers as H2
        from cuda_transformer_b200 import amp
        from cuda_transformer_b200.layout import CONFIGS, param_layout
        from oracle import ref_step as O
        slots = param_layout(CONFIGS["readme"])
        cfg = amp.make_schedule(growth_interval=2)
        fused = amp.FusedZero1Optimizer(slots, cfg, loss_scale=65536.0, history_len=16)
        engines = amp.FusedZero1Optimizer(slots, cfg, loss_scale=65536.0, history_len=16, rs_mover="ce_pull",
                                          ag_mover="ce", pieces=5)
        pushed = amp.FusedZero1Optimizer(slots, cfg, loss_scale=65536.0, history_len=16, rs_mover="ce_push",
                                         ag_mover="sm", pieces=3)
        nccl = amp.ShardedAmpOptimizer(slots, cfg, loss_scale=65536.0, history_len=16)
        gen = torch.Generator().manual_seed(0)
        init = torch.randn(fused.n_params, generator=gen) * 0.02
        for opt in (fused, engines, pushed, nccl):
            opt.set_params(init)
        single = O.OracleStep(init.numpy(), fused.table, O.make_schedule(growth_interval=2), loss_scale=65536.0,
                              history_len=16)
        gen = torch.Generator().manual_seed(rank + 1)
        agree(True, "set-up")
        for k in range(4):
            problem = None
            try:
                scale = fused.read_state().loss_scale
                g = (torch.randn(fused.n, generator=gen) * 1e-3 * scale).half()
                if k == 2 and rank == 1:
                    g[4242] = float("nan")
                for opt in (fused, engines, pushed, nccl):
                    opt.grads16.copy_(g)
                    opt.optimizer_step()
                torch.cuda.synchronize()
            except Exception:       # noqa: BLE001
                problem = traceback.format_exc()
            agree(problem is None, f"step {k} (launch)\n{problem or ''}")
            reduced = torch.zeros(fused.n, dtype=torch.float16, device=fused.device)
            dist.all_gather_into_tensor(reduced, fused.grad_shard)          # test plumbing
            try:
                # the copy-engine forms (pull + push of weights; push of gradients) are the fused form bit for bit
                for other in (engines, pushed):
                    assert bytes(other.read_state()) == bytes(fused.read_state()), (k, other.rs_mover)
                    for name in ("grad_shard", "master", "m", "v", "weights16", "pairs"):
                        a_bits = getattr(other, name).view(torch.uint8)   # bytes: a NaN sum must compare equal too
                        assert torch.equal(a_bits, getattr(fused, name).view(torch.uint8)), (k, other.rs_mover, name)
                    assert other.sync_status() == (k + 1, 0)
                assert fused.sync_status() == (k + 1, 0)
                single.step_f16(H2.f16_bits(reduced.cpu()))
                a, b = fused.read_state(), nccl.read_state()
                for f in ("loss_scale", "inv_scale", "good_steps", "found_inf", "skipped", "step", "adam_t"):
                    assert getattr(a, f) == getattr(single.state, f) == getattr(b, f), (k, f)
                if k != 2:
                    assert abs(a.grad_norm - single.state.grad_norm) <= 1e-6 * single.state.grad_norm
                sl = slice(fused.begin, fused.end)
                assert H2.rel_err(single.master[sl], fused.master.cpu().numpy()) <= H2.STATE_TOL
                assert H2.rel_err(single.m[sl], fused.m.cpu().numpy()) <= H2.STATE_TOL
                assert H2.rel_err(single.v[sl], fused.v.cpu().numpy()) <= H2.STATE_TOL
                assert H2.half_ulp_distance(single.weights16, H2.f16_bits(fused.weights16.cpu())) <= 1
                assert H2.rel_err(nccl.master.cpu().numpy(), fused.master.cpu().numpy()) <= 1e-4
            except Exception:       # noqa: BLE001
                problem = traceback.format_exc()
            agree(problem is None, f"step {k} (checks)\n{problem or ''}")
        assert fused.read_state().skipped == 1
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_gpus_fused_step_matches_oracle_and_nccl_path(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_two_gpu_rank, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(2))
