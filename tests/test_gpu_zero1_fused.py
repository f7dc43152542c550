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
        g = (rng.standard_normal(n) * 1e-3 * scale).astype(np.float16)
        if poison is not None:
            g[poison] = np.float16(np.inf)
        return g.view(np.uint16)

    for trial, poison in enumerate((None, (world - 1, per * (world // 2) + 17))):
        arenas_bits = [rank_grads(r, poison[1] if poison and poison[0] == r else None) for r in range(world)]
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
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import helpers as H2
        from cuda_transformer_b200 import amp
        from cuda_transformer_b200.layout import CONFIGS, param_layout
        from oracle import ref_step as O
        slots = param_layout(CONFIGS["readme"])
        cfg = amp.make_schedule(growth_interval=2)
        fused = amp.FusedZero1Optimizer(slots, cfg, loss_scale=65536.0, history_len=16)
        nccl = amp.ShardedAmpOptimizer(slots, cfg, loss_scale=65536.0, history_len=16)
        gen = torch.Generator().manual_seed(0)
        init = torch.randn(fused.n_params, generator=gen) * 0.02
        fused.set_params(init)
        nccl.set_params(init)
        single = O.OracleStep(init.numpy(), fused.table, O.make_schedule(growth_interval=2), loss_scale=65536.0,
                              history_len=16)
        gen = torch.Generator().manual_seed(rank + 1)
        for k in range(4):
            scale = fused.read_state().loss_scale
            g = (torch.randn(fused.n, generator=gen) * 1e-3 * scale).half()
            if k == 2 and rank == 1:
                g[4242] = float("nan")
            fused.grads16.copy_(g)
            nccl.grads16.copy_(g)
            fused.optimizer_step()
            nccl.optimizer_step()
            torch.cuda.synchronize()
            reduced = torch.zeros(fused.n, dtype=torch.float16, device=fused.device)
            dist.all_gather_into_tensor(reduced, fused.grad_shard)          # test plumbing
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
