"""The ZeRO-1 orchestration (cuda_transformer_b200.amp.Zero1Step) on CPU: two gloo ranks.

The collectives, the shard ranges, the rank-ordered reduction of {norm^2, flag} and the
in-place weight all-gather are the product's own code; only the three compute hooks are
bound to the CPU oracle here (on a GPU box they are the CUDA kernels, covered by the gpu
tests). The check: every rank ends with the state a single process computes from the
reduced gradients, and an overflow seen by one rank skips the step on all of them."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import helpers as H

WORLD = 2
STEPS = 5
BAD_STEP = 2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_class():
    from cuda_transformer_b200.amp import Zero1Step
    from oracle import ref_step as O

    class OracleZero1(Zero1Step):
        """Compute hooks on numpy through the oracle (tests only)."""

        def _oracle(self):
            cfg = O.Schedule.from_buffer_copy(bytes(self.sched))
            step = O.OracleStep(self.master.numpy(), self.table, cfg, eps=self.eps, arena_offset=self.begin)
            step.m, step.v = self.m.numpy(), self.v.numpy()
            step.master = self.master.numpy()
            step.weights16 = self.weights16[self.begin:self.end].view(torch.int16).numpy().view(np.uint16)
            step.state = O.StepState.from_buffer_copy(self.state.numpy().tobytes())
            return step

        def _put_state(self, step):
            self.state.copy_(torch.frombuffer(bytearray(bytes(step.state)), dtype=torch.uint8))

        def _pass1(self):
            s, bad = self._oracle().pass1_f16(H.f16_bits(self.grad_shard))
            self.sums_local[0] = s
            self.sums_local[1] = float(bad)

        def _finalize(self):
            step = self._oracle()
            pairs = self.sums_all.view(-1, 2).tolist()
            step.finalize_sums([(p[0], p[1] != 0.0) for p in pairs])
            self._put_state(step)

        def _pass2(self):
            self._oracle().pass2_f16(H.f16_bits(self.grad_shard))     # arrays are views: updated in place

        def _cast_weights(self, full_fp32):
            self.weights16.copy_(torch.from_numpy(O.float_to_half(full_fp32.numpy()).view(np.float16)))

    return OracleZero1, O


def _rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    try:
        from cuda_transformer_b200.amp import make_schedule
        OracleZero1, O = _make_class()
        slots = H.debug_slots()
        cfg = make_schedule(grad_clip=0.25, growth_interval=3)
        z = OracleZero1(slots, cfg, eps=1e-8, loss_scale=65536.0, history_len=16, device="cpu", group=None)
        init = torch.from_numpy(H.debug_init())
        z.set_params(init)
        assert z.n == 370_688 and z.n_local == z.n // world and z.begin == rank * z.n_local

        # the single-process answer, computed by every rank from the REDUCED gradients
        full_init = np.zeros(z.n, dtype=np.float32)
        full_init[: z.n_params] = H.debug_init()
        single = O.OracleStep(full_init, z.table, O.Schedule.from_buffer_copy(bytes(cfg)), eps=1e-8,
                              loss_scale=65536.0, history_len=16)
        gen = torch.Generator().manual_seed(rank + 1)
        for k in range(STEPS):
            scale = z.read_state().loss_scale
            g = (torch.randn(z.n, generator=gen) * 1e-3 * scale).half()
            g[z.n_params:] = 0
            if k == BAD_STEP and rank == 1:
                g[1234] = float("inf")              # rank 1 alone overflows, in rank 0's slice
            z.grads16.copy_(g)
            z.optimizer_step()
            reduced = torch.zeros(z.n, dtype=torch.float16)
            dist.all_gather_into_tensor(reduced, z.grad_shard)      # test plumbing: what the ranks stepped on
            single.step_f16(H.f16_bits(reduced))
            st = z.read_state()
            for f in ("loss_scale", "inv_scale", "good_steps", "found_inf", "skipped", "step", "adam_t"):
                assert getattr(st, f) == getattr(single.state, f), (k, f)
            assert abs(st.grad_norm - single.state.grad_norm) <= 1e-6 * abs(single.state.grad_norm) \
                or not np.isfinite(single.state.grad_norm)
            assert st.found_inf == (1 if k == BAD_STEP else 0)
            sl = slice(z.begin, z.end)
            assert H.rel_err(single.master[sl], z.master.numpy()) <= H.STATE_TOL
            assert H.rel_err(single.m[sl], z.m.numpy()) <= H.STATE_TOL
            assert H.rel_err(single.v[sl], z.v.numpy()) <= H.STATE_TOL
            # after the all-gather every rank holds every rank's fp16 weights
            assert H.half_ulp_distance(single.weights16, H.f16_bits(z.weights16)) <= 1
            # identical state bits on every rank
            mine = torch.frombuffer(bytearray(z.state.numpy().tobytes()), dtype=torch.uint8)
            both = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(both, mine)
            assert all(torch.equal(both[0], b) for b in both)
        # ---- sharded state -> one GPTC checkpoint -> back into fresh shards (cuda/checkpoint.cu:288-315)
        from cuda_transformer_b200 import checkpoint as ck
        full = ck.checkpoint_of(z, ck.ModelShape(4098, 4160, 64, 2, 4, 64, 1e-5), ck.RunInfo(B=4))
        assert full.params.size == z.n_params and bytes(full.state) == bytes(z.read_state())
        assert np.array_equal(full.m[z.begin:min(z.end, z.n_params)], z.m.numpy()[: max(0, min(z.end, z.n_params) - z.begin)])
        assert H.rel_err(single.master[: z.n_params], full.params) <= H.STATE_TOL
        path = os.path.join(out_dir, f"zero1_rank{rank}.ckpt")
        ck.write_checkpoint(path, full)
        z2 = OracleZero1(slots, cfg, eps=1e-8, loss_scale=1.0, history_len=16, device="cpu", group=None)
        ck.restore(z2, ck.read_checkpoint(path))
        g = (torch.randn(z.n, generator=gen) * 1e-3 * z.read_state().loss_scale).half()
        g[z.n_params:] = 0
        for o in (z, z2):
            o.grads16.copy_(g)
            o.optimizer_step()
        assert bytes(z.read_state()) == bytes(z2.read_state())
        assert torch.equal(z.master, z2.master) and torch.equal(z.m, z2.m) and torch.equal(z.v, z2.v)
        assert torch.equal(z.weights16, z2.weights16)
        z.write_state(full.state)       # the counters the assertions below look at
        st = z.read_state()
        assert st.skipped == 1 and st.adam_t == STEPS - 1 and st.loss_scale == 32768.0 and st.good_steps == 2
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_zero1_step_matches_single_process(tmp_path):
    mp.spawn(_rank_main, args=(WORLD, _free_port(), str(tmp_path)), nprocs=WORLD, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(WORLD))
