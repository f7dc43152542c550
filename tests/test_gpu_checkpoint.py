"""Resume through a GPTC v2 file on the GPU: N steps straight against N/2 + checkpoint + N/2 in a
fresh optimizer, as resume_checks of the reference (cuda/tests/test_checkpoint.cu:81-180) does.
The step is deterministic, so the two runs must agree bit for bit."""
import numpy as np
import pytest
import torch

import helpers as H
from inputs import GradStream

pytestmark = pytest.mark.gpu


def test_resume_from_checkpoint_is_bit_identical(tmp_path):
    from cuda_transformer_b200 import amp, checkpoint as ck
    from cuda_transformer_b200.layout import CONFIGS
    slots = H.debug_slots()
    shapes = H.debug_shapes()
    cfg = amp.make_schedule(lr=6e-4, min_lr=6e-5, warmup_steps=3, max_steps=40, grad_clip=0.25, growth_interval=3)
    init = torch.from_numpy(H.debug_init())
    shape = ck.ModelShape(4098, 4160, 64, 2, 4, 64, 1e-5)
    run = ck.RunInfo(B=4, max_steps=40, eval_every=10, warmup_steps=3, lr=6e-4, min_lr=6e-5, keep="10,20")

    def grads_for(stream, opt):
        g = stream.next_fp16_scaled(opt.read_state().loss_scale)
        flat = torch.cat([t.reshape(-1) for t in g])
        out = torch.zeros(opt.n, dtype=torch.float16)
        out[: opt.n_params] = flat
        return out

    straight = amp.AmpOptimizer(slots, cfg, loss_scale=65536.0, history_len=8)
    straight.set_params(init)
    stream = GradStream(shapes, seed=5)
    for k in range(8):
        g = grads_for(stream, straight)
        if k == 2:
            g[100] = float("inf")
        straight.grads16.copy_(g)
        straight.optimizer_step()

    first = amp.AmpOptimizer(slots, cfg, loss_scale=65536.0, history_len=8)
    first.set_params(init)
    stream = GradStream(shapes, seed=5)
    for k in range(4):
        g = grads_for(stream, first)
        if k == 2:
            g[100] = float("inf")
        first.grads16.copy_(g)
        first.optimizer_step()
    path = str(tmp_path / "resume.ckpt")
    ck.write_checkpoint(path, ck.checkpoint_of(first, shape, run))
    loaded = ck.read_checkpoint(path)
    assert bytes(loaded.state) == bytes(first.read_state()) and loaded.state.skipped == 1 and loaded.state.step == 4
    second = amp.AmpOptimizer(slots, cfg, loss_scale=1.0, history_len=8)
    ck.restore(second, loaded)
    assert torch.equal(second.weights16, first.weights16), "restore rebuilds the fp16 copy"
    for k in range(4, 8):
        second.grads16.copy_(grads_for(stream, second))
        second.optimizer_step()
    assert bytes(second.read_state()) == bytes(straight.read_state())
    for a, b in ((second.master, straight.master), (second.m, straight.m), (second.v, straight.v),
                 (second.weights16, straight.weights16)):
        assert torch.equal(a, b)
    st = second.read_state()
    assert st.step == 8 and st.adam_t == 7 and st.skipped == 1
    with pytest.raises(ck.CheckpointError):
        wrong = ck.read_checkpoint(path)
        wrong.params = wrong.params[:-8]
        ck.restore(second, wrong)


def test_weights_export_after_training_matches_the_reference_export(tmp_path):
    """After a few steps the fp16 arena, written as a float16 weights.bin, is byte for byte the
    file the reference's writer makes from the fp32 master (cuda/train_fast.cu:915 with fp16 on),
    and a fresh optimizer loaded from the fp32 file has the same master and fp16 copy."""
    import os
    import subprocess
    import sys
    from cuda_transformer_b200 import amp, checkpoint as ck, weights as wt
    slots = H.debug_slots()
    shapes = H.debug_shapes()
    cfg = amp.make_schedule(lr=6e-4, min_lr=6e-4, warmup_steps=0, max_steps=1 << 30)
    opt = amp.AmpOptimizer(slots, cfg, loss_scale=65536.0)
    opt.set_params(torch.from_numpy(H.debug_init()))
    stream = GradStream(shapes, seed=11)
    for _ in range(3):
        g = stream.next_fp16_scaled(opt.read_state().loss_scale)
        opt.grads16.zero_()
        opt.grads16[: opt.n_params].copy_(torch.cat([t.reshape(-1) for t in g]))
        opt.optimizer_step()
    shape = ck.ModelShape(4098, 4160, 64, 2, 4, 64, 1e-5)
    f32, f16 = str(tmp_path / "weights.bin"), str(tmp_path / "weights16.bin")
    wt.write_weights(f32, shape, opt.master)
    wt.write_weights(f16, shape, opt.weights16, fp16=True)
    back = wt.read_weights(f32)
    assert np.array_equal(back.params, opt.master[: opt.n_params].cpu().numpy())
    assert np.array_equal(wt.read_weights(f16).params, opt.weights16[: opt.n_params].float().cpu().numpy())
    fresh = amp.AmpOptimizer(slots, cfg, loss_scale=65536.0)
    wt.load_into(fresh, back)
    assert torch.equal(fresh.master, opt.master) and torch.equal(fresh.weights16, opt.weights16)
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
    import build_ref_tests
    tool = build_ref_tests.WEIGHTS_ROUNDTRIP
    if not os.path.exists(tool):
        pytest.skip("oracle/_ref/bin/weights_roundtrip was not built (no reference checkout at build time)")
    theirs = str(tmp_path / "theirs16.bin")
    proc = subprocess.run([tool, f32, theirs, "f16"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stderr
    assert open(theirs, "rb").read() == open(f16, "rb").read()
