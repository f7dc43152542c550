"""GPTC v2 checkpoints (cuda_transformer_b200/checkpoint.py) on the CPU: round trip, the
reference's error cases (cuda/tests/test_checkpoint.cu:165-177: truncated and foreign files),
atomic replace, and - where the reference checkout was present at build time - a file written
here is read by the REFERENCE's reader and written back by its writer byte for byte."""
import os
import subprocess
import sys

import numpy as np
import pytest

from cuda_transformer_b200 import checkpoint as ck
from cuda_transformer_b200._lib import StepState

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _sample(n=1000, seed=0) -> ck.Checkpoint:
    rng = np.random.default_rng(seed)
    st = StepState()
    st.loss_scale, st.inv_scale, st.good_steps, st.skipped = 32768.0, 1.0 / 32768.0, 17, 3
    st.step, st.adam_t, st.lr, st.grad_norm, st.clip_coef = 120, 117, 5.5e-4, 3.25, 0.3
    st.step_size, st.bc2_sqrt, st.decay, st.loss, st.n_valid = 6e-4, 0.99, 0.99994, 4.125, 256
    return ck.Checkpoint(
        ck.ModelShape(4098, 4160, 64, 2, 4, 64, 1e-5),
        ck.RunInfo(B=16, max_steps=5000, eval_every=250, warmup_steps=200, sft=0, lr=6e-4, min_lr=6e-5,
                   data="data/chat/pretrain", starts="", decay_steps=400, beta2=0.95, keep="97600,195200",
                   branch="ckpt/base.ckpt", best_val=3.875, best_step=100),
        st, rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32),
        rng.random(n).astype(np.float32))


def _f32(x):
    return float(np.float32(x)) if isinstance(x, float) else x


def _fields(obj) -> dict:
    return {k: _f32(v) for k, v in vars(obj).items()}      # the file holds float32: compare at that precision


def _same(a: ck.Checkpoint, b: ck.Checkpoint) -> bool:
    return (_fields(a.cfg) == _fields(b.cfg) and _fields(a.run) == _fields(b.run)
            and bytes(a.state) == bytes(b.state)
            and np.array_equal(a.params, b.params) and np.array_equal(a.m, b.m) and np.array_equal(a.v, b.v))


def test_round_trip_and_layout(tmp_path):
    c = _sample()
    path = str(tmp_path / "a.ckpt")
    ck.write_checkpoint(path, c)
    assert not os.path.exists(path + ".tmp")
    raw = open(path, "rb").read()
    assert raw[:4] == b"GPTC" and int.from_bytes(raw[4:8], "little") == 2
    assert int.from_bytes(raw[72:76], "little") == 60            # sizeof(StepState) sits after 8 + 28 + 36 bytes
    assert raw[76:136] == bytes(c.state)
    assert len(raw) == 136 + (4 + 18) + 4 + 8 + (4 + 12) + (4 + 14) + 8 + 12 * 1000
    assert _same(ck.read_checkpoint(path), c)
    # a second write replaces the file in one step
    c2 = _sample(seed=1)
    ck.write_checkpoint(path, c2)
    assert _same(ck.read_checkpoint(path), c2)


def test_bad_files_are_refused(tmp_path):
    c = _sample()
    path = str(tmp_path / "a.ckpt")
    ck.write_checkpoint(path, c)
    raw = open(path, "rb").read()
    cut = str(tmp_path / "cut.ckpt")
    open(cut, "wb").write(raw[:len(raw) // 2])
    with pytest.raises(ck.CheckpointError):
        ck.read_checkpoint(cut)
    foreign = str(tmp_path / "foreign.ckpt")
    open(foreign, "wb").write(b"GPTW" + raw[4:])
    with pytest.raises(ck.CheckpointError, match="not a GPTC"):
        ck.read_checkpoint(foreign)
    future = str(tmp_path / "v9.ckpt")
    open(future, "wb").write(raw[:4] + (9).to_bytes(4, "little") + raw[8:])
    with pytest.raises(ck.CheckpointError, match="version 9"):
        ck.read_checkpoint(future)
    other_state = str(tmp_path / "state.ckpt")
    open(other_state, "wb").write(raw[:72] + (64).to_bytes(4, "little") + raw[76:])
    with pytest.raises(ck.CheckpointError, match="StepState"):
        ck.read_checkpoint(other_state)
    with pytest.raises(ck.CheckpointError):
        ck.read_checkpoint(str(tmp_path / "missing.ckpt"))
    bad = _sample()
    bad.m = bad.m[:-1]
    with pytest.raises(ck.CheckpointError):
        ck.write_checkpoint(str(tmp_path / "b.ckpt"), bad)


def test_version_1_files_still_read(tmp_path):
    c = _sample()
    path = str(tmp_path / "a.ckpt")
    ck.write_checkpoint(path, c)
    raw = open(path, "rb").read()
    head = 136 + (4 + 18) + 4                         # through the starts string
    v2_extra = 8 + (4 + 12) + (4 + 14)                # decay_steps, beta2, keep, branch
    v1 = raw[:4] + (1).to_bytes(4, "little") + raw[8:head] + raw[head + v2_extra:]
    p1 = str(tmp_path / "v1.ckpt")
    open(p1, "wb").write(v1)
    got = ck.read_checkpoint(p1)
    assert got.run.decay_steps == 0 and got.run.beta2 == 0.95 and got.run.keep == "" and got.run.branch == ""
    assert np.array_equal(got.v, c.v) and bytes(got.state) == bytes(c.state)


def test_reference_reader_and_writer_reproduce_our_file(tmp_path):
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import build_ref_tests
    if not os.path.exists(build_ref_tests.ROUNDTRIP):
        pytest.skip("oracle/_ref/bin/ckpt_roundtrip was not built (no reference checkout at build time)")
    c = _sample(n=4096, seed=3)
    ours, theirs = str(tmp_path / "ours.ckpt"), str(tmp_path / "theirs.ckpt")
    ck.write_checkpoint(ours, c)
    proc = subprocess.run([build_ref_tests.ROUNDTRIP, ours, theirs], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stderr
    assert "step 120 adam_t 117 loss_scale 32768 n 4096 keep '97600,195200'" in proc.stdout
    assert open(ours, "rb").read() == open(theirs, "rb").read()
    assert _same(ck.read_checkpoint(theirs), c)
    # and the reference's reader refuses what ours refuses
    cut = str(tmp_path / "cut.ckpt")
    open(cut, "wb").write(open(ours, "rb").read()[:500])
    proc = subprocess.run([build_ref_tests.ROUNDTRIP, cut, theirs], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 1
