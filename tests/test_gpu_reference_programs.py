"""The reference's OWN test programs, unmodified, linked against libb200amp.so.

oracle/build_ref_tests.py compiles cuda/tests/test_fast.cu and cuda/tests/test_checkpoint.cu of
the reference with all of its model code (forward, backward, GEMMs, attention, checkpoint
files), once with the reference's own optimizer objects ("stock") and once with scaler.o,
adamw_multi.o and graph.o replaced by oracle/link_shim.cu over the library ("b200amp"). The
programs print a table of checks and exit non-zero on a failure (cuda/tests/test_fast.cu:44-52,
473-506). What is asserted here: every check that passes in the stock build passes with the
library underneath, and every check that touches the optimizer step passes outright.
Skipped where the binaries were not built (no reference checkout at build time)."""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OPTIMIZER_CHECKS = (
    "finite gradients: not skipped", "step 1, AdamW t 1", "S unchanged, 1 good step",
    "the fp16 weight copy is exactly fp16(params) after the step",
    "an inf gradient is found and the step is skipped", "AdamW t stays 0, the schedule step moves on",
    "the parameters did not move", "AdamW m did not move", "S halved",
    "the next step runs (t 1, step 2)", "and moves the parameters",
    "2 finite steps in a row: S doubles back to 65,536", "S = 2^30 overflows fp16: found and skipped",
    "S halved to 2^29", "capturing ran nothing", "both took 4 steps", "the graph replays give the eager losses",
    "every gradient is 0",
)


def _programs():
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import build_ref_tests
    if not build_ref_tests.available():
        pytest.skip("oracle/_ref test programs were not built (no reference checkout at build time)")
    return build_ref_tests.binaries(), build_ref_tests.DUMP


def _run(exe, dump, cwd):
    proc = subprocess.run([exe, dump], capture_output=True, text=True, timeout=900, cwd=cwd)
    lines = proc.stdout.splitlines()
    failed = [re.sub(r"\s+", " ", l).strip() for l in lines if l.rstrip().endswith("FAILED")]
    ok = [re.sub(r"\s+ok$", "", l).strip() for l in lines if l.rstrip().endswith(" ok")]
    return proc, failed, ok


@pytest.mark.parametrize("prog", ["test_fast", "test_checkpoint"])
def test_reference_program_passes_on_the_library(prog, tmp_path):
    bins, dump = _programs()
    stock, stock_failed, _ = _run(bins[f"{prog}_stock"], dump, tmp_path)
    ours, ours_failed, ours_ok = _run(bins[f"{prog}_b200amp"], dump, tmp_path)
    out_dir = os.environ.get("B200AMP_TEST_LOG_DIR") or str(tmp_path)     # keep the programs' full output
    os.makedirs(out_dir, exist_ok=True)
    for tag, proc in (("stock", stock), ("b200amp", ours)):
        with open(os.path.join(out_dir, f"ref_{prog}_{tag}.log"), "w") as f:
            f.write(proc.stdout + "\n---- stderr ----\n" + proc.stderr + f"\nexit {proc.returncode}\n")
    sys.stdout.write(ours.stdout[-6000:])
    assert ours.returncode in (0, 1), ours.stderr[-2000:]          # 0 all passed, 1 some table row failed
    new_failures = [f for f in ours_failed if f not in stock_failed]
    assert not new_failures, f"checks that pass with the reference's optimizer but fail on the library: {new_failures}"
    if stock.returncode == 0:
        assert ours.returncode == 0
    if prog == "test_fast":
        seen = " | ".join(ours_ok)
        for name in OPTIMIZER_CHECKS:
            assert name in seen, f"optimizer check did not pass: {name}"
    else:
        assert "FAILED" not in ours.stdout or stock.returncode != 0


def _train(exe, dump, tokens, out_dir, steps=60, extra=()):
    cmd = [exe, "-d", dump, "-D", tokens, "-n", str(steps), "-e", "20", "-b", "4", "-c", out_dir] + list(extra)
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    return proc


def _log_rows(path):
    rows = [line.rstrip("\n").split(",") for line in open(path)][1:]
    # step, train, val, lr, norm, ms, scale, skipped, counted, val_bpb: everything but the time
    return [[c for i, c in enumerate(r) if i != 5] for r in rows]


def test_reference_trainer_runs_on_the_library_and_trains_the_same(tmp_path):
    """The reference's whole training program (cuda/train_fast.cu: data batches, forward, backward,
    the optimizer step replayed as a CUDA Graph, evals, the per-step log from the history ring,
    GPTC checkpoints, weights.bin) linked against the library instead of its own scaler.o,
    adamw_multi.o and graph.o, on seeded random tokens: 60 steps, then 20 more continued from the
    checkpoint (--branch). It has to exit 0 and train the same: every logged column (loss, lr, norm,
    loss scale, skips) and the saved checkpoint and weights equal the stock program's bit for
    bit if two stock runs are themselves reproducible, else within the spread between them."""
    import numpy as np
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import build_ref_tests
    from cuda_transformer_b200 import checkpoint as ck, weights as wt
    if not build_ref_tests.trainer_available():
        pytest.skip("oracle/_ref/bin/train_fast_* were not built (no reference checkout at build time)")
    bins, dump, tokens = build_ref_tests.trainer_binaries(), build_ref_tests.DUMP, build_ref_tests.TOKENS
    out_dir = os.environ.get("B200AMP_TEST_LOG_DIR") or str(tmp_path)
    os.makedirs(out_dir, exist_ok=True)
    runs = {}
    for tag, exe in (("stock", bins["stock"]), ("stock_again", bins["stock"]), ("b200amp", bins["b200amp"])):
        d = str(tmp_path / tag)
        proc = _train(exe, dump, tokens, d)
        with open(os.path.join(out_dir, f"ref_train_fast_{tag}.log"), "w") as f:
            f.write(proc.stdout + "\n---- stderr ----\n" + proc.stderr + f"\nexit {proc.returncode}\n")
        assert proc.returncode == 0, f"{tag}: {proc.stdout[-2000:]}{proc.stderr[-2000:]}"
        assert "done   best val" in proc.stdout and "saved" in proc.stdout
        runs[tag] = dict(dir=d, rows=_log_rows(os.path.join(d, "fast_log.csv")),
                         ckpt=ck.read_checkpoint(os.path.join(d, "ckpt.bin")),
                         weights=wt.read_weights(os.path.join(d, "weights.bin")))
    sys.stdout.write(open(os.path.join(out_dir, "ref_train_fast_b200amp.log")).read()[-3000:])
    stock, again, ours = runs["stock"], runs["stock_again"], runs["b200amp"]
    assert len(ours["rows"]) == len(stock["rows"]) == 61                # the step-0 eval + 60 steps
    assert ours["ckpt"].state.step == 60 and bytes(ours["ckpt"].state)[:4] == bytes(stock["ckpt"].state)[:4]

    def spread(a, b):
        worst = 0.0
        for ra, rb in zip(a["rows"], b["rows"]):
            for i, (x, y) in enumerate(zip(ra, rb)):
                if x == y:
                    continue
                assert i in (1, 2, 4, 8), f"columns other than the losses and the norm differ: {ra} / {rb}"
                worst = max(worst, abs(float(x) - float(y)) / max(abs(float(y)), 1e-12))
        for name in ("params", "m", "v"):
            x, y = getattr(a["ckpt"], name), getattr(b["ckpt"], name)
            worst = max(worst, float(np.max(np.abs(x - y))) / max(float(np.max(np.abs(y))), 1e-30))
        return worst

    reproducible = spread(stock, again) == 0.0
    if reproducible:
        assert ours["rows"] == stock["rows"], "the training log differs from the stock program's"
        assert bytes(ours["ckpt"].state) == bytes(stock["ckpt"].state)
        for name in ("params", "m", "v"):
            assert np.array_equal(getattr(ours["ckpt"], name), getattr(stock["ckpt"], name)), name
        assert np.array_equal(ours["weights"].params, stock["weights"].params)
    else:
        assert spread(ours, stock) <= max(4 * spread(stock, again), 1e-5)
    print("stock runs reproducible:", reproducible, "| library vs stock spread:", spread(ours, stock))
    # continue each run from its own checkpoint for 20 more steps (--branch: the checkpoint's weights,
    # AdamW state, step and settings, cuda/train_fast.cu:84-86)
    for tag in ("stock", "b200amp"):
        branch_dir = runs[tag]["dir"] + "_branch"
        cmd = [bins[tag], "--branch", os.path.join(runs[tag]["dir"], "ckpt.bin"), "-n", "80", "-e", "20", "-c",
               branch_dir]
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
        with open(os.path.join(out_dir, f"ref_train_fast_{tag}_branch.log"), "w") as f:
            f.write(proc.stdout + "\n---- stderr ----\n" + proc.stderr + f"\nexit {proc.returncode}\n")
        assert proc.returncode == 0, f"{tag} branch: {proc.stdout[-2000:]}{proc.stderr[-2000:]}"
        runs[tag]["resumed"] = ck.read_checkpoint(os.path.join(branch_dir, "ckpt.bin"))
    a, b = runs["b200amp"]["resumed"], runs["stock"]["resumed"]
    assert a.state.step == 80 and b.state.step == 80 and a.state.skipped == b.state.skipped
    if reproducible:
        assert bytes(a.state) == bytes(b.state) and np.array_equal(a.params, b.params)
    # and the library's file is one our own reader, writer and the weights export agree on
    assert wt.read_weights(os.path.join(runs["b200amp"]["dir"] + "_branch", "weights.bin")).params.size == a.params.size


def test_reference_trainer_on_the_native_step_agrees_to_fp16_rounding_of_the_gradients(tmp_path):
    """The same trainer with the link shim built -DB200AMP_SHIM_NATIVE: its three optimizer calls
    become the fp32 -> fp16 bridge (pass 1 folded in, fp32 arena cleared behind it), the finalize
    on the bridge's sums and the native pass 2 on an fp16 gradient arena: the 30 B/param step
    (+ the bridge) under the reference's unmodified training program, replayed as a CUDA Graph.
    The optimizer then sees gradients rounded to fp16 (relative 5e-4 per element), so the run is
    held to the stock program's within that: same skip decisions and loss scale, losses within
    1e-3 relative, m and v within 1e-3 of their largest value. Parameters are held to 1e-3 of
    the largest: AdamW divides by sqrt(v), so an element whose gradient is so small that its fp16
    value has only a few significant bits moves by up to the learning rate per step either way
    (the reference notes the same about near-zero gradients, reference/dump.py:54-65)."""
    import numpy as np
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import build_ref_tests
    from cuda_transformer_b200 import checkpoint as ck
    bins = build_ref_tests.trainer_binaries()
    if not build_ref_tests.trainer_available() or not os.path.exists(bins["b200amp_native"]):
        pytest.skip("oracle/_ref/bin/train_fast_* were not built (no reference checkout at build time)")
    dump, tokens = build_ref_tests.DUMP, build_ref_tests.TOKENS
    out_dir = os.environ.get("B200AMP_TEST_LOG_DIR") or str(tmp_path)
    os.makedirs(out_dir, exist_ok=True)
    runs = {}
    for tag in ("stock", "b200amp_native"):
        d = str(tmp_path / tag)
        proc = _train(bins[tag], dump, tokens, d)
        with open(os.path.join(out_dir, f"ref_train_fast_{tag}_60.log"), "w") as f:
            f.write(proc.stdout + "\n---- stderr ----\n" + proc.stderr + f"\nexit {proc.returncode}\n")
        assert proc.returncode == 0, f"{tag}: {proc.stdout[-2000:]}{proc.stderr[-2000:]}"
        runs[tag] = dict(rows=_log_rows(os.path.join(d, "fast_log.csv")),
                         ckpt=ck.read_checkpoint(os.path.join(d, "ckpt.bin")))
    stock, ours = runs["stock"], runs["b200amp_native"]
    assert len(ours["rows"]) == len(stock["rows"]) == 61
    for ra, rb in zip(ours["rows"][1:], stock["rows"][1:]):
        assert ra[0] == rb[0] and ra[3] == rb[3] and ra[5:8] == rb[5:8], (ra, rb)    # step, lr, scale, skipped, counted
        assert abs(float(ra[1]) - float(rb[1])) <= 1e-3 * abs(float(rb[1])), (ra, rb)      # train loss
        assert abs(float(ra[4]) - float(rb[4])) <= 2e-3 * abs(float(rb[4])), (ra, rb)      # gradient norm
    a, b = ours["ckpt"], stock["ckpt"]
    assert (a.state.step, a.state.adam_t, a.state.skipped, a.state.loss_scale) == \
           (b.state.step, b.state.adam_t, b.state.skipped, b.state.loss_scale)
    worst = {}
    for name in ("params", "m", "v"):
        x, y = getattr(a, name), getattr(b, name)
        worst[name] = float(np.max(np.abs(x - y))) / float(np.max(np.abs(y)))
    print("native trainer vs stock after 60 steps, max |diff| / max |ref|:", worst)
    assert worst["params"] <= 1e-3 and worst["m"] <= 1e-3 and worst["v"] <= 1e-3
