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
