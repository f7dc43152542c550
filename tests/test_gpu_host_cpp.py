"""Runs the C++ host-layer test programs (tests/cpp/) on the GPU."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "cpp"))


def test_cpp_host_program_builds():
    """CPU-side: the reference-signature shim and the C++ owner class compile and link against
    the library (nvcc cross-compiles without a GPU)."""
    import build_host_test
    from cuda_transformer_b200 import build as lib_build
    lib_build.build()
    exes = build_host_test.build_all()
    want = ["test_amp_host", "test_zero1_host", "peer_bandwidth"]
    if build_host_test.nccl_paths() is not None:
        want.append("test_zero1_nccl_host")
    assert [os.path.basename(e) for e in exes] == want
    assert all(os.path.exists(e) for e in exes)


@pytest.mark.gpu
def test_cpp_host_program_checks_pass():
    import build_host_test
    exe = build_host_test.build()
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    sys.stdout.write(proc.stdout)
    sys.stderr.write(proc.stderr)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    assert "all checks passed" in proc.stdout and "FAILED" not in proc.stdout


@pytest.mark.gpu
def test_cpp_zero1_host_program_checks_pass():
    """One process, R = 1, 2, 4, 8 ranks over the GPUs present (all on one GPU where there is one),
    events between the phases, against the one-GPU step on the averaged gradients."""
    import build_host_test
    exe = build_host_test.build(program="test_zero1_host")
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    sys.stdout.write(proc.stdout)
    sys.stderr.write(proc.stderr)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    assert "all checks passed" in proc.stdout and "FAILED" not in proc.stdout
    assert proc.stdout.count(" ok\n") == 4 * 10


@pytest.mark.gpu
def test_peer_bandwidth_program_reports_sane_nvlink_figures():
    """tests/cpp/peer_bandwidth.cu: on one GPU it says so and measures nothing; on two or more every
    mover's figure must be a plausible NVLink rate and the copied bytes must have arrived; on four
    or eight the all-to-all table of the ZeRO-1 pattern must be there too."""
    import re

    import torch

    import build_host_test
    exe = build_host_test.build(program="peer_bandwidth")
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    sys.stdout.write(proc.stdout)
    sys.stderr.write(proc.stderr)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    count = torch.cuda.device_count()
    if count < 2:
        assert "nothing measured" in proc.stdout
        return
    if "cannot map" in proc.stdout:
        return
    rows = re.findall(r"^(copy engine|SM ld / st \(256-bit\)|bulk through shared memory)\s+(read|write)\s+"
                      r"([0-9.]+)\s+([0-9.]+) \|\s+([0-9.]+)", proc.stdout, re.M)
    assert len(rows) == 6, proc.stdout
    for name, way, one, both0, both1 in rows:
        assert all(200.0 < float(x) < 1000.0 for x in (one, both0, both1)), (name, way, one, both0, both1)
    assert "expected 2 and 1" in proc.stdout
    if count >= 4:
        table = re.findall(r"^all-to-all R=(\d) (.{28})\s+([0-9.]+) \.\.\s+([0-9.]+)", proc.stdout, re.M)
        assert len(table) >= 4, proc.stdout
        for r, label, lo, hi in table:
            assert 100.0 < float(lo) <= float(hi) < 1000.0, (r, label, lo, hi)


@pytest.mark.gpu
def test_cpp_zero1_nccl_host_program_checks_pass():
    """One process, NCCL around the passes (ncclCommInitAll), R = 2, 4, 8 ranks on as many distinct
    GPUs as the machine has; with one GPU the program says so and checks nothing."""
    import torch

    import build_host_test
    if build_host_test.nccl_paths() is None:
        pytest.skip("no NCCL headers and library in this environment")
    exe = build_host_test.build(program="test_zero1_nccl_host")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([exe], capture_output=True, text=True, timeout=900, env=env)
    sys.stdout.write(proc.stdout)
    sys.stderr.write(proc.stderr)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    if torch.cuda.device_count() < 2:
        assert "nothing to check" in proc.stdout
        return
    assert "all checks passed" in proc.stdout and "FAILED" not in proc.stdout
    groups = sum(1 for r in (2, 4, 8) if r <= torch.cuda.device_count())
    assert proc.stdout.count(" ok\n") == groups * 11
