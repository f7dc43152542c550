"""Runs the C++ host-layer test program (tests/cpp/test_amp_host.cpp) on the GPU."""
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
    assert [os.path.basename(e) for e in exes] == ["test_amp_host", "test_zero1_host", "peer_bandwidth"]
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
