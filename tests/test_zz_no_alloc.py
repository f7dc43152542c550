"""b200amp_pass1_f16_static: pass 1 for callers that cannot allocate device memory (all of it
went to their own arenas at start-up, they live inside someone else's memory pool, or they
cannot afford cudaMalloc's device-wide synchronisation inside the step loop). Its scratch is an
array inside the library image, shared by every call on the device.

Checked here through the C ABI: two calls in a row give exactly the {sum of squares, flag} pair
that the workspace-taking entry point b200amp_pass1_f16 gives on the same gradients (same
summation order, so the comparison is bit for bit; the parity tests allow 1e-6 on the norm
elsewhere), the second call is not disturbed by what the first left in the shared array, and a
size beyond the stated maximum is refused without touching the GPU.

This file sorts last on purpose, so a run that stops at the first failure has already run
every other test. It passes alone in a fresh process and after the rest of the suite."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(n, seed, loss_scale, poison=None):
    gen = torch.Generator().manual_seed(seed)
    g = (torch.randn(n, generator=gen) * 1e-3 * loss_scale).half()
    if poison is not None:
        g[poison] = float("inf")
    return g.cuda()


def test_static_scratch_pass1_matches_workspace_pass1_twice_in_a_row():
    from cuda_transformer_b200 import _lib, amp
    lib = _lib.load()
    _lib.check(lib.b200amp_device_check())
    n = (1 << 22) + 8 * 123                      # a ragged last virtual block
    loss_scale = 65536.0
    state = torch.frombuffer(bytearray(bytes(amp.initial_state(loss_scale))), dtype=torch.uint8).cuda()
    workspace = torch.zeros(lib.b200amp_workspace_bytes(), dtype=torch.uint8, device="cuda")
    out = torch.full((2,), -1.0, dtype=torch.float64, device="cuda")

    calls = [(_inputs(n, 1, loss_scale), 0.0), (_inputs(n, 2, loss_scale, poison=n - 5), 1.0)]
    for grads, want_flag in calls:
        amp.pass1_f16(grads, n, state, workspace)                   # the existing entry point
        want = workspace[:16].view(torch.float64).clone()
        out.fill_(-1.0)
        amp.pass1_f16_static(grads, n, state, out)                  # the one that brings its own scratch
        torch.cuda.synchronize()
        got, ref = out.cpu().numpy(), want.cpu().numpy()
        assert got[1] == ref[1] == want_flag
        if want_flag == 0.0:
            assert got[0] == ref[0], (got[0], ref[0])               # same order of additions: same bits
            exact = float((grads.double() / loss_scale).pow(2).sum())
            assert abs(got[0] - exact) <= 1e-6 * exact
        else:
            assert np.isinf(got[0]) and np.isinf(ref[0])

    # a third call after the poisoned one: the flag left in the shared array must not leak
    amp.pass1_f16_static(calls[0][0], n, state, out)
    torch.cuda.synchronize()
    assert out.cpu().numpy()[1] == 0.0


def test_static_scratch_pass1_refuses_sizes_beyond_its_maximum():
    from cuda_transformer_b200 import _lib, amp
    lib = _lib.load()
    small = torch.zeros(8, dtype=torch.float16, device="cuda")
    state = torch.frombuffer(bytearray(bytes(amp.initial_state(1.0))), dtype=torch.uint8).cuda()
    out = torch.zeros(2, dtype=torch.float64, device="cuda")
    status = lib.b200amp_pass1_f16_static(small.data_ptr(), (1 << 32) + 8, state.data_ptr(), out.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    assert status == _lib.ERR_LIMIT
    assert b"beyond" in lib.b200amp_last_error()
    with pytest.raises(amp.B200AmpError):
        amp.pass1_f16_static(small, 8, state, None)                 # no output buffer
    amp.pass1_f16_static(small, 8, state, out)                      # and the smallest size works
    torch.cuda.synchronize()
    assert out.cpu().tolist() == [0.0, 0.0]


def test_static_scratch_pass1_refused_calls_leave_the_stream_and_the_scratch_alone():
    """A call with a bad size, a null or a misaligned pointer is refused before anything is
    enqueued: the answer of the next good call is what it would have been without them."""
    from cuda_transformer_b200 import amp
    n = 1 << 16
    grads = _inputs(n, 3, 1024.0)
    state = torch.frombuffer(bytearray(bytes(amp.initial_state(1024.0))), dtype=torch.uint8).cuda()
    out = torch.full((2,), -1.0, dtype=torch.float64, device="cuda")
    amp.pass1_f16_static(grads, n, state, out)
    torch.cuda.synchronize()
    want = out.cpu().numpy().copy()
    out.fill_(-1.0)
    torch.cuda.synchronize()
    for bad_call in (lambda: amp.pass1_f16_static(grads, 0, state, out),
                     lambda: amp.pass1_f16_static(grads, n + 4, state, out),
                     lambda: amp.pass1_f16_static(None, n, state, out),
                     lambda: amp.pass1_f16_static(grads, n, None, out),
                     lambda: amp.pass1_f16_static(grads.data_ptr() + 2, n - 8, state, out)):
        with pytest.raises(amp.B200AmpError):
            bad_call()
    torch.cuda.synchronize()
    assert out.cpu().tolist() == [-1.0, -1.0], "a refused call wrote its output"
    amp.pass1_f16_static(grads, n, state, out)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want)


def test_static_scratch_pass1_on_a_second_device():
    """Each GPU holds its own copy of the array, looked up with that GPU current."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from cuda_transformer_b200 import _lib, amp
    lib = _lib.load()
    n = 1 << 18
    host = _inputs(n, 4, 2048.0).cpu()
    answers = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            grads = host.to(f"cuda:{dev}")
            state = torch.frombuffer(bytearray(bytes(amp.initial_state(2048.0))), dtype=torch.uint8).to(f"cuda:{dev}")
            workspace = torch.zeros(lib.b200amp_workspace_bytes(), dtype=torch.uint8, device=f"cuda:{dev}")
            out = torch.zeros(2, dtype=torch.float64, device=f"cuda:{dev}")
            amp.pass1_f16(grads, n, state, workspace)
            amp.pass1_f16_static(grads, n, state, out)
            torch.cuda.synchronize()
            assert torch.equal(out, workspace[:16].view(torch.float64))
            answers.append(out.cpu().numpy())
    assert np.array_equal(answers[0], answers[1])
