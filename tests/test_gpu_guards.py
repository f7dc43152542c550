"""Out-of-bounds writes, caught without a sanitizer: every array a kernel may write sits between
two guard pads filled with a byte pattern, and the pads must be intact after each kernel family
has run on small, ragged and larger sizes (the native step in all its launch shapes incl. the
staged kernel, the compat launchers, the fp32 -> fp16 bridge, the fused ZeRO-1 kernels with
emulated ranks, the no-alloc pass 1). Reads past the end would not show here; the kernels' index
arithmetic for those is covered by the parity tests on the same sizes."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

PAD = 4096              # bytes on each side
PATTERN = 0xA5


class Guarded:
    """A device array of `count` elements of `dtype` between two pads."""

    def __init__(self, count, dtype, fill=None):
        item = torch.empty((), dtype=dtype).element_size()
        self.bytes = count * item
        self.raw = torch.full((PAD + self.bytes + PAD,), PATTERN, dtype=torch.uint8, device="cuda")
        self.t = self.raw[PAD:PAD + self.bytes].view(dtype)
        if fill is None:
            self.t.zero_()
        else:
            self.t.copy_(fill)

    def intact(self):
        head, tail = self.raw[:PAD], self.raw[PAD + self.bytes:]
        return bool((head == PATTERN).all()) and bool((tail == PATTERN).all())


def _state(amp, scale=65536.0):
    return Guarded(60, torch.uint8, torch.frombuffer(bytearray(bytes(amp.initial_state(scale))), dtype=torch.uint8))


def _table(amp, n):
    from cuda_transformer_b200._lib import TensorInfo
    cut = max(4, n // 3 // 4 * 4)
    rows = [(0, cut, 1), (cut, n - cut, 0)] if n > cut else [(0, n, 1)]
    arr = (TensorInfo * len(rows))(*[TensorInfo(o, c, d) for o, c, d in rows])
    return torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).cuda(), len(rows)


@pytest.mark.parametrize("n", [8, 16 * 37, 8 * 1024 + 8, (1 << 20) + 32])
def test_no_kernel_writes_outside_its_arrays(n):
    from cuda_transformer_b200 import _lib, amp
    lib = _lib.load()
    rng = np.random.default_rng(n)
    cfg = amp.make_schedule()
    g16_host = torch.from_numpy((rng.standard_normal(n) * 1e-3 * 65536.0).astype(np.float16))
    master = Guarded(n, torch.float32, torch.from_numpy((rng.standard_normal(n) * 0.02).astype(np.float32)))
    m, v = Guarded(n, torch.float32), Guarded(n, torch.float32)
    w16, g16 = Guarded(n, torch.float16), Guarded(n, torch.float16, g16_host)
    g32 = Guarded(n, torch.float32, g16_host.float())
    state, history = _state(amp), Guarded(60 * 4, torch.uint8)
    ws = Guarded(lib.b200amp_workspace_bytes(), torch.uint8)
    partial = Guarded(512, torch.float32)
    sums = Guarded(2, torch.float64)
    tensors, ntensors = _table(amp, n)
    everything = dict(master=master, m=m, v=v, w16=w16, g16=g16, g32=g32, state=state, history=history, ws=ws,
                      partial=partial, sums=sums)

    def check(what):
        torch.cuda.synchronize()
        broken = [name for name, g in everything.items() if not g.intact()]
        assert not broken, f"{what}: wrote outside {broken}"

    # native step in every launch shape
    knobs = [dict(pass2_variant=0, pass2_threads=256, pass2_blocks_per_sm=2, pass1_blocks_per_sm=4),
             dict(pass2_variant=0, pass2_threads=512, pass2_blocks_per_sm=1, pass1_blocks_per_sm=1),
             dict(pass2_variant=0, pass2_threads=1024, pass2_blocks_per_sm=1, pass1_blocks_per_sm=32),
             dict(pass2_variant=1, pass2_stages=3), dict(pass2_variant=1, pass2_stages=7)]
    saved = {}
    for key in {k for kn in knobs for k in kn}:
        val = C.c_int()
        _lib.check(lib.b200amp_tune_get(key.encode(), C.byref(val)))
        saved[key] = val.value
    try:
        for kn in knobs:
            for key, val in kn.items():
                _lib.check(lib.b200amp_tune_set(key.encode(), val))
            amp.step_f16(master.t, m.t, v.t, g16.t, w16.t, n, tensors, ntensors, state.t, ws.t, cfg, history.t, 4,
                         cfg.beta1, cfg.beta2, 1e-8)
            check(f"native step {kn}")
    finally:
        for key, val in saved.items():
            lib.b200amp_tune_set(key.encode(), val)
    # compat launchers (the reference's arguments)
    amp.begin_step(state.t)
    amp.unscale_and_norm(g32.t, n, state.t, partial.t)
    amp.finalize_step(state.t, partial.t, cfg, history.t, 4)
    amp.adamw_multi(master.t, w16.t, g32.t, m.t, v.t, n, tensors, ntensors, state.t, cfg.beta1, cfg.beta2, 1e-8)
    amp.cast_to_x(w16.t, master.t, n)
    check("compat launchers")
    # the bridge, clearing its source, and the no-alloc pass 1
    g32.t.copy_(g16_host.float())
    amp.cast_pass1_f32(g32.t, g16.t, n, True, state.t, ws.t, cfg, history.t, 4)
    amp.pass1_f16_static(g16.t, n, state.t, sums.t)
    check("bridge and static pass 1")
    # fused ZeRO-1 kernels, 2 emulated ranks (needs two whole 8-element groups per rank)
    if n % 16 == 0:
        per = n // 2
        peer_g = Guarded(n, torch.float16, g16_host)
        peer_w = Guarded(n, torch.float16)
        reduced = Guarded(per, torch.float16)
        pairs = [Guarded(4, torch.float64), Guarded(4, torch.float64)]
        everything.update(peer_g=peer_g, peer_w=peer_w, reduced=reduced, pairs0=pairs[0], pairs1=pairs[1])
        for r in range(2):
            src = [g16.t.data_ptr() + 2 * r * per, peer_g.t.data_ptr() + 2 * r * per]
            amp.rs_pass1_f16(src, r, reduced.t, per, state.t, ws.t, [p.t.data_ptr() for p in pairs])
            amp.finalize_sums(state.t, pairs[r].t, 2, cfg, history.t, 4)
            dst = [w16.t.data_ptr() + 2 * r * per, peer_w.t.data_ptr() + 2 * r * per]
            sl = slice(r * per, (r + 1) * per)
            amp.pass2_ag_f16(master.t[sl], m.t[sl], v.t[sl], reduced.t, dst, per, r * per, tensors, ntensors, state.t,
                             cfg.beta1, cfg.beta2, 1e-8)
            check(f"fused ZeRO-1 kernels, rank {r}")
    flag = C.c_int(-1)
    _lib.check(lib.b200amp_device_error(C.byref(flag)))
    assert flag.value == 0
