"""CPU-only checks of the boundary: the shared library loads, exports every symbol the header
declares, the host-only entry points behave, and the arena layout has the reference's sizes.
No kernel is launched here."""
import ctypes as C
import os
import re

import pytest

from cuda_transformer_b200 import _lib, build
from cuda_transformer_b200.layout import CONFIGS, num_params, padded, param_layout, shard_range, tensor_table

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(REPO, "include", "b200amp.h")).read()
    return sorted(set(re.findall(r"B200AMP_API[^;(]*?\b(b200amp_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_library_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) >= 24
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/b200amp.h but not exported"
    assert sorted(_lib.PROTOTYPES) == names, "the ctypes prototypes and the header disagree"


def test_struct_layouts_are_the_reference_abi():
    assert C.sizeof(_lib.StepState) == 60       # cuda/kernels/fast.h:104-121; checkpoint ABI, cuda/checkpoint.cu:102-103
    assert C.sizeof(_lib.ScheduleConfig) == 44  # cuda/kernels/fast.h:123-133
    assert C.sizeof(_lib.TensorInfo) == 24      # cuda/kernels/fast.h:153-158
    assert _lib.StepState.loss_scale.offset == 0 and _lib.StepState.found_inf.offset == 12
    assert _lib.StepState.adam_t.offset == 24 and _lib.StepState.n_valid.offset == 56
    assert _lib.TensorInfo.decay.offset == 16


def test_host_only_entry_points(lib):
    assert re.fullmatch(r"\d+\.\d+\.\d+", lib.b200amp_version().decode())
    st = _lib.StepState()
    assert lib.b200amp_initial_state(65536.0, C.byref(st)) == _lib.OK
    assert st.loss_scale == 65536.0 and st.inv_scale == 1.0 / 65536.0
    assert st.clip_coef == 1.0 and st.decay == 1.0
    assert (st.good_steps, st.found_inf, st.skipped, st.step, st.adam_t, st.n_valid) == (0,) * 6
    assert lib.b200amp_initial_state(1.0, None) == _lib.ERR_ARG
    assert b"null" in lib.b200amp_last_error()
    assert lib.b200amp_workspace_bytes() >= 16 + 8 * 148 * 32


def test_tuning_knobs_round_trip(lib):
    v = C.c_int()
    assert lib.b200amp_tune_get(b"pass2_blocks_per_sm", C.byref(v)) == _lib.OK
    old = v.value
    assert lib.b200amp_tune_set(b"pass2_blocks_per_sm", 6) == _lib.OK
    assert lib.b200amp_tune_get(b"pass2_blocks_per_sm", C.byref(v)) == _lib.OK and v.value == 6
    assert lib.b200amp_tune_set(b"pass2_blocks_per_sm", old) == _lib.OK
    assert lib.b200amp_tune_set(b"pass2_blocks_per_sm", 0) == _lib.ERR_ARG
    assert lib.b200amp_tune_set(b"no_such_knob", 1) == _lib.ERR_ARG


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(build, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


@pytest.mark.parametrize("name,n,n_pad,ntensors", [
    ("debug", 370_432, 370_688, 28),
    ("readme", 12_343_296, 12_343_296, 76),
    ("gpt2-small", 124_475_904, 124_476_416, 148),
    ("1.3b", 1_315_819_520, 1_315_819_520, 292),
])
def test_arena_layout_sizes(name, n, n_pad, ntensors):
    """n = Vp*C + n_ctx*C + L*(12C^2 + 13C) + 2C (cuda/gpt.cu:82-101)."""
    cfg = CONFIGS[name]
    slots = param_layout(cfg)
    C_ = cfg.C
    assert num_params(slots) == n == cfg.Vp * C_ + cfg.n_ctx * C_ + cfg.L * (12 * C_ * C_ + 13 * C_) + 2 * C_
    assert padded(n) == n_pad and len(slots) == ntensors <= 1024
    at = 0
    for s in slots:
        assert s.offset == at and s.offset % 8 == 0 and s.count % 8 == 0   # cuda/gpt_fast.cu:111
        at += s.count
    table = tensor_table(slots)
    assert [d for _, _, d in table[:4]] == [1, 1, 0, 0]      # wte, wpe decay; ln1.w, ln1.b do not
    assert sum(d for _, _, d in table) == 2 + 4 * cfg.L


def test_shard_ranges_tile_the_arena():
    n = padded(124_475_904)
    for world in (1, 2, 4, 8):
        at = 0
        for r in range(world):
            b, e = shard_range(n, r, world)
            assert b == at and (e - b) % 128 == 0
            at = e
        assert at == n


def test_tensor_table_check_is_host_only_and_strict(lib):
    """b200amp_check_tensor_table: what the kernels assume about the table, checked once on the host."""
    from cuda_transformer_b200 import amp

    def status(rows, n=0):
        arr = (_lib.TensorInfo * max(1, len(rows)))(*[_lib.TensorInfo(o, c, d) for o, c, d in rows])
        return lib.b200amp_check_tensor_table(C.cast(arr, C.c_void_p), len(rows), n), lib.b200amp_last_error().decode()

    for name, cfg in CONFIGS.items():
        slots = param_layout(cfg)
        assert status(list(tensor_table(slots)), padded(num_params(slots)))[0] == _lib.OK, name
    assert status([(0, 8, 1), (8, 4, 0), (12, 4, 1)], 16)[0] == _lib.OK
    assert status([(0, 8, 1), (12, 4, 0)], 16)[0] == _lib.OK                  # a hole between tensors is allowed
    bad = {
        "no entries": ([], 0),
        "offset 6": ([(6, 8, 1)], 0),
        "negative offset": ([(-4, 8, 1)], 0),
        "empty tensor": ([(0, 0, 1)], 0),
        "overlap": ([(0, 12, 1), (8, 4, 0)], 0),
        "descending": ([(8, 4, 1), (0, 4, 0)], 0),
        "past the arena": ([(0, 8, 1), (8, 12, 0)], 16),
        "decay flag 2": ([(0, 8, 2)], 0),
    }
    for name, (rows, n) in bad.items():
        code, text = status(rows, n)
        assert code == _lib.ERR_ARG and text.startswith("tensor table"), (name, code, text)
    assert lib.b200amp_check_tensor_table(None, 1, 0) == _lib.ERR_ARG
    too_many = [(4 * k, 4, k % 2) for k in range(1025)]
    assert status(too_many)[0] == _lib.ERR_ARG
    with pytest.raises(amp.B200AmpError, match="reaches into"):
        amp.check_tensor_table([(0, 12, 1), (8, 4, 0)])
    amp.check_tensor_table([(0, 8, 1), (8, 8, 0)], 16)


def test_new_struct_sizes_match_the_header_as_a_c_compiler_sees_it(tmp_path):
    """b200amp_zero1_sync and b200amp_decay_runs cross the ABI by pointer from ctypes: their
    ctypes mirrors must have the size and field offsets gcc gives the header's structs."""
    import subprocess
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "b200amp.h"\n'
                   'int main(void) { printf("%zu %zu %zu %zu %zu %d %d\\n", sizeof(b200amp_zero1_sync), '
                   'offsetof(b200amp_zero1_sync, wait_limit), sizeof(b200amp_decay_runs), '
                   'offsetof(b200amp_decay_runs, nruns), offsetof(b200amp_decay_runs, flag0), '
                   'B200AMP_ZERO1_SYNC_BYTES, B200AMP_MAX_RUNS); return 0; }\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", os.path.join(REPO, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert got == [C.sizeof(_lib.Zero1Sync), _lib.Zero1Sync.wait_limit.offset, C.sizeof(_lib.DecayRuns),
                   _lib.DecayRuns.nruns.offset, _lib.DecayRuns.flag0.offset, _lib.ZERO1_SYNC_BYTES, 256]


def test_decay_runs_builder_merges_neighbours_with_equal_flags(lib):
    from cuda_transformer_b200 import amp
    runs = amp.decay_runs_build([(0, 8, 1), (8, 8, 1), (16, 4, 0), (20, 4, 0), (32, 8, 1)])
    assert (runs.nruns, runs.flag0, list(runs.first4[:3])) == (3, 1, [0, 4, 8])
    runs = amp.decay_runs_build([(8, 8, 0)])
    assert (runs.nruns, runs.flag0, runs.first4[0]) == (1, 0, 2)
    for name, cfg in CONFIGS.items():
        slots = param_layout(cfg)
        r = amp.decay_runs_build(list(tensor_table(slots)))
        assert r.nruns == 8 * cfg.L + 2 and r.flag0 == 1, name          # wte+wpe | per layer 8 | ln_f joins the last run
    with pytest.raises(amp.B200AmpError) as err:
        amp.decay_runs_build([(4 * k, 4, k % 2) for k in range(257)])
    assert err.value.status == _lib.ERR_LIMIT
    with pytest.raises(amp.B200AmpError, match="tensor table"):
        amp.decay_runs_build([(0, 12, 1), (8, 4, 0)])                      # checked like any table


def test_pass1_partition_is_a_function_of_n_alone(lib):
    from cuda_transformer_b200 import amp
    assert amp.pass1_partition(8) == (1, 8192)
    assert amp.pass1_partition(8192 * 14 - 8) == (14, 8192)
    vblocks, per = amp.pass1_partition(1_315_819_520)
    assert vblocks <= 4736 and per % 8192 == 0 and (vblocks - 1) * per < 1_315_819_520 <= vblocks * per
    with pytest.raises(amp.B200AmpError):
        amp.pass1_partition(12)


def test_self_ordering_entry_points_refuse_bad_arguments_before_any_launch(lib):
    """Host-side argument checks only: nothing here reaches a CUDA call."""
    sync = _lib.Zero1Sync()
    assert lib.b200amp_zero1_barrier(None, 2, 0, 0, 3, None) == _lib.ERR_ARG
    assert lib.b200amp_zero1_barrier(C.byref(sync), 3, 0, 0, 3, None) == _lib.ERR_ARG      # 3 ranks
    assert lib.b200amp_zero1_barrier(C.byref(sync), 2, 2, 0, 3, None) == _lib.ERR_ARG      # rank 2 of 2
    assert lib.b200amp_zero1_barrier(C.byref(sync), 2, 0, 5, 3, None) == _lib.ERR_ARG      # phase 5
    assert lib.b200amp_zero1_barrier(C.byref(sync), 2, 0, 0, 0, None) == _lib.ERR_ARG      # nothing to do
    assert lib.b200amp_zero1_barrier(C.byref(sync), 2, 0, 0, 3, None) == _lib.ERR_ARG      # null flag blocks
    assert b"flag block" in lib.b200amp_last_error()
    assert lib.b200amp_zero1_sync_init(None, None) == _lib.ERR_ARG
    assert lib.b200amp_zero1_sync_read(None, None, None) == _lib.ERR_ARG
    assert lib.b200amp_copy_async(None, None, 16, None) == _lib.ERR_ARG
