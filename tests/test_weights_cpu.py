"""weights.bin (cuda_transformer_b200/weights.py) on the CPU: round trip in both dtypes, the
refusals of the reference's reader (cuda/weights.cu:35-98), and - where the reference checkout
was present at build time - files written here go through the REFERENCE's reader and writer
byte for byte, and the fp16 file equals the reference's own fp16 export of the same master."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.filterwarnings("ignore:overflow encountered in cast")

from cuda_transformer_b200 import weights as wt
from cuda_transformer_b200.checkpoint import ModelShape

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEBUG = ModelShape(4098, 4160, 64, 2, 4, 64, 1e-5)          # 370,432 parameters


def _master(seed=0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    n = wt.expected_count(DEBUG)
    x = (rng.standard_normal(n) * 0.02).astype(np.float32)
    x[:64] = np.float32(65504.0) * np.linspace(0.999, 1.001, 64, dtype=np.float32)   # around the fp16 maximum
    x[64:128] = np.float32(6e-8) * np.linspace(0.1, 2.0, 64, dtype=np.float32)       # fp16 subnormals and ties
    return x


def test_count_and_header(tmp_path):
    assert wt.expected_count(DEBUG) == 370432
    path = str(tmp_path / "w.bin")
    x = _master()
    wt.write_weights(path, DEBUG, x)
    raw = open(path, "rb").read()
    assert not os.path.exists(path + ".tmp")
    assert len(raw) == 48 + 4 * x.size and raw[:4] == b"GPTW"
    assert [int.from_bytes(raw[4 * i:4 * i + 4], "little") for i in range(1, 8)] == [1, 4098, 4160, 64, 2, 4, 64]
    assert int.from_bytes(raw[36:40], "little") == 0 and int.from_bytes(raw[40:48], "little") == x.size
    got = wt.read_weights(path)
    assert got.dtype == 0 and vars(got.cfg) == vars(DEBUG) | {"ln_eps": float(np.float32(1e-5))}
    assert np.array_equal(got.params, x)


def test_fp16_file_from_either_arena(tmp_path):
    x = _master(1)
    padded = np.concatenate([x, np.zeros(512, np.float32)])          # arenas are padded; the file is not
    a, b = str(tmp_path / "a.bin"), str(tmp_path / "b.bin")
    wt.write_weights(a, DEBUG, padded, fp16=True)
    wt.write_weights(b, DEBUG, padded.astype(np.float16), fp16=True)
    assert open(a, "rb").read() == open(b, "rb").read()
    assert len(open(a, "rb").read()) == 48 + 2 * x.size
    got = wt.read_weights(a)
    assert got.dtype == 1 and np.array_equal(got.params, x.astype(np.float16).astype(np.float32))


def test_bad_files_are_refused(tmp_path):
    path = str(tmp_path / "w.bin")
    x = _master()
    wt.write_weights(path, DEBUG, x)
    raw = open(path, "rb").read()

    def variant(name, data):
        p = str(tmp_path / name)
        open(p, "wb").write(data)
        return p

    with pytest.raises(wt.WeightsError, match="not a weights.bin"):
        wt.read_weights(variant("foreign.bin", b"GPTC" + raw[4:]))
    with pytest.raises(wt.WeightsError, match="version 2"):
        wt.read_weights(variant("v2.bin", raw[:4] + (2).to_bytes(4, "little") + raw[8:]))
    with pytest.raises(wt.WeightsError, match="dtype 7"):
        wt.read_weights(variant("dtype.bin", raw[:36] + (7).to_bytes(4, "little") + raw[40:]))
    with pytest.raises(wt.WeightsError, match="wrong size"):
        wt.read_weights(variant("cut.bin", raw[:-4]))
    with pytest.raises(wt.WeightsError, match="wrong size"):
        wt.read_weights(variant("long.bin", raw + b"\0"))
    with pytest.raises(wt.WeightsError, match="holds"):
        wt.read_weights(variant("count.bin", raw[:40] + (5).to_bytes(8, "little") + raw[48:]))
    with pytest.raises(wt.WeightsError, match="bad sizes"):
        wt.read_weights(variant("heads.bin", raw[:24] + (5).to_bytes(4, "little") + raw[28:]))   # C % H != 0
    with pytest.raises(wt.WeightsError):
        wt.read_weights(str(tmp_path / "missing.bin"))
    with pytest.raises(wt.WeightsError, match="a model of these sizes"):
        wt.write_weights(str(tmp_path / "short.bin"), DEBUG, x[:-1])
    with pytest.raises(wt.WeightsError, match="float32 or float16"):
        wt.write_weights(str(tmp_path / "f64.bin"), DEBUG, x.astype(np.float64))


def test_reference_reader_and_writer_reproduce_our_files(tmp_path):
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import build_ref_tests
    tool = build_ref_tests.WEIGHTS_ROUNDTRIP
    if not os.path.exists(tool):
        pytest.skip("oracle/_ref/bin/weights_roundtrip was not built (no reference checkout at build time)")
    x = _master(2)
    ours32, ours16 = str(tmp_path / "ours32.bin"), str(tmp_path / "ours16.bin")
    wt.write_weights(ours32, DEBUG, x)
    wt.write_weights(ours16, DEBUG, x.astype(np.float16), fp16=True)

    def through(src, kind):
        dst = str(tmp_path / f"theirs_{kind}.bin")
        proc = subprocess.run([tool, src, dst, kind], capture_output=True, text=True, timeout=120)
        assert proc.returncode == 0, proc.stderr
        assert "V 4098 Vp 4160 n_ctx 64 L 2 H 4 C 64 n 370432" in proc.stdout
        return open(dst, "rb").read()

    assert through(ours32, "f32") == open(ours32, "rb").read()
    # the reference's fp16 export of our fp32 file == our file written from the fp16 arena
    assert through(ours32, "f16") == open(ours16, "rb").read()
    assert through(ours16, "f16") == open(ours16, "rb").read()
    # and its reader refuses what ours refuses
    cut = str(tmp_path / "cut.bin")
    open(cut, "wb").write(open(ours32, "rb").read()[:-4])
    proc = subprocess.run([tool, cut, str(tmp_path / "x.bin"), "f32"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 1 and "wrong size" in proc.stderr
