"""The history-ring log in the reference's CSV format (cuda/train_fast.cu:775,813-856). CPU only."""
import io

import pytest

from cuda_transformer_b200 import history
from cuda_transformer_b200._lib import StepState


def _state(step, loss=4.25, lr=6e-4, norm=3.5123, scale=65536.0, found_inf=0, n_valid=4096):
    st = StepState()
    st.step, st.loss, st.lr, st.grad_norm, st.loss_scale, st.found_inf, st.n_valid = \
        step, loss, lr, norm, scale, found_inf, n_valid
    return st


def test_rows_have_the_reference_format():
    assert history.HEADER == "step,train,val,lr,norm,ms,scale,skipped,counted,val_bpb"
    row = history.format_row(_state(9), ms=6.234)
    assert row == "10,4.250000,,6.000000e-04,3.5123,6.23,65536,0,4096,"
    row = history.format_row(_state(249, scale=131072.0, found_inf=1), ms=12.0, val=3.875, val_bpb=1.25)
    assert row == "250,4.250000,3.875000,6.000000e-04,3.5123,12.00,131072,1,4096,1.250000"


def test_window_comes_out_of_the_ring_in_step_order():
    ring_len = 8
    ring = [StepState() for _ in range(ring_len)]
    for step in range(13):                      # steps 5..12 survive in a ring of 8
        ring[step % ring_len] = _state(step, scale=65536.0 if step < 10 else 131072.0, found_inf=int(step == 7))
    window = history.ring_window(ring, first_step=5, count=8)
    assert [st.step for st in window] == list(range(5, 13))
    with pytest.raises(ValueError):
        history.ring_window(ring, first_step=4, count=8)        # step 4 was overwritten by step 12
    with pytest.raises(ValueError):
        history.ring_window(ring, first_step=5, count=9)
    out = io.StringIO()
    history.write_window(out, window, [1.0] * 8, val=3.5, val_bpb=1.5)
    lines = out.getvalue().splitlines()
    assert len(lines) == 8 and lines[0].startswith("6,") and lines[-1].endswith(",3.500000,6.000000e-04,3.5123,1.00,131072,0,4096,1.500000")
    assert all(line.split(",")[2] == "" for line in lines[:-1])
    notes = history.notices(window, growth_interval=2000)
    assert notes == ["       step 8 skipped: inf or NaN in the gradients, loss scale now 65536",
                     "       step 11: 2000 finite steps in a row, loss scale up to 131072"]
