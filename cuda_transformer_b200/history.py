"""The per-step log a trainer writes from the history ring, in the reference's CSV format.

The step state of every finished step is left in a device-resident ring
(history[step % history_len], cuda/kernels/scaler.cu:165-168); the trainer reads a whole
window of it at each evaluation instead of syncing every step, and writes one row per step
(cuda/train_fast.cu:775,813-856):

    step,train,val,lr,norm,ms,scale,skipped,counted,val_bpb
    %d,%.6f,%s,%.6e,%.4f,%.2f,%g,%d,%d,%s

`val` and `val_bpb` are filled on the last row of a window only. Host code; no GPU needed.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, TextIO

from ._lib import StepState

HEADER = "step,train,val,lr,norm,ms,scale,skipped,counted,val_bpb"


def ring_window(ring: Sequence[StepState], first_step: int, count: int) -> List[StepState]:
    """The states of steps first_step .. first_step + count - 1 out of a ring that holds step i at
    i % len(ring) (count must not exceed the ring's length, or older steps were overwritten)."""
    if count > len(ring):
        raise ValueError(f"{count} steps asked of a ring of {len(ring)}")
    window = [ring[(first_step + k) % len(ring)] for k in range(count)]
    for k, st in enumerate(window):
        if st.step != first_step + k:
            raise ValueError(f"ring slot {(first_step + k) % len(ring)} holds step {st.step}, not {first_step + k}")
    return window


def _g(x: float) -> str:
    return "%g" % x


def format_row(st: StepState, ms: float, val: Optional[float] = None, val_bpb: Optional[float] = None) -> str:
    val_text = ("%f" % val) if val is not None else ""          # std::to_string(float) prints %f
    bpb_text = ("%.6f" % val_bpb) if val_bpb is not None else ""
    return "%d,%.6f,%s,%.6e,%.4f,%.2f,%s,%d,%d,%s" % (st.step + 1, st.loss, val_text, st.lr, st.grad_norm, ms,
                                                     _g(st.loss_scale), st.found_inf, st.n_valid, bpb_text)


def notices(window: Sequence[StepState], growth_interval: int) -> List[str]:
    """The lines the reference prints for skipped steps and loss-scale growth (train_fast.cu:847-856)."""
    out = []
    for k, st in enumerate(window):
        if st.found_inf:
            out.append("       step %d skipped: inf or NaN in the gradients, loss scale now %s"
                       % (st.step + 1, _g(st.loss_scale)))
        elif k > 0 and st.loss_scale != window[k - 1].loss_scale:
            out.append("       step %d: %d finite steps in a row, loss scale up to %s"
                       % (st.step + 1, growth_interval, _g(st.loss_scale)))
    return out


def write_window(log: TextIO, window: Sequence[StepState], ms_per_step: Iterable[float],
                 val: Optional[float] = None, val_bpb: Optional[float] = None) -> None:
    """One row per step; val / val_bpb go on the last row, as the reference writes them."""
    ms_list = list(ms_per_step)
    for k, st in enumerate(window):
        last = k == len(window) - 1
        log.write(format_row(st, ms_list[k], val if last else None, val_bpb if last else None) + "\n")
    log.flush()
