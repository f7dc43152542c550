"""Host side of the AMP optimizer step, over the C ABI of libb200amp.so.

Two layers:

* free functions with the reference's names and argument meaning
  (cuda/kernels/fast.h:136-166, cuda/graph.h:14-30): initial_state, begin_step,
  unscale_and_norm, finalize_step, adamw_multi, lr_on_gpu, cast_to_x, CudaGraph. They
  take raw device pointers (ints) or torch tensors and raise B200AmpError where the
  reference would print and exit(1) (cuda/common.h:10-20).

* AmpOptimizer: what FastGPT keeps for its optimizer (cuda/gpt_fast.cu:96-149,
  245-253, 438-467): the arenas, the tensor table, the device-resident step state and
  history ring, reset / set_params / optimizer_step / read_state, with the fp16
  gradient arena the native kernels read. ShardedAmpOptimizer is the ZeRO-1 form over
  torch.distributed: reduce-scatter of fp16 gradients, the two passes on the rank's
  shard, an all-gather of the 16-byte {norm^2, flag} pairs, and an in-place
  all-gather of the fp16 weights. FusedZero1Optimizer folds the two collectives into
  the passes (peer loads and stores over NVLink, or the copy engines) and orders the
  ranks with the library's own bounded flag words. HostGradientFeed (mixed into the
  owners) feeds steps from pinned host memory through two gradient arenas taking turns.

torch is used for device memory, streams and the process group only; every
arithmetic step runs in the CUDA kernels of the library.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import B200AmpError, DecayRuns, ScheduleConfig, StepState, TensorInfo, Zero1Sync, check
from .layout import ParamSlot, padded, shard_range, tensor_table

__all__ = [
    "StepState", "ScheduleConfig", "TensorInfo", "B200AmpError",
    "initial_state", "begin_step", "unscale_and_norm", "finalize_step", "adamw_multi", "lr_on_gpu",
    "cast_to_x", "CudaGraph", "AmpOptimizer", "Zero1Step", "ShardedAmpOptimizer", "make_schedule",
    "pass1_f16", "pass1_f16_static", "cast_pass1_f32", "pass1_finalize_f16", "rs_pass1_f16", "pass2_ag_f16",
    "FusedZero1Optimizer", "finalize_sums", "pass2_f16", "step_f16", "check_tensor_table", "HostGradientFeed",
    "pass1_partition", "rs_pass1_f16_part", "copy_async", "rs_pass1_f16_ce", "pass2_ag_f16_ce",
    "DecayRuns", "decay_runs_build", "pass2_f16_runs", "Zero1Sync", "make_sync", "zero1_sync_init", "zero1_sync_read", "zero1_barrier", "rs_pass1_f16_sync",
    "finalize_sums_sync", "device_error", "RankWaitError",
]


def _ptr(x) -> Optional[int]:
    """Device pointer of a tensor (or pass an int / None through)."""
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        if not x.is_cuda:
            raise ValueError("expected a CUDA tensor: the step has no CPU path")
        if not x.is_contiguous():
            raise ValueError("expected a contiguous tensor")
        return x.data_ptr()
    return int(x)


def _stream(stream) -> int:
    """cudaStream_t handle: a torch stream, a raw handle, or None = torch's current stream."""
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)


def make_schedule(lr=6e-4, min_lr=6e-4, warmup_steps=0, max_steps=1 << 30, beta1=0.9, beta2=0.95,
                  weight_decay=0.1, grad_clip=1.0, growth_interval=2000, dynamic_scale=1,
                  decay_steps=0) -> ScheduleConfig:
    """A ScheduleConfig; the defaults are the flat-lr setting the reference's tests use
    (cuda/tests/test_fast.cu:85-92) with the reference's AdamW numbers (reference/config.py)."""
    return ScheduleConfig(lr, min_lr, warmup_steps, max_steps, beta1, beta2, weight_decay, grad_clip,
                          growth_interval, dynamic_scale, decay_steps)


# ------------------------------------------------------------------ the reference's launchers

def initial_state(scale: float) -> StepState:
    """cuda/kernels/scaler.cu:21-29."""
    st = StepState()
    check(_lib.load().b200amp_initial_state(scale, C.byref(st)))
    return st


def begin_step(st, stream=None) -> None:
    """cuda/kernels/scaler.cu:173-177."""
    check(_lib.load().b200amp_begin_step(_ptr(st), _stream(stream)))


def unscale_and_norm(grads, n: int, st, partial, stream=None) -> None:
    """cuda/kernels/scaler.cu:179-184: fp32 grads *= inv_scale in place, flag, partial[512]."""
    check(_lib.load().b200amp_unscale_and_norm_f32(_ptr(grads), n, _ptr(st), _ptr(partial), _stream(stream)))


def finalize_step(st, partial, cfg: ScheduleConfig, history=None, history_len: int = 0, stream=None) -> None:
    """cuda/kernels/scaler.cu:186-192."""
    check(_lib.load().b200amp_finalize_step(_ptr(st), _ptr(partial), C.byref(cfg), _ptr(history), history_len,
                                            _stream(stream)))


def adamw_multi(params, params_x, grads, m, v, n: int, tensors, ntensors: int, st, beta1: float, beta2: float,
                eps: float, stream=None) -> None:
    """cuda/kernels/adamw_multi.cu:93-108 (unscaled fp32 gradients; params_x may be None)."""
    check(_lib.load().b200amp_adamw_multi_f32(_ptr(params), _ptr(params_x), _ptr(grads), _ptr(m), _ptr(v), n,
                                              _ptr(tensors), ntensors, _ptr(st), beta1, beta2, eps,
                                              _stream(stream)))


def lr_on_gpu(step: int, cfg: ScheduleConfig) -> float:
    """cuda/kernels/scaler.cu:100-110."""
    out = C.c_double()
    check(_lib.load().b200amp_lr_on_gpu(step, C.byref(cfg), C.byref(out)))
    return out.value


def cast_to_x(out_f16, inp_f32, n: int, stream=None) -> None:
    """cuda/kernels/fused.cu:319-323 in the fp16 build."""
    check(_lib.load().b200amp_cast_to_x(_ptr(out_f16), _ptr(inp_f32), n, _stream(stream)))


# ------------------------------------------------------------------ native entry points

def pass1_f16(grads16, n: int, st, workspace, stream=None) -> None:
    check(_lib.load().b200amp_pass1_f16(_ptr(grads16), n, _ptr(st), _ptr(workspace), _stream(stream)))


def pass1_f16_static(grads16, n: int, st, sums_out, stream=None) -> None:
    """Pass 1 on the library's own scratch: for callers that cannot allocate device memory.
    sums_out: device memory for two doubles {sum of squares, flag}. See include/b200amp.h."""
    check(_lib.load().b200amp_pass1_f16_static(_ptr(grads16), n, _ptr(st), _ptr(sums_out), _stream(stream)))


def cast_pass1_f32(grads32, grads16, n: int, clear_source: bool, st, workspace, cfg: Optional[ScheduleConfig] = None,
                   history=None, history_len: int = 0, stream=None) -> None:
    """fp32 loss-scaled gradients -> fp16 arena + pass 1 (+ finalize when cfg is given) in one sweep;
    clear_source zeroes the fp32 arena behind it (the reference's per-step grads.zero)."""
    check(_lib.load().b200amp_cast_pass1_f32(_ptr(grads32), _ptr(grads16), n, 1 if clear_source else 0, _ptr(st),
                                             _ptr(workspace), C.byref(cfg) if cfg is not None else None,
                                             _ptr(history), history_len, _stream(stream)))


def pass1_finalize_f16(grads16, n: int, st, workspace, cfg: ScheduleConfig, history=None, history_len: int = 0,
                       stream=None) -> None:
    check(_lib.load().b200amp_pass1_finalize_f16(_ptr(grads16), n, _ptr(st), _ptr(workspace), C.byref(cfg),
                                                 _ptr(history), history_len, _stream(stream)))


def finalize_sums(st, sums, nranks: int, cfg: ScheduleConfig, history=None, history_len: int = 0,
                  stream=None) -> None:
    check(_lib.load().b200amp_finalize_sums(_ptr(st), _ptr(sums), nranks, C.byref(cfg), _ptr(history),
                                            history_len, _stream(stream)))


def pass2_f16(master, m, v, grads16, weights16, n: int, arena_offset: int, tensors, ntensors: int, st,
              beta1: float, beta2: float, eps: float, stream=None) -> None:
    check(_lib.load().b200amp_pass2_f16(_ptr(master), _ptr(m), _ptr(v), _ptr(grads16), _ptr(weights16), n,
                                        arena_offset, _ptr(tensors), ntensors, _ptr(st), beta1, beta2, eps,
                                        _stream(stream)))


def decay_runs_build(table: Sequence[Tuple[int, int, int]]) -> DecayRuns:
    """The (offset, count, decay) rows merged into runs of equal decay flag, for pass2_f16_runs.
    Raises B200AmpError (status ERR_LIMIT) when the table has more than 256 runs."""
    arr = (TensorInfo * max(1, len(table)))(*[TensorInfo(o, c, d) for o, c, d in table])
    runs = DecayRuns()
    check(_lib.load().b200amp_decay_runs_build(C.cast(arr, C.c_void_p), len(table), C.byref(runs)))
    return runs


def pass2_f16_runs(master, m, v, grads16, weights16, n: int, arena_offset: int, runs: DecayRuns, st,
                   beta1: float, beta2: float, eps: float, stream=None) -> None:
    """pass2_f16 with the decay runs passed as a kernel parameter (no table in device memory)."""
    check(_lib.load().b200amp_pass2_f16_runs(_ptr(master), _ptr(m), _ptr(v), _ptr(grads16), _ptr(weights16), n,
                                             arena_offset, C.byref(runs), _ptr(st), beta1, beta2, eps,
                                             _stream(stream)))


def _pointer_array(pointers: Sequence[int]):
    return (C.c_void_p * len(pointers))(*[C.c_void_p(int(p)) for p in pointers])


def rs_pass1_f16(grads16_by_rank: Sequence[int], my_rank: int, reduced16, n: int, st, workspace,
                 pair_table_by_rank: Optional[Sequence[int]] = None, stream=None) -> None:
    """Reduce-scatter + pass 1 in one kernel. grads16_by_rank[r]: device pointer (valid in THIS process)
    to the start of this rank's slice in rank r's gradient arena."""
    tables = _pointer_array(pair_table_by_rank) if pair_table_by_rank is not None else None
    check(_lib.load().b200amp_rs_pass1_f16(_pointer_array(grads16_by_rank), len(grads16_by_rank), my_rank,
                                           _ptr(reduced16), n, _ptr(st), _ptr(workspace), tables,
                                           _stream(stream)))


def pass2_ag_f16(master, m, v, reduced16, weights16_by_rank: Sequence[int], n: int, arena_offset: int, tensors,
                 ntensors: int, st, beta1: float, beta2: float, eps: float, stream=None) -> None:
    """Pass 2 + all-gather in one kernel. weights16_by_rank[r]: device pointer to the start of this
    rank's slice in rank r's weight arena (own arena included)."""
    check(_lib.load().b200amp_pass2_ag_f16(_ptr(master), _ptr(m), _ptr(v), _ptr(reduced16),
                                           _pointer_array(weights16_by_rank), len(weights16_by_rank), n,
                                           arena_offset, _ptr(tensors), ntensors, _ptr(st), beta1, beta2, eps,
                                           _stream(stream)))


def pass1_partition(n: int):
    """(virtual blocks, elements per virtual block) of the fixed partition pass 1 sums a range of
    n elements over."""
    vblocks, per = C.c_int(), C.c_longlong()
    check(_lib.load().b200amp_pass1_partition(n, C.byref(vblocks), C.byref(per)))
    return vblocks.value, per.value


def rs_pass1_f16_part(grads16_by_rank: Sequence[int], my_rank: int, reduced16, n: int, vblock_first: int,
                      vblock_count: int, last_part: bool, st, workspace,
                      pair_table_by_rank: Optional[Sequence[int]] = None, stream=None) -> None:
    """rs_pass1_f16 on the virtual blocks vblock_first .. vblock_first + vblock_count - 1 of the slice."""
    tables = _pointer_array(pair_table_by_rank) if pair_table_by_rank is not None else None
    check(_lib.load().b200amp_rs_pass1_f16_part(_pointer_array(grads16_by_rank), len(grads16_by_rank), my_rank,
                                                _ptr(reduced16), n, vblock_first, vblock_count,
                                                1 if last_part else 0, _ptr(st), _ptr(workspace), tables,
                                                _stream(stream)))


def copy_async(dst, src, nbytes: int, stream=None) -> None:
    """Copy-engine transfer between two device pointers of this process (peer mappings included)."""
    check(_lib.load().b200amp_copy_async(_ptr(dst), _ptr(src), nbytes, _stream(stream)))


# ---- ordering between one-process-per-GPU ranks (include/b200amp.h, "owned by the library")

def make_sync(block_by_rank: Sequence[int], wait_limit: int = 0) -> Zero1Sync:
    """block_by_rank[r]: rank r's block of flag words as a device pointer of THIS process."""
    sync = Zero1Sync()
    for r, p in enumerate(block_by_rank):
        sync.block_by_rank[r] = int(p)
    sync.wait_limit = wait_limit
    return sync


def zero1_sync_init(block, stream=None) -> None:
    check(_lib.load().b200amp_zero1_sync_init(_ptr(block), _stream(stream)))


def zero1_sync_read(block) -> Tuple[int, int]:
    """(steps completed, error word) of a rank's own block; synchronous."""
    steps, error = C.c_uint(), C.c_uint()
    check(_lib.load().b200amp_zero1_sync_read(_ptr(block), C.byref(steps), C.byref(error)))
    return steps.value, error.value


def zero1_barrier(sync: Zero1Sync, nranks: int, my_rank: int, phase: int, what: int, stream=None) -> None:
    check(_lib.load().b200amp_zero1_barrier(C.byref(sync), nranks, my_rank, phase, what, _stream(stream)))


def rs_pass1_f16_sync(grads16_by_rank: Sequence[int], my_rank: int, reduced16, n: int, st, workspace,
                      pair_table_by_rank: Sequence[int], sync: Zero1Sync, stream=None) -> None:
    check(_lib.load().b200amp_rs_pass1_f16_sync(_pointer_array(grads16_by_rank), len(grads16_by_rank), my_rank,
                                                _ptr(reduced16), n, _ptr(st), _ptr(workspace),
                                                _pointer_array(pair_table_by_rank), C.byref(sync), _stream(stream)))


def finalize_sums_sync(st, sums, nranks: int, my_rank: int, cfg: ScheduleConfig, sync: Zero1Sync, history=None,
                       history_len: int = 0, stream=None) -> None:
    check(_lib.load().b200amp_finalize_sums_sync(_ptr(st), _ptr(sums), nranks, my_rank, C.byref(cfg), _ptr(history),
                                                 history_len, C.byref(sync), _stream(stream)))


def rs_pass1_f16_ce(grads16_by_rank: Sequence[int], my_rank: int, staging16, reduced16, n: int, pieces: int, st,
                    workspace, pair_table_by_rank: Optional[Sequence[int]] = None,
                    sync: Optional[Zero1Sync] = None, stream=None) -> None:
    """Reduce-scatter + pass 1 with the peers' slices pulled by the copy engines into staging16
    ((nranks - 1) * n fp16 values, local), piece by piece, while earlier pieces are reduced."""
    tables = _pointer_array(pair_table_by_rank) if pair_table_by_rank is not None else None
    check(_lib.load().b200amp_rs_pass1_f16_ce(_pointer_array(grads16_by_rank), len(grads16_by_rank), my_rank,
                                              _ptr(staging16), _ptr(reduced16), n, pieces, _ptr(st),
                                              _ptr(workspace), tables,
                                              C.byref(sync) if sync is not None else None, _stream(stream)))


def rs_push_f16_ce(grads16, staging_by_rank: Sequence[int], my_rank: int, n: int, pieces: int, sync: Zero1Sync,
                   stream=None) -> None:
    """Reduce-scatter by push, sender's side: slice q of this rank's arena into row my_rank of rank
    q's staging buffer, piece by piece, each piece followed by its flag (copy engines)."""
    check(_lib.load().b200amp_rs_push_f16_ce(_ptr(grads16), _pointer_array(staging_by_rank), len(staging_by_rank),
                                             my_rank, n, pieces, C.byref(sync), _stream(stream)))


def rs_pass1_f16_pushed(own_slice16, staging16, nranks: int, my_rank: int, reduced16, n: int, pieces: int, st,
                        workspace, pair_table_by_rank: Sequence[int], sync: Zero1Sync, stream=None) -> None:
    """Reduce-scatter by push, owner's side: pass 1 over the rank's own slice and the staging rows
    its peers filled, each piece waiting (bounded) for its flags."""
    check(_lib.load().b200amp_rs_pass1_f16_pushed(_ptr(own_slice16), _ptr(staging16), nranks, my_rank,
                                                  _ptr(reduced16), n, pieces, _ptr(st), _ptr(workspace),
                                                  _pointer_array(pair_table_by_rank), C.byref(sync),
                                                  _stream(stream)))


def pass2_ag_f16_ce(master, m, v, reduced16, weights16_by_rank: Sequence[int], my_rank: int, n: int,
                    arena_offset: int, tensors, ntensors: int, st, beta1: float, beta2: float, eps: float,
                    pieces: int, stream=None) -> None:
    """Pass 2 + all-gather with every piece of fp16 weights pushed to the peers by the copy
    engines while pass 2 runs on the next piece."""
    check(_lib.load().b200amp_pass2_ag_f16_ce(_ptr(master), _ptr(m), _ptr(v), _ptr(reduced16),
                                              _pointer_array(weights16_by_rank), len(weights16_by_rank), my_rank, n,
                                              arena_offset, _ptr(tensors), ntensors, _ptr(st), beta1, beta2, eps,
                                              pieces, _stream(stream)))


def device_error() -> int:
    """Bit mask of what gave up a bounded wait on the current device since the last call (1: a bulk
    copy of the staged pass 2, 2: a wait on another rank); reading clears it. Synchronises."""
    out = C.c_int()
    check(_lib.load().b200amp_device_error(C.byref(out)))
    return out.value


class RankWaitError(B200AmpError):
    """A kernel of the ZeRO-1 step stopped waiting for another rank. The step was not applied."""


def step_f16(master, m, v, grads16, weights16, n: int, tensors, ntensors: int, st, workspace,
             cfg: ScheduleConfig, history, history_len: int, beta1: float, beta2: float, eps: float,
             stream=None) -> None:
    check(_lib.load().b200amp_step_f16(_ptr(master), _ptr(m), _ptr(v), _ptr(grads16), _ptr(weights16), n,
                                       _ptr(tensors), ntensors, _ptr(st), _ptr(workspace), C.byref(cfg),
                                       _ptr(history), history_len, beta1, beta2, eps, _stream(stream)))


class CudaGraph:
    """capture / launch / ready, as cuda/graph.h:14-30. The body runs once in capture
    mode (nothing executes) and is replayed by launch()."""

    def __init__(self) -> None:
        self._handle = C.c_void_p()

    def ready(self) -> bool:
        return bool(self._handle)

    def capture(self, stream, body) -> None:
        lib = _lib.load()
        if self.ready():
            check(lib.b200amp_graph_destroy(self._handle))
            self._handle = C.c_void_p()
        s = _stream(stream)
        check(lib.b200amp_graph_begin_capture(s))
        try:
            body()
        finally:
            status = lib.b200amp_graph_end_capture(s, C.byref(self._handle))
        check(status)

    def launch(self, stream=None) -> None:
        check(_lib.load().b200amp_graph_launch(self._handle, _stream(stream)))

    def __del__(self) -> None:
        try:
            if self._handle:
                _lib.load().b200amp_graph_destroy(self._handle)
                self._handle = C.c_void_p()
        except Exception:
            pass


# ------------------------------------------------------------------ arena owners

def _upload_struct(struct_obj, device) -> torch.Tensor:
    raw = bytes(struct_obj)
    host = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    return host.to(device)


def check_tensor_table(table: Sequence[Tuple[int, int, int]], n: int = 0) -> None:
    """Raises B200AmpError unless the (offset, count, decay) rows are a table the kernels can
    trust: ascending, offsets multiples of 4, no overlap, inside n elements when n > 0."""
    arr = (TensorInfo * max(1, len(table)))(*[TensorInfo(o, c, d) for o, c, d in table])
    check(_lib.load().b200amp_check_tensor_table(C.cast(arr, C.c_void_p), len(table), n))


def _tensor_table_device(table: Sequence[Tuple[int, int, int]], device, n: int = 0) -> torch.Tensor:
    check_tensor_table(table, n)
    arr = (TensorInfo * len(table))(*[TensorInfo(o, c, d) for o, c, d in table])
    host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
    return host.to(device)


class HostGradientFeed:
    """Steps fed from the host: for a caller whose loss-scaled fp16 gradients arrive in pinned host
    memory (an offloaded backward pass, a parameter server, a benchmark of the whole path).

        ticket = opt.submit_host_gradients(pinned_fp16)     # returns at once
        state = opt.collect(ticket)                         # the step's 60-byte state, when it is done

    Two device gradient arenas take turns: while pass 2 of step k reads one, the copy engine fills
    the other with step k + 1's gradients, so a step costs the longer of its host-to-device copy
    and its kernels instead of their sum. The copy runs on its own stream; the step (and the
    device-to-host copy of its state into pinned memory) runs on a second one, behind an event of
    the copy; an arena is refilled only after the step that read it has finished. At most two
    steps are in flight: submitting a third collects the first. Mixed into the optimizers below;
    the host class provides _feed_arenas() and _feed_step(arena_index)."""

    def _feed_setup(self) -> None:
        dev = self.device
        with torch.cuda.device(dev):
            self._feed = {
                "copy": torch.cuda.Stream(device=dev), "step": torch.cuda.Stream(device=dev),
                "copied": [torch.cuda.Event() for _ in range(2)], "done": [torch.cuda.Event() for _ in range(2)],
                "host_state": [torch.empty(C.sizeof(StepState), dtype=torch.uint8, pin_memory=True) for _ in range(2)],
                "arenas": self._feed_arenas(), "next": 0, "results": {}, "pending": set(),
            }
            torch.cuda.current_stream(dev).synchronize()

    def submit_host_gradients(self, host_grads16: torch.Tensor) -> int:
        if getattr(self, "_feed", None) is None:
            self._feed_setup()
        f = self._feed
        ticket = f["next"]
        slot = ticket % 2
        if ticket - 2 in f["pending"]:
            # its pinned state buffer and its arena are about to be reused: fetch its result now and keep it
            f["results"][ticket - 2] = self.collect(ticket - 2)
        arena = f["arenas"][slot]
        if host_grads16.numel() != arena.numel() or host_grads16.dtype != torch.float16:
            raise ValueError(f"expected {arena.numel()} fp16 gradients, got {host_grads16.numel()} of {host_grads16.dtype}")
        with torch.cuda.device(self.device):
            if ticket == 0:
                # whatever the caller enqueued on its current stream before the first submission comes first
                first = torch.cuda.Event()
                first.record(torch.cuda.current_stream(self.device))
                f["copy"].wait_event(first)
                f["step"].wait_event(first)
            if ticket >= 2:
                f["copy"].wait_event(f["done"][slot])   # the step that read this arena has finished
            with torch.cuda.stream(f["copy"]):
                arena.copy_(host_grads16, non_blocking=True)
                f["copied"][slot].record(f["copy"])
            f["step"].wait_event(f["copied"][slot])
            with torch.cuda.stream(f["step"]):
                self._feed_step(slot)
                f["host_state"][slot].copy_(self.state, non_blocking=True)
                f["done"][slot].record(f["step"])
        f["pending"].add(ticket)
        f["next"] = ticket + 1
        return ticket

    def collect(self, ticket: int) -> StepState:
        """The state after the step of `ticket` (blocks until that step and its read-back are done)."""
        f = self._feed
        if ticket in f["results"]:
            return f["results"].pop(ticket)
        if ticket not in f["pending"]:
            raise ValueError(f"ticket {ticket} was never submitted or has been collected already")
        slot = ticket % 2
        f["done"][slot].synchronize()
        st = StepState.from_buffer_copy(f["host_state"][slot].numpy().tobytes())
        f["pending"].discard(ticket)
        return st

    def host_feed_streams(self):
        """(copy stream, step stream) of the feed, for a caller that wants to put its own events on them."""
        if getattr(self, "_feed", None) is None:
            self._feed_setup()
        return self._feed["copy"], self._feed["step"]

    def drain_host_feed(self) -> None:
        """Waits for every submitted step; results not collected yet stay available to collect()."""
        f = getattr(self, "_feed", None)
        if f is None:
            return
        for ticket in sorted(f["pending"]):
            f["results"][ticket] = self.collect(ticket)
        f["step"].synchronize()


class AmpOptimizer(HostGradientFeed):
    """The optimizer state of one GPU that holds the whole arena.

    Arenas (flat, in param_layout order, cuda/gpt_fast.cu:96-115): master, m, v (fp32),
    weights16 (fp16 copy the GEMMs read) and grads16 (fp16, loss-scaled, written by the
    caller before each step). Step state, history ring and the pass-1 workspace live in
    device memory; nothing crosses to the host inside optimizer_step().
    """

    def __init__(self, slots: List[ParamSlot], cfg: ScheduleConfig, eps: float = 1e-8,
                 loss_scale: float = 65536.0, history_len: int = 256, device="cuda:0"):
        self.lib = _lib.load()
        check(self._with_device(device, self.lib.b200amp_device_check))
        self.device = torch.device(device)
        self.slots = slots
        self.n_params = slots[-1].offset + slots[-1].count
        self.n = padded(self.n_params)
        self.sched = cfg
        self.beta1, self.beta2, self.eps = cfg.beta1, cfg.beta2, eps
        self.history_len = history_len
        table = list(tensor_table(slots))
        if self.n > self.n_params:
            table.append((self.n_params, self.n - self.n_params, 0))       # zero padding: never decayed
        self.ntensors = len(table)
        with torch.cuda.device(self.device):
            self.tensors = _tensor_table_device(table, self.device, self.n)
            self.master = torch.zeros(self.n, dtype=torch.float32, device=self.device)
            self.m = torch.zeros_like(self.master)
            self.v = torch.zeros_like(self.master)
            self.weights16 = torch.zeros(self.n, dtype=torch.float16, device=self.device)
            self.grads16 = torch.zeros(self.n, dtype=torch.float16, device=self.device)
            self.state = torch.zeros(C.sizeof(StepState), dtype=torch.uint8, device=self.device)
            self.history = torch.zeros(C.sizeof(StepState) * history_len, dtype=torch.uint8, device=self.device)
            self.workspace = torch.zeros(self.lib.b200amp_workspace_bytes(), dtype=torch.uint8, device=self.device)
        self.reset(loss_scale)

    @staticmethod
    def _with_device(device, fn):
        with torch.cuda.device(torch.device(device)):
            return fn()

    def reset(self, loss_scale: float) -> None:
        """m = v = grads = 0 and a fresh state (cuda/gpt_fast.cu:245-253)."""
        self.m.zero_()
        self.v.zero_()
        self.grads16.zero_()
        self.history.zero_()
        self.workspace.zero_()
        self.write_state(initial_state(loss_scale))

    def write_state(self, st: StepState) -> None:
        self.state.copy_(_upload_struct(st, self.device))
        torch.cuda.current_stream(self.device).synchronize()

    def set_params(self, host_params: torch.Tensor) -> None:
        """Upload fp32 parameters and rebuild the fp16 copy (cuda/gpt_fast.cu:274-286)."""
        flat = host_params.reshape(-1).to(torch.float32)
        if flat.numel() != self.n_params:
            raise ValueError(f"{flat.numel()} parameters given, the arena holds {self.n_params}")
        self.master.zero_()
        self.master[: self.n_params].copy_(flat)
        with torch.cuda.device(self.device):
            cast_to_x(self.weights16, self.master, self.n)

    def decay_runs(self) -> DecayRuns:
        """The tensor table merged into runs of equal decay flag (built once, on the host)."""
        if getattr(self, "_runs", None) is None:
            table = list(tensor_table(self.slots))
            if self.n > self.n_params:
                table.append((self.n_params, self.n - self.n_params, 0))
            self._runs = decay_runs_build(table)
        return self._runs

    def optimizer_step(self, stream=None, pass2: str = "table") -> None:
        """The two launches of the step (the place of cuda/gpt_fast.cu:438-450). pass2 = "runs"
        hands the decay flags to pass 2 as a kernel parameter (tables of at most 256 runs)
        instead of the table in device memory; the results are the same bits."""
        with torch.cuda.device(self.device):
            if pass2 == "runs":
                pass1_finalize_f16(self.grads16, self.n, self.state, self.workspace, self.sched, self.history,
                                   self.history_len, stream)
                pass2_f16_runs(self.master, self.m, self.v, self.grads16, self.weights16, self.n, 0,
                               self.decay_runs(), self.state, self.beta1, self.beta2, self.eps, stream)
                return
            step_f16(self.master, self.m, self.v, self.grads16, self.weights16, self.n, self.tensors,
                     self.ntensors, self.state, self.workspace, self.sched, self.history, self.history_len,
                     self.beta1, self.beta2, self.eps, stream)

    # -- HostGradientFeed
    def _feed_arenas(self):
        return [self.grads16, torch.zeros_like(self.grads16)]

    def _feed_step(self, slot: int) -> None:
        grads = self._feed["arenas"][slot]
        pass1_finalize_f16(grads, self.n, self.state, self.workspace, self.sched, self.history, self.history_len)
        pass2_f16(self.master, self.m, self.v, grads, self.weights16, self.n, 0, self.tensors, self.ntensors,
                  self.state, self.beta1, self.beta2, self.eps)

    def read_state(self) -> StepState:
        """Sync + D2H of the 60-byte state (cuda/gpt_fast.cu:461-467). When the staged pass 2 is
        selected (tuning knob pass2_variant = 1) its give-up flag is checked here too: a launch
        that stopped waiting for a bulk copy has updated some tiles only, and the caller must not
        go on with that state."""
        self.drain_host_feed()          # steps submitted through the host feed run on their own stream
        raw = bytes(self.state.cpu().numpy().tobytes())
        variant = C.c_int()
        check(self.lib.b200amp_tune_get(b"pass2_variant", C.byref(variant)))
        if variant.value == 1:
            with torch.cuda.device(self.device):
                if device_error() & 1:
                    raise B200AmpError(_lib.ERR_CUDA, "the staged pass 2 gave up waiting for a bulk copy: master, m "
                                       "and v are partly updated; restore them from a checkpoint")
        return StepState.from_buffer_copy(raw)

    def read_history(self) -> List[StepState]:
        raw = self.history.cpu().numpy().tobytes()
        size = C.sizeof(StepState)
        return [StepState.from_buffer_copy(raw[i * size:(i + 1) * size]) for i in range(self.history_len)]


class Zero1Step:
    """Orchestration of the ZeRO-1 step over a torch.distributed process group.

    Every rank holds the full fp16 gradient arena (its own micro-batch's gradients) and
    the full fp16 weight arena; master, m and v exist only for the rank's slice
    [begin, end) of the arena. One step:
        reduce-scatter(AVG) of grads16 into the rank's slice  ->  pass 1 on the slice
        ->  all-gather of {sum of squares, flag} (16 B per rank)  ->  finalize (replicated,
        pairs added in rank order so every rank holds identical state bits)
        ->  pass 2 on the slice, writing fp16 weights into the slice of weights16
        ->  in-place all-gather of weights16.
    The inf/NaN flag and the norm are taken on the averaged gradients, as DDP +
    GradScaler would see them.

    This class owns the buffers and the collectives and is backend-agnostic (NCCL on
    GPUs; the CPU test-suite drives it over gloo). The three compute hooks (_pass1,
    _finalize, _pass2) are abstract here: ShardedAmpOptimizer below binds them to the
    CUDA kernels and is the only implementation the package ships.
    """

    def __init__(self, slots: List[ParamSlot], cfg: ScheduleConfig, eps: float, loss_scale: float,
                 history_len: int, device, group):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.slots = slots
        self.n_params = slots[-1].offset + slots[-1].count
        self.n = padded(self.n_params)
        self.begin, self.end = shard_range(self.n, self.rank, self.world)
        self.n_local = self.end - self.begin
        self.sched = cfg
        self.beta1, self.beta2, self.eps = cfg.beta1, cfg.beta2, eps
        self.history_len = history_len
        self.device = torch.device(device)
        self.table = list(tensor_table(slots))
        if self.n > self.n_params:
            self.table.append((self.n_params, self.n - self.n_params, 0))      # zero padding: never decayed
        self.ntensors = len(self.table)
        dev = self.device
        self.master = torch.zeros(self.n_local, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.weights16 = self._alloc_arena16("weights16")
        self.grads16 = self._alloc_arena16("grads16")
        self.grad_shard = torch.zeros(self.n_local, dtype=torch.float16, device=dev)
        self.state = torch.zeros(C.sizeof(StepState), dtype=torch.uint8, device=dev)
        self.history = torch.zeros(C.sizeof(StepState) * history_len, dtype=torch.uint8, device=dev)
        self.sums_local = torch.zeros(2, dtype=torch.float64, device=dev)      # {sum of squares, flag}
        self.sums_all = torch.zeros(2 * self.world, dtype=torch.float64, device=dev)
        self.reset(loss_scale)

    def _alloc_arena16(self, name: str) -> torch.Tensor:
        """A full-length fp16 arena (gradients or weights). Subclasses that map the arenas into
        the other ranks' address spaces allocate them differently."""
        return torch.zeros(self.n, dtype=torch.float16, device=self.device)

    # -- compute hooks, bound by the subclass
    def _pass1(self) -> None:
        """grad_shard -> sums_local = {sum of squares of the unscaled slice, flag}."""
        raise NotImplementedError

    def _finalize(self) -> None:
        """sums_all (rank-ordered pairs) -> state, history."""
        raise NotImplementedError

    def _pass2(self) -> None:
        """AdamW on the slice; fp16 weights into weights16[begin:end]."""
        raise NotImplementedError

    def _cast_weights(self, full_fp32: torch.Tensor) -> None:
        """weights16 = fp16(full_fp32), at set-up."""
        raise NotImplementedError

    # -- state
    def reset(self, loss_scale: float) -> None:
        self.m.zero_()
        self.v.zero_()
        self.grads16.zero_()
        self.history.zero_()
        self.write_state(initial_state_host(loss_scale))

    def write_state(self, st: StepState) -> None:
        self.state.copy_(torch.frombuffer(bytearray(bytes(st)), dtype=torch.uint8))
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()

    def read_state(self) -> StepState:
        return StepState.from_buffer_copy(self.state.cpu().numpy().tobytes())

    def set_params(self, host_params: torch.Tensor) -> None:
        """Every rank passes the same full fp32 parameter vector; it keeps its slice."""
        flat = torch.zeros(self.n, dtype=torch.float32)
        flat[: self.n_params] = host_params.reshape(-1).to(torch.float32)
        self.master.copy_(flat[self.begin:self.end])
        self._cast_weights(flat)

    # -- collectives
    def reduce_scatter_grads(self) -> None:
        self.dist.reduce_scatter_tensor(self.grad_shard, self.grads16, op=self.dist.ReduceOp.AVG, group=self.group)

    def gather_sums(self) -> None:
        self.dist.all_gather_into_tensor(self.sums_all, self.sums_local, group=self.group)

    def all_gather_weights(self) -> None:
        self.dist.all_gather_into_tensor(self.weights16, self.weights16[self.begin:self.end], group=self.group)

    def optimizer_step(self) -> None:
        self.reduce_scatter_grads()
        self._pass1()
        self.gather_sums()
        self._finalize()
        self._pass2()
        self.all_gather_weights()


def initial_state_host(scale: float) -> StepState:
    """initial_state() without touching the library (cuda/kernels/scaler.cu:21-29): plain field
    assignments, used where a state is built before any device is chosen."""
    st = StepState()
    st.loss_scale = scale
    st.inv_scale = 1.0 / scale
    st.clip_coef = 1.0
    st.decay = 1.0
    return st


class ShardedAmpOptimizer(Zero1Step):
    """Zero1Step bound to the CUDA kernels: one rank per B200, NCCL process group."""

    def __init__(self, slots: List[ParamSlot], cfg: ScheduleConfig, eps: float = 1e-8,
                 loss_scale: float = 65536.0, history_len: int = 256, device=None, group=None):
        self.lib = _lib.load()
        device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        if device.type != "cuda":
            raise ValueError("ShardedAmpOptimizer runs on CUDA devices only")
        with torch.cuda.device(device):
            check(self.lib.b200amp_device_check())
            super().__init__(slots, cfg, eps, loss_scale, history_len, device, group)
            self.tensors = _tensor_table_device(self.table, self.device, self.n)
            self.workspace = torch.zeros(self.lib.b200amp_workspace_bytes(), dtype=torch.uint8, device=self.device)
            # pass 1 publishes {sum, flag} in the first 16 bytes of its workspace
            self.sums_local = self.workspace[:16].view(torch.float64)

    def _pass1(self) -> None:
        pass1_f16(self.grad_shard, self.n_local, self.state, self.workspace)

    def _finalize(self) -> None:
        finalize_sums(self.state, self.sums_all, self.world, self.sched, self.history, self.history_len)

    def _pass2(self) -> None:
        pass2_f16(self.master, self.m, self.v, self.grad_shard, self.weights16[self.begin:self.end], self.n_local,
                  self.begin, self.tensors, self.ntensors, self.state, self.beta1, self.beta2, self.eps)

    def _cast_weights(self, full_fp32: torch.Tensor) -> None:
        with torch.cuda.device(self.device):
            full = full_fp32.to(self.device)
            cast_to_x(self.weights16, full, self.n)
            torch.cuda.current_stream().synchronize()

    def optimizer_step(self) -> None:
        with torch.cuda.device(self.device):
            super().optimizer_step()


class FusedZero1Optimizer(ShardedAmpOptimizer, HostGradientFeed):
    """ZeRO-1 with the collectives folded into the two passes instead of NCCL calls around them,
    and the ordering between the ranks done by the library's own flag words.

    The fp16 gradient arena, the fp16 weight arena, the table of {sum, flag} pairs and one
    1 KB block of flag words are allocated as symmetric memory
    (torch.distributed._symmetric_memory, used for the allocation and the mapping only): every
    rank's buffers are mapped into every process, so a kernel reads a peer's gradients and writes a
    peer's weights with ordinary loads and stores over NVLink. Multicast binding is switched off
    for these allocations (the kernels use no multimem instruction). One step on each rank, four
    launches on one stream, nothing on the host in between:

        rs_pass1 (sync)     every CTA announces "my gradients are ready" and waits for every
                            rank's; pull + average my slice, norm partials, pair -> every table;
                            the last CTA announces "my pair is written"
        finalize (sync)     waits for every rank's pair; replicated, rank-ordered: identical
                            state bits everywhere
        pass2_ag            AdamW on my slice, fp16 weights -> every arena
        barrier             announces "my weights have landed", waits for every rank's, advances
                            the step counter that lives in the flag block

    The NVLink bytes can be moved by the copy engines instead, phase by phase; the results are
    the same bits. rs_mover: "sm" (peer loads of the kernel), "ce_pull" (peers' slices pulled into
    local staging, b200amp_rs_pass1_f16_ce) or "ce_push" (every rank writes its slices into the
    owners' staging rows, b200amp_rs_push_f16_ce + b200amp_rs_pass1_f16_pushed). ag_mover: "sm"
    (peer stores of the kernel) or "ce" (pieces pushed under pass 2, b200amp_pass2_ag_f16_ce).
    `pieces` sets the pipelining of the copy-engine forms.

    Every wait is bounded (several seconds by default; `wait_limit` polls). A rank that never shows up makes
    the others' kernels return without applying the step; read_state() then raises
    RankWaitError naming the phase and the missing rank. The averaged gradient is rounded to
    fp16 once from an fp32 sum, so it is at least as accurate as an fp16 NCCL reduction; norm and
    flag are taken on exactly the stored averaged values.
    """

    PHASE_NAMES = ("gradients ready", "pairs written", "weights written", "a pushed piece of gradients")

    def __init__(self, slots: List[ParamSlot], cfg: ScheduleConfig, eps: float = 1e-8,
                 loss_scale: float = 65536.0, history_len: int = 256, device=None, group=None,
                 rs_mover: str = "sm", ag_mover: str = "sm", pieces: int = 4, wait_limit: int = 0):
        import os
        import torch.distributed as dist
        # the kernels use plain peer loads and stores: do not bind the arenas to an NVLink multicast
        # object (a rank that dies while bound to one can fault its peers' GPUs)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        if rs_mover not in ("sm", "ce_pull", "ce_push"):
            raise ValueError(f"rs_mover = {rs_mover!r}: expected 'sm', 'ce_pull' or 'ce_push'")
        if ag_mover not in ("sm", "ce"):
            raise ValueError(f"ag_mover = {ag_mover!r}: expected 'sm' or 'ce'")
        self.rs_mover, self.ag_mover, self.pieces = rs_mover, ag_mover, pieces
        self._symm_mem = symm_mem
        self._symm_group = group if group is not None else dist.group.WORLD
        self._handles = {}
        super().__init__(slots, cfg, eps, loss_scale, history_len, device, group)
        with torch.cuda.device(self.device):
            self.pairs = symm_mem.empty(2 * self.world, dtype=torch.float64, device=self.device)
            self.pairs.zero_()
            self.sync_block = symm_mem.empty(_lib.ZERO1_SYNC_BYTES // 4, dtype=torch.int32, device=self.device)
            zero1_sync_init(self.sync_block)
            torch.cuda.current_stream().synchronize()
            for name in ("pairs", "sync_block", "grads16", "weights16"):
                self._handles[name] = symm_mem.rendezvous(getattr(self, name), self._symm_group)
            shard_bytes = self.begin * 2
            self._grad_ptrs = [int(p) + shard_bytes for p in self._handles["grads16"].buffer_ptrs]
            self._weight_ptrs = [int(p) + shard_bytes for p in self._handles["weights16"].buffer_ptrs]
            self._pair_ptrs = [int(p) for p in self._handles["pairs"].buffer_ptrs]
            self.sync = make_sync([int(p) for p in self._handles["sync_block"].buffer_ptrs], wait_limit)
            self.staging = None             # ce_pull: (world - 1) slices, local, allocated on first use
            self.push_rows = None           # ce_push: world rows of one slice, mapped by every rank (below)
            self._push_ptrs = None
            torch.cuda.current_stream().synchronize()
        if rs_mover == "ce_push":
            self.enable_push()
        # once, on the host: every rank's block is zeroed and mapped before any rank announces anything
        dist.barrier(group=self._symm_group)

    def enable_push(self) -> None:
        """Allocates and maps the staging rows the ce_push reduce-scatter writes into. Collective:
        every rank calls it."""
        if self.push_rows is not None or self.world == 1:
            return
        with torch.cuda.device(self.device):
            self.push_rows = self._symm_mem.empty(self.world * self.n_local, dtype=torch.float16, device=self.device)
            self.push_rows.zero_()
            torch.cuda.current_stream().synchronize()
            self._handles["push_rows"] = self._symm_mem.rendezvous(self.push_rows, self._symm_group)
            self._push_ptrs = [int(p) for p in self._handles["push_rows"].buffer_ptrs]

    def _alloc_arena16(self, name: str) -> torch.Tensor:
        with torch.cuda.device(self.device):
            t = self._symm_mem.empty(self.n, dtype=torch.float16, device=self.device)
            t.zero_()
            return t

    def fused_pass1(self) -> None:
        if self.world > 1 and self.rs_mover == "ce_pull":
            if self.staging is None:
                self.staging = torch.empty((self.world - 1) * self.n_local, dtype=torch.float16, device=self.device)
            rs_pass1_f16_ce(self._grad_ptrs, self.rank, self.staging, self.grad_shard, self.n_local, self.pieces,
                            self.state, self.workspace, self._pair_ptrs, self.sync)
        elif self.world > 1 and self.rs_mover == "ce_push":
            if self._push_ptrs is None:
                raise RuntimeError("rs_mover 'ce_push' needs enable_push() on every rank first")
            rs_push_f16_ce(self.grads16, self._push_ptrs, self.rank, self.n_local, self.pieces, self.sync)
            rs_pass1_f16_pushed(self.grads16[self.begin:self.end], self.push_rows, self.world, self.rank,
                                self.grad_shard, self.n_local, self.pieces, self.state, self.workspace,
                                self._pair_ptrs, self.sync)
        else:
            rs_pass1_f16_sync(self._grad_ptrs, self.rank, self.grad_shard, self.n_local, self.state, self.workspace,
                              self._pair_ptrs, self.sync)

    def finalize_pairs(self) -> None:
        finalize_sums_sync(self.state, self.pairs, self.world, self.rank, self.sched, self.sync, self.history,
                           self.history_len)

    def fused_pass2(self) -> None:
        if self.world > 1 and self.ag_mover == "ce":
            pass2_ag_f16_ce(self.master, self.m, self.v, self.grad_shard, self._weight_ptrs, self.rank,
                            self.n_local, self.begin, self.tensors, self.ntensors, self.state, self.beta1,
                            self.beta2, self.eps, self.pieces)
        else:
            pass2_ag_f16(self.master, self.m, self.v, self.grad_shard, self._weight_ptrs, self.n_local, self.begin,
                         self.tensors, self.ntensors, self.state, self.beta1, self.beta2, self.eps)

    # -- HostGradientFeed: a second gradient arena that every rank maps (collective on first use)
    def _feed_arenas(self):
        with torch.cuda.device(self.device):
            alt = self._symm_mem.empty(self.n, dtype=torch.float16, device=self.device)
            alt.zero_()
            torch.cuda.current_stream().synchronize()
            self._handles["grads16_alt"] = self._symm_mem.rendezvous(alt, self._symm_group)
            shard_bytes = self.begin * 2
            self._feed_grad_ptrs = [self._grad_ptrs,
                                    [int(p) + shard_bytes for p in self._handles["grads16_alt"].buffer_ptrs]]
            self._feed_grads = [self.grads16, alt]
        return self._feed_grads

    def _feed_step(self, slot: int) -> None:
        keep_ptrs, keep_arena = self._grad_ptrs, self.grads16
        self._grad_ptrs, self.grads16 = self._feed_grad_ptrs[slot], self._feed_grads[slot]
        try:
            self.optimizer_step()
        finally:
            self._grad_ptrs, self.grads16 = keep_ptrs, keep_arena

    def end_step(self) -> None:
        zero1_barrier(self.sync, self.world, self.rank, _lib.PHASE_WEIGHTS,
                      _lib.SYNC_SIGNAL | _lib.SYNC_WAIT | _lib.SYNC_ADVANCE)

    def optimizer_step(self) -> None:
        with torch.cuda.device(self.device):
            self.fused_pass1()
            self.finalize_pairs()
            self.fused_pass2()
            self.end_step()

    def sync_status(self) -> Tuple[int, int]:
        """(steps the flag block has counted, error word); synchronises this rank's stream."""
        with torch.cuda.device(self.device):
            return zero1_sync_read(self.sync_block)

    def read_state(self) -> StepState:
        """The 60-byte state; raises RankWaitError if a kernel of this rank stopped waiting for
        another rank (the step in flight was not applied and the ranks are out of step: restore
        a checkpoint and build the optimizers again)."""
        self.drain_host_feed()          # steps submitted through the host feed run on their own stream
        st = super().read_state()
        _, error = self.sync_status()
        if error != 0:
            phase, missing = (error & 0xFF) - 1, error >> 8
            what = self.PHASE_NAMES[phase] if 0 <= phase < 4 else f"phase {phase}"
            raise RankWaitError(_lib.ERR_CUDA, f"rank {self.rank} gave up waiting for '{what}' of rank {missing}; "
                                "the step was not applied")
        return st
