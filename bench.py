#!/usr/bin/env python
"""Benchmark of the AMP AdamW optimizer step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over the whole parameter arena: pass 1 (unscale +
inf/NaN flag + squared-norm partials + finalize) and pass 2 (clip + AdamW on fp32
master/m/v + fp16 weight cast) on loss-scaled fp16 gradients. The default workload is the
1.3 B-parameter arena (L24 H16 C2048 Vp50304 n_ctx2048, 1,315,819,520 parameters, 292
tensors); at N > 1 the same arena is sharded ZeRO-1 style over the ranks (strong scaling):
reduce-scatter of fp16 gradients, the two passes on the shard, a 16-byte exchange for the
norm and flag, and an all-gather of the fp16 weights.

Prints ONE JSON line (rank 0). `value` is Gparams/s with every input resident in HBM;
`e2e` is the same metric when each step first copies its fp16 gradients from pinned host
memory and ends with a device-to-host read of the 60-byte step state. `roofline` is the
dominant kernel (pass 2, 28 algorithmic bytes per parameter) against the measured HBM copy
bandwidth, or at N > 1 against the NVLink copy bandwidth measured in the same run.
`cpu_baseline` / `--impl reference` time the reference's PyTorch CPU path (torch AdamW +
GradScaler + clip_grad_norm_) on the host cores over the whole arena of the same workload.
`reference_cuda_kernels` (N = 1, when the reference's own kernels were built for sm_100a) times
the reference's launches on the same arenas in the same process. At N > 1 `parity` holds the
checks of one extra step and of one skipped step made after the timed region; a mismatch exits
non-zero.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

METRIC = "amp_adamw_step_throughput"
UNIT = "Gparams/s"
BYTES_PASS1 = 2            # per parameter: read the fp16 gradient
BYTES_PASS2 = 28           # read g16 2 + master 4 + m 4 + v 4; write master 4 + m 4 + v 4 + fp16 weight 2
BYTES_STEP = BYTES_PASS1 + BYTES_PASS2
# DRAM traffic of pass 2 per element, from one ncu capture (dram__bytes_read.sum +
# dram__bytes_write.sum) of a launch on the gpt2-small arena: 1.742767 GB read + 1.684984 GB
# written over 124,476,416 elements. Every element is touched once, so traffic scales with the
# element count; the 1.3 B arena is too large to capture under ncu's replay.
PASS2_DRAM_BYTES_PER_PARAM_NCU = 27.54
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
NVLINK_FALLBACK_GBS = 770.0     # per direction per GPU; used only if the in-run copy measurement fails
REF_KERNELS_LIB = os.path.join(REPO, "oracle", "_ref", "libref_amp.so")


def measured_hbm_peak():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------- clocks

class ClockSampler:
    """nvidia-smi in the background during the timed region (read-only queries)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_indices):
        self.gpus = set(int(g) for g in gpu_indices)
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, smax = [], set(), None
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 8 or not f[0].isdigit() or int(f[0]) not in self.gpus:
                    continue
                try:
                    sm.append(float(f[1]))
                    smax = float(f[2])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     f[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            # "under load": the upper half of the samples (idle samples before/after the region drop out)
            sm.sort()
            out["sm_mhz"] = statistics.median(sm[len(sm) // 2:])
            out["samples"] = len(sm)
        out["sm_max_mhz"] = smax
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------- workloads

def workload_slots(name: str):
    from cuda_transformer_b200.layout import CONFIGS, param_layout
    return param_layout(CONFIGS[name])


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_cpu_reference(workload: str, steps: int, warmup: int) -> dict:
    """The reference's PyTorch CPU path (reference/train.py:147-153 order, the optimizer of
    reference/model.py:254-260) on the host cores, over every tensor of the workload's arena.
    If the host cannot hold the arena four times over in fp32, the largest prefix of the arena
    that fits is timed instead and the line says so."""
    import torch
    from oracle.torch_ref import time_cpu_step
    # every host core the process may use: torchrun exports OMP_NUM_THREADS=1, which would
    # otherwise pin the CPU path to one thread
    cores = host_cores()
    torch.set_num_threads(max(1, cores))
    slots = workload_slots(workload)
    shapes = [s.shape for s in slots]
    total = sum(s.count for s in slots)
    what = f"the whole {workload} arena ({len(shapes)} tensors)"
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = None
    need = total * 26                       # params, .grad, m, v in fp32, the fp16 gradients, and slack
    if avail is not None and need > 0.8 * avail:
        keep, acc = [], 0
        for s in slots:
            if (acc + s.count) * 26 > 0.8 * avail:
                break
            keep.append(s.shape)
            acc += s.count
        shapes = keep
        what = (f"the first {len(keep)} of {len(slots)} tensors of the {workload} arena ({acc:,} of {total:,} "
                f"parameters: the host has {avail / 2**30:.0f} GiB free, the whole arena needs {need / 2**30:.0f})")
    r = time_cpu_step(shapes, steps=max(1, steps), warmup=max(1, warmup), loss_scale=32768.0)
    gps = r["params"] / r["seconds_per_step"] / 1e9
    return {"value": gps, "unit": UNIT, "cores": r["threads"], "kind": "port",
            "sample": f"{what}: {r['params']:,} params/step, median of {max(1, steps)} steps; "
                      "torch.optim.AdamW(foreach=False) + GradScaler('cpu') + clip_grad_norm_, "
                      f"host has {os.cpu_count()} logical cores",
            "whole_arena": r["params"] == total,
            "ms_per_step": r["seconds_per_step"] * 1e3, "params": r["params"]}


# ---------------------------------------------------------------------------- GPU arm

def fill_normal_(t, std, seed, chunk=1 << 27):
    """t ~ N(0, std) from a seeded device generator, in chunks (no arena-sized temporary)."""
    import torch
    gen = torch.Generator(device=t.device).manual_seed(seed)
    for at in range(0, t.numel(), chunk):
        sl = t[at:at + chunk]
        sl.copy_(torch.randn(sl.numel(), generator=gen, device=t.device, dtype=torch.float32) * std)


def checksum(t):
    """Two 64-bit sums over the bit patterns of a tensor (plain and position-weighted), on the
    device in chunks. Equal arrays give equal pairs; a changed or moved element changes them."""
    import torch
    bits = t.view(torch.int16) if t.element_size() == 2 else t.view(torch.int32)
    a = torch.zeros((), dtype=torch.int64, device=t.device)
    b = torch.zeros((), dtype=torch.int64, device=t.device)
    chunk = 1 << 26
    for at in range(0, bits.numel(), chunk):
        x = bits[at:at + chunk].to(torch.int64)
        a += x.sum()
        w = (torch.arange(at, at + x.numel(), device=t.device, dtype=torch.int64) % 65521) + 1
        b += (x * w).sum()
    return torch.stack([a, b])


def reference_cuda_kernels_leg(opt, amp, torch, reps: int) -> dict:
    """The reference's own launches on this GPU, same process, same arenas: begin_step ->
    unscale_and_norm -> finalize_step -> adamw_multi (cuda/gpt_fast.cu:438-450) plus the per-step
    grads.zero memset (cuda/gpt_fast.cu:455), compiled from the reference's sources for sm_100a.
    The fp32 gradient arena is refilled from the fp16 gradients between repetitions, outside the
    timed events. Runs last: it steps master / m / v with its own copy of the step state."""
    lib = ctypes.CDLL(REF_KERNELS_LIB)
    P, LL, I, F = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    lib.refamp_begin_step.argtypes = [P, P]
    lib.refamp_unscale_and_norm.argtypes = [P, LL, P, P, P]
    lib.refamp_finalize_step.argtypes = [P, P, P, P, I, P]
    lib.refamp_adamw_multi.argtypes = [P, P, P, P, P, LL, P, I, P, F, F, F, P]
    for fn in (lib.refamp_begin_step, lib.refamp_unscale_and_norm, lib.refamp_finalize_step, lib.refamp_adamw_multi):
        fn.restype = None
    n = opt.n
    g32 = torch.empty(n, dtype=torch.float32, device=opt.device)
    partial = torch.zeros(512, dtype=torch.float32, device=opt.device)
    state = opt.state.clone()
    history = torch.zeros_like(opt.history)
    s = torch.cuda.current_stream().cuda_stream
    cfg = opt.sched
    chunk = 1 << 27

    def refill():
        for at in range(0, n, chunk):
            g32[at:at + chunk].copy_(opt.grads16[at:at + chunk])

    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(reps + 1)]
    for k in range(reps + 1):                       # repetition 0 warms up
        refill()
        marks[k][0].record()
        lib.refamp_begin_step(state.data_ptr(), s)
        lib.refamp_unscale_and_norm(g32.data_ptr(), n, state.data_ptr(), partial.data_ptr(), s)
        lib.refamp_finalize_step(state.data_ptr(), partial.data_ptr(), ctypes.addressof(cfg), history.data_ptr(),
                                 opt.history_len, s)
        marks[k][1].record()
        lib.refamp_adamw_multi(opt.master.data_ptr(), opt.weights16.data_ptr(), g32.data_ptr(), opt.m.data_ptr(),
                               opt.v.data_ptr(), n, opt.tensors.data_ptr(), opt.ntensors, state.data_ptr(),
                               cfg.beta1, cfg.beta2, opt.eps, s)
        marks[k][2].record()
        g32.zero_()                                  # a cudaMemsetAsync, as grads.zero
        marks[k][3].record()
    torch.cuda.synchronize()

    def avg(i, j):
        return sum(marks[k][i].elapsed_time(marks[k][j]) for k in range(1, reps + 1)) / reps

    del g32
    return {"ms_per_step": avg(0, 3),
            "kernels_ms": {"begin_step+unscale_and_norm+finalize_step": avg(0, 1), "adamw_multi": avg(1, 2),
                           "grads_zero_memset": avg(2, 3)},
            "bytes_per_param": 42, "steps": reps,
            "what": "the reference's scaler.cu + adamw_multi.cu compiled from its sources for sm_100a: fp32 "
                    "gradient arena unscaled in place, three launches + begin_step + memset, same arenas"}


def nvlink_probe(opt, amp, torch, dist, world, rank, max_over_ranks) -> dict:
    """The NVLink rate this run's GPUs reach with both directions of every pair busy: every rank
    exchanges up to 1 GiB with rank ^ 1 through the mapped gradient arenas, all pairs at once.
    Copy engine (cudaMemcpyAsync) pulling and pushing, and SM-issued loads (the fused
    reduce-scatter kernel with one source, the peer's arena). GB/s per direction, slowest rank."""
    out = {}
    try:
        peer = rank ^ 1
        handle = opt._handles["grads16"]
        peer_base = int(handle.buffer_ptrs[peer])
        size = min(1 << 30, opt.n) // 4096 * 4096                   # bytes; at most half of the 2n-byte arena
        local = torch.empty(size // 2, dtype=torch.float16, device=opt.device)
        peer_upper = peer_base + opt.n * 2 - size                   # pulls read the peer's lower half, pushes
                                                                    # land in its upper half

        def timed(fn, reps=3):
            fn()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return size / (max_over_ranks(e0.elapsed_time(e1)) / reps * 1e-3) / 1e9

        out["copy_engine_pull_gbs"] = timed(lambda: amp.copy_async(local, peer_base, size))
        out["copy_engine_push_gbs"] = timed(lambda: amp.copy_async(peer_upper, local, size))
        ws = torch.zeros_like(opt.workspace)
        out["sm_loads_gbs"] = timed(lambda: amp.rs_pass1_f16([peer_base], 0, local, size // 2, opt.state, ws))
        out["bytes"] = size
        out["pattern"] = "rank r <-> rank r^1, every pair at once, both directions busy"
        del local
        dist.barrier()
        torch.cuda.synchronize()
    except Exception as e:      # noqa: BLE001
        out["error"] = f"{type(e).__name__}: {e}"[:200]
    return out


def mover_sweep(opt, amp, lib, torch, dist, world, max_over_ranks, n, steps=10) -> list:
    """Per-phase times of the fused ZeRO-1 step with each mover of the NVLink bytes, on the optimizer
    the timed region used (the settings give the same bits; only who moves the bytes changes):
    kernel-issued peer loads / stores, copy engines pulling, copy engines pushing, for 2 / 4 / 8
    pieces and 2 or world - 1 copy streams. CUDA events around the four launches, max over ranks."""
    from cuda_transformer_b200 import _lib
    link = (world - 1) / world * 2 * n
    opt.enable_push()
    settings = [("sm", "sm", 1, 2)]
    for rs, ag in (("ce_pull", "sm"), ("ce_push", "sm"), ("sm", "ce"), ("ce_push", "ce")):
        for pieces in (2, 4, 8):
            for lanes in sorted(set(min(x, world - 1) for x in (2, 7))):
                settings.append((rs, ag, pieces, lanes))
    keep = (opt.rs_mover, opt.ag_mover, opt.pieces)
    rows = []
    for rs, ag, pieces, lanes in settings:
        opt.rs_mover, opt.ag_mover, opt.pieces = rs, ag, pieces
        _lib.check(lib.b200amp_tune_set(b"ce_lanes", lanes))
        for _ in range(2):
            opt.optimizer_step()
        torch.cuda.synchronize()
        dist.barrier()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
        for k in range(steps):
            ev[k][0].record()
            opt.fused_pass1()
            ev[k][1].record()
            opt.finalize_pairs()
            ev[k][2].record()
            opt.fused_pass2()
            ev[k][3].record()
            opt.end_step()
            ev[k][4].record()
        torch.cuda.synchronize()
        dist.barrier()

        def avg(i, j):
            return max_over_ranks(sum(ev[k][i].elapsed_time(ev[k][j]) for k in range(steps)) / steps)

        row = {"rs_mover": rs, "ag_mover": ag, "pieces": pieces, "copy_streams": lanes, "step_ms": avg(0, 4),
               "rs_ms": avg(0, 1), "finalize_wait_ms": avg(1, 2), "ag_ms": avg(2, 3), "end_barrier_ms": avg(3, 4)}
        row["rs_nvlink_gbs"] = link / row["rs_ms"] / 1e6
        row["ag_nvlink_gbs"] = link / row["ag_ms"] / 1e6
        st = opt.read_state()                       # raises if a wait on another rank gave up
        row["skipped"] = st.skipped
        rows.append(row)
    opt.rs_mover, opt.ag_mover, opt.pieces = keep
    _lib.check(lib.b200amp_tune_set(b"ce_lanes", 2))
    return rows


def run_gpu(args) -> dict:
    import torch
    import torch.distributed as dist
    from cuda_transformer_b200 import _lib, amp
    from cuda_transformer_b200.layout import padded

    fused = False
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N > 1 with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    lib = _lib.load()
    _lib.check(lib.b200amp_device_check())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    slots = workload_slots(args.workload)
    n_params = slots[-1].offset + slots[-1].count
    n = padded(n_params)
    loss_scale = 32768.0
    cfg = amp.make_schedule(lr=6e-4, min_lr=6e-4, beta1=0.9, beta2=0.95, weight_decay=0.1, grad_clip=1.0,
                            growth_interval=2000, dynamic_scale=1)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def min_over_ranks(x: float) -> float:
        return -max_over_ranks(-x)

    runs = None
    if world == 1:
        opt = amp.AmpOptimizer(slots, cfg, eps=1e-8, loss_scale=loss_scale, device=dev)
        fill_normal_(opt.master[:n_params], 0.02, seed=0)
        amp.cast_to_x(opt.weights16, opt.master, n)
        if args.pass2 == "runs":
            runs = opt.decay_runs()

        def step_fn():
            opt.optimizer_step(pass2=args.pass2)
    else:
        fused = args.collectives == "fused"
        fused_note = None
        if fused:
            # symmetric memory needs peer access between all ranks' GPUs; where the box cannot give
            # it, every rank falls back together to NCCL around the passes (and the line says so)
            try:
                opt = amp.FusedZero1Optimizer(slots, cfg, eps=1e-8, loss_scale=loss_scale, device=dev,
                                              rs_mover=args.rs_mover, ag_mover=args.ag_mover, pieces=args.pieces)
                ok = torch.ones(1, device=dev)
            except Exception as e:      # noqa: BLE001
                opt, ok, fused_note = None, torch.zeros(1, device=dev), f"{type(e).__name__}: {e}"[:200]
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok.item()) < 1.0:
                fused = False
                opt = None
                torch.cuda.empty_cache()
        if not fused:
            opt = amp.ShardedAmpOptimizer(slots, cfg, eps=1e-8, loss_scale=loss_scale, device=dev)
        # the same master values as the 1-GPU run would hold in this slice would need the whole
        # stream; a per-rank seed gives the same distribution, which is all the timing needs
        fill_normal_(opt.master, 0.02, seed=100 + rank)
        opt.weights16.zero_()
        amp.cast_to_x(opt.weights16[opt.begin:opt.end], opt.master, opt.n_local)
        opt.all_gather_weights()
        step_fn = opt.optimizer_step

    # fp16 gradients = N(0, 1e-3) * loss_scale, generated on the device (rank r: seed r + 1)
    def fill_grads(seed):
        gen = torch.Generator(device=dev).manual_seed(seed)
        chunk = 1 << 27
        for at in range(0, n_params, chunk):
            m_ = min(chunk, n_params - at)
            opt.grads16[at:at + m_].copy_(
                (torch.randn(m_, generator=gen, device=dev, dtype=torch.float32) * (1e-3 * loss_scale)).half())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # m and v pre-warmed by 5 seeded steps of the implementation itself (untimed)
    for k in range(5):
        fill_grads(1000 * (k + 1) + rank + 1)
        barrier()
        step_fn()
    barrier()
    nvlink = {}
    if fused:
        nvlink = nvlink_probe(opt, amp, torch, dist, world, rank, max_over_ranks)    # overwrites gradients
    fill_grads(rank + 1)
    barrier()
    st = opt.read_state()
    if st.skipped != 0 or st.adam_t != 5:
        raise SystemExit(f"pre-warm went wrong: {st.as_dict()}")

    # ------------------------------------------------------------------ device-resident timing
    for _ in range(args.warmup):
        step_fn()
    barrier()
    sampler = ClockSampler(range(world))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    launches_before = lib.b200amp_launch_count()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(args.steps)]
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record()
    if world == 1:
        for k in range(args.steps):
            ev[k][0].record()
            amp.pass1_finalize_f16(opt.grads16, opt.n, opt.state, opt.workspace, opt.sched, opt.history,
                                   opt.history_len)
            ev[k][1].record()
            if runs is not None:
                amp.pass2_f16_runs(opt.master, opt.m, opt.v, opt.grads16, opt.weights16, opt.n, 0, runs, opt.state,
                                   opt.beta1, opt.beta2, opt.eps)
            else:
                amp.pass2_f16(opt.master, opt.m, opt.v, opt.grads16, opt.weights16, opt.n, 0, opt.tensors,
                              opt.ntensors, opt.state, opt.beta1, opt.beta2, opt.eps)
            ev[k][2].record()
    elif fused:
        for k in range(args.steps):
            ev[k][0].record()
            opt.fused_pass1()
            ev[k][1].record()
            opt.finalize_pairs()
            ev[k][2].record()
            opt.fused_pass2()
            ev[k][3].record()
            opt.end_step()
            ev[k][4].record()
    else:
        for k in range(args.steps):
            ev[k][0].record()
            opt.reduce_scatter_grads()
            ev[k][1].record()
            opt._pass1()
            ev[k][2].record()
            opt.gather_sums()
            opt._finalize()
            ev[k][3].record()
            opt._pass2()
            ev[k][4].record()
            opt.all_gather_weights()
            ev[k][5].record()
    t_end.record()
    barrier()
    launches = lib.b200amp_launch_count() - launches_before
    total_ms = max_over_ranks(t_begin.elapsed_time(t_end))
    if rank == 0:
        time.sleep(0.2)
        clocks = sampler.stop()
    ms_per_step = total_ms / args.steps

    def avg(i, j):
        return sum(ev[k][i].elapsed_time(ev[k][j]) for k in range(args.steps)) / args.steps

    phases = {}
    coll_bytes = (world - 1) / world * 2 * n                # per GPU per direction, each collective
    if world == 1:
        pass1_ms, pass2_ms = avg(0, 1), avg(1, 2)
        n_local = n
    elif fused:
        # the first kernel of a step is where a rank that arrives early waits for the others
        phases = {"rs_pass1_ms": max_over_ranks(avg(0, 1)), "wait_finalize_ms": max_over_ranks(avg(1, 2)),
                  "pass2_ag_ms": max_over_ranks(avg(2, 3)), "end_barrier_ms": max_over_ranks(avg(3, 4))}
        pass1_ms, pass2_ms = phases["rs_pass1_ms"], phases["pass2_ag_ms"]
        n_local = opt.n_local
        phases["rs_pass1_nvlink_gbs"] = coll_bytes / (phases["rs_pass1_ms"] * 1e-3) / 1e9
        phases["pass2_ag_nvlink_gbs"] = coll_bytes / (phases["pass2_ag_ms"] * 1e-3) / 1e9
        if args.rs_mover != "sm" or args.ag_mover != "sm":
            phases["collectives"] = (f"reduce-scatter mover {args.rs_mover}, all-gather mover {args.ag_mover}, "
                                     f"{args.pieces} pieces (sm: peer loads / stores issued by the fused kernel; "
                                     "ce_*: cudaMemcpyAsync under kernels that touch local memory only); ranks "
                                     "ordered by the library's flag words, every wait bounded")
        else:
            phases["collectives"] = ("fused into the passes: plain peer loads (rs_pass1) and peer stores "
                                     "(pass2_ag); ranks ordered by the library's flag words, every wait bounded")
    else:
        phases = {"reduce_scatter_ms": max_over_ranks(avg(0, 1)), "pass1_ms": max_over_ranks(avg(1, 2)),
                  "norm_gather_finalize_ms": max_over_ranks(avg(2, 3)), "pass2_ms": max_over_ranks(avg(3, 4)),
                  "all_gather_ms": max_over_ranks(avg(4, 5))}
        pass1_ms, pass2_ms = phases["pass1_ms"], phases["pass2_ms"]
        n_local = opt.n_local
        phases["reduce_scatter_gbs"] = coll_bytes / (phases["reduce_scatter_ms"] * 1e-3) / 1e9
        phases["all_gather_gbs"] = coll_bytes / (phases["all_gather_ms"] * 1e-3) / 1e9
        phases["collectives"] = "NCCL reduce_scatter_tensor(AVG) / all_gather_into_tensor around the passes"
        if args.collectives == "fused":
            phases["collectives"] += " (fused path unavailable on this box: %s)" % (fused_note or "a peer rank failed")
    if nvlink:
        phases["nvlink_measured_in_run"] = nvlink
    st = opt.read_state()
    if st.skipped != 0:
        raise SystemExit("a timed step was skipped: the timing would count 2 B/param steps")

    # ------------------------------------------------------------------ end to end: host gradients in, state out
    e2e_steps = max(3, min(args.steps, 10))
    host_grads = torch.empty(n, dtype=torch.float16, pin_memory=True)
    host_grads.copy_(opt.grads16)
    host_state = torch.empty(opt.state.numel(), dtype=torch.uint8, pin_memory=True)
    torch.cuda.synchronize()

    pipelined = hasattr(opt, "submit_host_gradients")
    if pipelined:
        # The optimizer's own host feed (HostGradientFeed): two device gradient arenas take turns, so
        # step k + 1's copy from pinned memory overlaps step k's kernels. Every step's gradients are
        # copied and every step's 60-byte state is read back inside the timed region.
        def e2e_run(count):
            last = None
            for _ in range(count):
                ticket = opt.submit_host_gradients(host_grads)
                if last is not None:
                    opt.collect(last)               # a real host sync on the previous step's result
                last = ticket
            return opt.collect(last)

        e2e_run(2)                                  # both arenas touched, streams and mappings set up
        opt.drain_host_feed()
        barrier()
        copy_stream, step_stream = opt.host_feed_streams()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(copy_stream)
        last_state = e2e_run(e2e_steps)
        e1.record(step_stream)
        opt.drain_host_feed()
        barrier()
        if last_state.skipped != 0:
            raise SystemExit("an end-to-end step was skipped")
    else:
        def e2e_step():
            opt.grads16.copy_(host_grads, non_blocking=True)
            step_fn()
            host_state.copy_(opt.state, non_blocking=True)
            torch.cuda.current_stream().synchronize()   # the caller reads the state: a real host sync

        e2e_step()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps

    # where the end-to-end time goes: the host-to-device copy of one rank alone, and of all ranks at once
    h2d = {}

    def h2d_gbs():
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        opt.grads16.copy_(host_grads, non_blocking=True)
        b.record()
        torch.cuda.synchronize()
        return 2 * n / (a.elapsed_time(b) * 1e-3) / 1e9

    if world > 1:
        alone = 0.0
        for r in range(world):
            barrier()
            if r == rank:
                alone = h2d_gbs()
        barrier()
        together = h2d_gbs()
        barrier()
        h2d = {"h2d_gbs_one_rank_alone_min": min_over_ranks(alone), "h2d_gbs_one_rank_alone_max": max_over_ranks(alone),
               "h2d_gbs_all_ranks_at_once_min": min_over_ranks(together),
               "h2d_gbs_all_ranks_at_once_max": max_over_ranks(together)}
    else:
        h2d = {"h2d_gbs": h2d_gbs()}

    graph_replay = None
    if world == 1:
        # The same step as ONE CUDA-graph launch (how the reference's trainer replays it,
        # cuda/train_fast.cu:720-730): per-replay times by events, median reported.
        side = torch.cuda.Stream(device=dev)
        graph = amp.CudaGraph()
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            graph.capture(side, lambda: opt.optimizer_step(side, pass2=args.pass2))
            for _ in range(3):
                graph.launch(side)
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
            marks[0].record(side)
            for k in range(args.steps):
                graph.launch(side)
                marks[k + 1].record(side)
        side.synchronize()
        times = sorted(marks[k].elapsed_time(marks[k + 1]) for k in range(args.steps))
        graph_replay = {"median_ms": statistics.median(times), "min_ms": times[0], "max_ms": times[-1],
                        "replays": args.steps}
        if opt.read_state().skipped != 0:
            raise SystemExit("a graph replay was skipped")

    skipped_step = None
    if world == 1:
        # A skipped step (an inf among the gradients) moves 2 B/param: pass 1 reads the arena, pass 2
        # returns at once. Timed apart from the metric; state and gradients are put back afterwards.
        saved_state, saved_head = opt.state.clone(), opt.grads16[:8].clone()
        opt.grads16[0] = float("inf")
        reps = 5
        step_fn()
        s0 = torch.cuda.Event(enable_timing=True)
        s1 = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s0.record()
        for _ in range(reps):
            step_fn()
        s1.record()
        torch.cuda.synchronize()
        if opt.read_state().skipped != reps + 1:
            raise SystemExit("the steps with an inf gradient were not skipped")
        skip_ms = s0.elapsed_time(s1) / reps
        skipped_step = {"ms_per_step": skip_ms, "hbm_gbs": BYTES_PASS1 * n / (skip_ms * 1e-3) / 1e9,
                        "bytes_per_param": BYTES_PASS1, "steps": reps}
        opt.state.copy_(saved_state)
        opt.grads16[:8].copy_(saved_head)
        torch.cuda.synchronize()

    sweep = None
    if world > 1 and fused and args.mover_sweep:
        sweep = mover_sweep(opt, amp, lib, torch, dist, world, max_over_ranks, n)

    parity = None
    if world > 1:
        parity = multi_gpu_parity(opt, amp, torch, dist, world, rank, dev, loss_scale, fused)

    ref_kernels = None
    if world == 1 and os.path.exists(REF_KERNELS_LIB) and not args.no_reference_kernels:
        free, _ = torch.cuda.mem_get_info()
        if free > 4 * n + (2 << 30):
            ref_kernels = reference_cuda_kernels_leg(opt, amp, torch, reps=5)

    peak, peak_kind = measured_hbm_peak()
    pass2_gbs = BYTES_PASS2 * n_local / (pass2_ms * 1e-3) / 1e9
    pass1_gbs = BYTES_PASS1 * n_local / (pass1_ms * 1e-3) / 1e9
    value = n_params / (ms_per_step * 1e-3) / 1e9
    hbm_gbs_step = BYTES_STEP * n_local / ((pass1_ms + pass2_ms) * 1e-3) / 1e9
    pass2_kernel = "pass2_f16_runs_kernel" if runs is not None else "pass2_f16_kernel"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {n_params:,} params, {len(slots)} tensors, fp16 grads "
                               f"N(0,1e-3)*{int(loss_scale)}, fp32 master/m/v, m and v pre-warmed by 5 steps, "
                               "AdamW lr 6e-4 betas (0.9,0.95) eps 1e-8 wd 0.1, clip 1.0",
                   "params": n_params, "arena": n, "parallelism": "single" if world == 1 else f"zero1-dp{world}",
                   "l2": "arenas are far larger than the 126 MB L2 (no flush needed between steps)"
                         if 18 * n_local > (1 << 30) else
                         "the shard's arenas (%d MB) are not far above the 126 MB L2" % (18 * n_local >> 20)},
        "hbm_gbs": hbm_gbs_step, "hbm_frac_of_nominal_8tbs": hbm_gbs_step / NOMINAL_HBM_GBS,
        "hbm_frac_of_measured": hbm_gbs_step / peak,
        "kernels_ms": {"pass1_finalize": pass1_ms, "pass2": pass2_ms},
        "roofline": {"bound": "hbm", "kernel": pass2_kernel, "achieved": pass2_gbs, "peak": peak,
                     "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s", "frac": pass2_gbs / peak,
                     "traffic": None, "algorithmic_bytes_per_launch": BYTES_PASS2 * n_local,
                     "pass1_achieved": pass1_gbs, "pass1_frac": pass1_gbs / peak},
        "e2e": {"value": n_params / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 2 * n, "d2h_bytes_per_step": int(opt.state.numel()), "steps": e2e_steps,
                "how": ("submit_host_gradients / collect: two gradient arenas take turns, the copy of step k + 1 "
                        "overlaps the kernels of step k" if pipelined else
                        "copy, step, read-back, one after the other"),
                **h2d},
        "gpu_launches": int(launches),
        "clocks": clocks if rank == 0 else None,
        "state": {k: v for k, v in st.as_dict().items() if k in ("step", "adam_t", "skipped", "loss_scale",
                                                                  "grad_norm", "clip_coef")},
    }
    if phases:
        line["phases"] = phases
    if skipped_step:
        line["skipped_step"] = skipped_step
    if graph_replay:
        line["graph_replay"] = graph_replay
    if parity is not None:
        line["parity"] = parity
    if sweep is not None:
        line["mover_sweep"] = sweep
    if ref_kernels is not None:
        ref_kernels["speedup"] = ref_kernels["ms_per_step"] / ms_per_step
        line["reference_cuda_kernels"] = ref_kernels
    line["roofline"]["traffic"] = PASS2_DRAM_BYTES_PER_PARAM_NCU * n_local
    line["roofline"]["traffic_source"] = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of the "
                                          "registers-only pass 2 on the gpt2-small arena, scaled by the element count")
    if world > 1 and fused:
        # A fused compute + collective kernel: its floor is the slower of the HBM time of its slice and
        # the time its bytes need on NVLink at the copy rate measured in this run (per direction per GPU).
        link_peak = max(nvlink.get("copy_engine_pull_gbs", 0.0), nvlink.get("copy_engine_push_gbs", 0.0))
        link_kind = "copy-engine rate between rank pairs measured in this run, both directions busy"
        if link_peak <= 0.0:
            link_peak, link_kind = NVLINK_FALLBACK_GBS, "fallback (the in-run copy measurement failed)"
        # HBM bytes of the fused pass 2 + all-gather on one GPU: 28 B per element of its own slice, plus
        # the 2 B per element of every other slice that the peers' stores write into this GPU's arena
        # while the kernel runs
        hbm_bytes = BYTES_PASS2 * n_local + 2 * (n - n_local)
        t_hbm = hbm_bytes / (peak * 1e9)
        t_link = coll_bytes / (link_peak * 1e9)
        by_link = t_link > t_hbm
        achieved = (coll_bytes if by_link else hbm_bytes) / (pass2_ms * 1e-3) / 1e9
        bound_peak = link_peak if by_link else peak
        line["roofline"].update({
            "bound": "nvlink" if by_link else "hbm",
            "kernel": "pass2_f16_kernel + cudaMemcpyAsync" if args.ag_mover == "ce" else "pass2_ag_f16_kernel",
            "achieved": achieved, "peak": bound_peak, "frac": achieved / bound_peak,
            "peak_kind": link_kind if by_link else f"{peak_kind} copy bandwidth",
            "algorithmic_bytes_per_launch": coll_bytes if by_link else hbm_bytes,
            "hbm_bytes_per_launch": hbm_bytes,
            "floor_ms": {"hbm": t_hbm * 1e3, "nvlink": t_link * 1e3}, "traffic": None,
            "traffic_source": None, "nvlink_bytes_per_launch": coll_bytes,
            "rs_pass1_frac_of_link_peak": phases["rs_pass1_nvlink_gbs"] / link_peak})
        line["kernels_ms"] = {"rs_pass1": pass1_ms, "pass2_ag": pass2_ms}
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        if rank == 0:
            print(json.dumps(line), flush=True)
        raise SystemExit("multi-GPU parity check failed: " + json.dumps(parity))
    return line if rank == 0 else None


def multi_gpu_parity(opt, amp, torch, dist, world, rank, dev, loss_scale, fused) -> dict:
    """One checked step and one skipped step after the timed region, on the real GPUs:

    * every rank's 60 state bytes are equal;
    * every rank's fp16 weight arena is equal (checksums, all-reduced MIN and MAX);
    * the rank's averaged gradient slice equals fp16(fp32 sum in rank order / R) of the slices
      gathered from all ranks (fused path; the NCCL path's own reduction order is not ours);
    * the rank's master / m / v / fp16 weights after the step equal, bit for bit, a replay of
      the one-GPU b200amp_pass2_f16 on a copy of the slice taken before the step, with the same
      reduced gradients and the same state;
    * the norm in the state agrees with an fp64 sum over all ranks' reduced slices to 1e-6;
    * an inf injected on the last rank: master, m, v and the weights stay bit-unchanged on
      every rank, the loss scale halves, adam_t stays, skipped advances (the expectations of
      the reference's scaler_checks, cuda/tests/test_fast.cu:272-326).
    """
    import numpy as np
    checks = {}

    def all_equal(t) -> bool:
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return bool(torch.equal(lo, hi))

    def everyone(ok: bool) -> bool:
        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(int(t.item()) == 1)

    nl = opt.n_local
    before = [t.clone() for t in (opt.master, opt.m, opt.v)]
    st0 = opt.read_state()
    opt.optimizer_step()
    torch.cuda.synchronize()
    st1 = opt.read_state()
    state_bytes = torch.frombuffer(bytearray(bytes(st1)), dtype=torch.uint8).to(dev).to(torch.int32)
    checks["state_bytes_equal_on_all_ranks"] = all_equal(state_bytes)
    checks["weights16_equal_on_all_ranks"] = all_equal(checksum(opt.weights16))
    checks["step_applied"] = everyone(st1.found_inf == 0 and st1.adam_t == st0.adam_t + 1 and st1.step == st0.step + 1)
    if fused:
        # the reduce-scatter against an independent reduction: one all-to-all brings slice `rank` of
        # every rank's gradient arena here, then fp32 sum in rank order, * 1/R, one rounding to fp16
        gathered = torch.empty(world * nl, dtype=torch.float16, device=dev)
        dist.all_to_all_single(gathered, opt.grads16[:world * nl])
        want = torch.zeros(nl, dtype=torch.float32, device=dev)
        for q in range(world):
            want += gathered[q * nl:(q + 1) * nl].float()
        same = bool(torch.equal((want * (1.0 / world)).half(), opt.grad_shard))
        del want, gathered
        checks["reduced_slice_is_fp16_of_fp32_sum_over_ranks"] = everyone(same)
    # replay of pass 2 on the copy taken before the step
    w16 = torch.zeros(nl, dtype=torch.float16, device=dev)
    amp.pass2_f16(before[0], before[1], before[2], opt.grad_shard, w16, nl, opt.begin, opt.tensors, opt.ntensors,
                  opt.state, opt.beta1, opt.beta2, opt.eps)
    torch.cuda.synchronize()
    replay_ok = (torch.equal(before[0], opt.master) and torch.equal(before[1], opt.m) and
                 torch.equal(before[2], opt.v) and torch.equal(w16, opt.weights16[opt.begin:opt.end]))
    checks["slice_equals_one_gpu_pass2_replay_bit_for_bit"] = everyone(bool(replay_ok))
    del before, w16
    sumsq = torch.zeros(1, dtype=torch.float64, device=dev)
    chunk = 1 << 26
    for at in range(0, nl, chunk):
        g = opt.grad_shard[at:at + chunk].double() / st0.loss_scale
        sumsq += (g * g).sum()
    dist.all_reduce(sumsq)
    norm = float(sumsq.item()) ** 0.5
    checks["grad_norm_rel_err_vs_fp64"] = abs(st1.grad_norm - norm) / norm
    checks["grad_norm_within_1e-6"] = checks["grad_norm_rel_err_vs_fp64"] <= 1e-6

    # a skipped step: an inf among the last rank's gradients
    sums_before = torch.cat([checksum(t) for t in (opt.master, opt.m, opt.v, opt.weights16)])
    saved = opt.grads16[opt.n // 2: opt.n // 2 + 8].clone()
    if rank == world - 1:
        opt.grads16[opt.n // 2 + 3] = float("inf")
    dist.barrier()
    opt.optimizer_step()
    torch.cuda.synchronize()
    st2 = opt.read_state()
    sums_after = torch.cat([checksum(t) for t in (opt.master, opt.m, opt.v, opt.weights16)])
    checks["skipped_step_leaves_master_m_v_weights_unchanged"] = everyone(bool(torch.equal(sums_before, sums_after)))
    checks["skipped_step_halves_the_scale_and_keeps_adam_t"] = everyone(
        st2.found_inf == 1 and st2.skipped == st1.skipped + 1 and st2.adam_t == st1.adam_t and
        st2.loss_scale == 0.5 * st1.loss_scale and st2.step == st1.step + 1)
    state2 = torch.frombuffer(bytearray(bytes(st2)), dtype=torch.uint8).to(dev).to(torch.int32)
    checks["state_bytes_equal_after_the_skipped_step"] = all_equal(state2)
    opt.grads16[opt.n // 2: opt.n // 2 + 8].copy_(saved)
    dist.barrier()
    ok = all(v for k, v in checks.items() if isinstance(v, (bool, np.bool_)))
    return {"ok": bool(ok), "ranks": world, **{k: (bool(v) if isinstance(v, (bool, np.bool_)) else v)
                                               for k, v in checks.items()}}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="1.3b", choices=["debug", "readme", "gpt2-small", "1.3b"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-kernels", action="store_true",
                    help="N = 1: skip the leg that times the reference's own CUDA kernels")
    ap.add_argument("--cpu-steps", type=int, default=3, help="timed steps of the cpu_baseline leg")
    ap.add_argument("--pass2", choices=["table", "runs"], default="table",
                    help="N = 1: decay flags from the tensor table in device memory, or as a kernel parameter")
    ap.add_argument("--collectives", choices=["fused", "nccl"], default="fused",
                    help="N > 1: fold reduce-scatter / all-gather into the passes, or call NCCL around them")
    ap.add_argument("--rs-mover", choices=["sm", "ce_pull", "ce_push"], default="sm",
                    help="N > 1, fused: who moves the reduce-scatter's bytes over NVLink (the kernel's peer loads, "
                         "or the copy engines pulling / pushing)")
    ap.add_argument("--ag-mover", choices=["sm", "ce"], default="sm",
                    help="N > 1, fused: who moves the all-gather's bytes (the kernel's peer stores, or the copy engines)")
    ap.add_argument("--pieces", type=int, default=4, help="pipelining of the copy-engine movers")
    ap.add_argument("--mover-sweep", action="store_true",
                    help="N > 1, fused: after the timed region, time the step's phases with every mover setting "
                         "(adds `mover_sweep` to the line)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    # plain peer loads and stores only: the symmetric allocations are not bound to a multicast object
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

    if args.impl == "reference":
        if rank != 0:
            return
        slots = workload_slots(args.workload)
        n_params = slots[-1].offset + slots[-1].count
        r = run_cpu_reference(args.workload, steps=args.steps, warmup=max(1, args.warmup))
        line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": f"{args.workload}: {n_params:,} params" +
                                       ("" if r["whole_arena"] else " (timed on a prefix of the arena, see "
                                                                    "cpu_baseline.sample)"), "params": n_params},
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "whole_arena")},
                "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return

    line = run_gpu(args)
    if line is None:
        return
    if not args.no_cpu_baseline:
        r = run_cpu_reference(args.workload, steps=args.cpu_steps, warmup=1)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "whole_arena")}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
