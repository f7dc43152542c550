#!/usr/bin/env python
"""Benchmark of the AMP AdamW optimizer step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over the whole parameter arena: pass 1 (unscale +
inf/NaN flag + squared-norm partials + finalize) and pass 2 (clip + AdamW on fp32
master/m/v + fp16 weight cast) on loss-scaled fp16 gradients. The default workload is the
1.3 B-parameter arena (L24 H16 C2048 Vp50304 n_ctx2048, 1,315,819,520 parameters, 292
tensors); at N > 1 the same arena is sharded ZeRO-1 style over the ranks (strong scaling):
reduce-scatter of fp16 gradients, the two passes on the shard, a 16-byte all-gather for the
norm and flag, and an all-gather of the fp16 weights.

Prints ONE JSON line (rank 0). `value` is Gparams/s with every input resident in HBM;
`e2e` is the same metric when each step first copies its fp16 gradients from pinned host
memory and ends with a device-to-host read of the 60-byte step state. `roofline` is the
dominant kernel (pass 2, 28 algorithmic bytes per parameter) against the measured HBM copy
bandwidth. `cpu_baseline` / `--impl reference` time the reference's PyTorch CPU path
(torch AdamW + GradScaler + clip_grad_norm_) on the host cores, on a bounded sample of the
same workload.
"""
from __future__ import annotations

import argparse
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
# DRAM traffic of pass 2 per element, from one ncu capture of a launch on the gpt2-small arena
# (1.742693 GB read + 1.686448 GB written over 124,476,416 elements; profiles/
# pass2_f16_kernel_gpt2-small_ncu_full.md). Every element is touched once, so traffic scales with
# the element count; the 1.3 B arena is too large to capture under ncu's replay.
PASS2_DRAM_BYTES_PER_PARAM_NCU = 27.55
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
NVLINK_MEASURED_GBS = 770.0     # per direction per GPU, measured peer copy on this pool


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


def cpu_sample_shapes(name: str):
    """A bounded sample of the workload for the CPU path: the first tensors of the arena after
    the token embedding (wpe, two whole layers) plus the final LayerNorm, with their real shapes."""
    slots = workload_slots(name)
    per_layer = 12
    keep = slots[1:2 + 2 * per_layer] + slots[-2:]
    return [s.shape for s in keep], "wpe + layers 0-1 + ln_f of the %s arena" % name


def run_cpu_reference(workload: str, steps: int, warmup: int) -> dict:
    """The reference's PyTorch CPU path (reference/train.py:147-153 order) on the host cores."""
    import torch
    from oracle.torch_ref import time_cpu_step
    # every host core the process may use: torchrun exports OMP_NUM_THREADS=1, which would
    # otherwise pin the CPU path to one thread
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))
    shapes, what = cpu_sample_shapes(workload)
    r = time_cpu_step(shapes, steps=max(1, steps), warmup=max(1, warmup), loss_scale=32768.0)
    gps = r["params"] / r["seconds_per_step"] / 1e9
    return {"value": gps, "unit": UNIT, "cores": r["threads"], "kind": "port",
            "sample": f"{what}: {r['params']:,} params/step, median of {max(1, steps)} steps; "
                      "torch.optim.AdamW(foreach=False) + GradScaler('cpu') + clip_grad_norm_, "
                      f"host has {os.cpu_count()} logical cores",
            "ms_per_step": r["seconds_per_step"] * 1e3, "params": r["params"]}


# ---------------------------------------------------------------------------- GPU arm

def fill_normal_(t, std, seed, chunk=1 << 27):
    """t ~ N(0, std) from a seeded device generator, in chunks (no arena-sized temporary)."""
    import torch
    gen = torch.Generator(device=t.device).manual_seed(seed)
    for at in range(0, t.numel(), chunk):
        sl = t[at:at + chunk]
        sl.copy_(torch.randn(sl.numel(), generator=gen, device=t.device, dtype=torch.float32) * std)


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

    if world == 1:
        opt = amp.AmpOptimizer(slots, cfg, eps=1e-8, loss_scale=loss_scale, device=dev)
        fill_normal_(opt.master[:n_params], 0.02, seed=0)
        amp.cast_to_x(opt.weights16, opt.master, n)
        step_fn = opt.optimizer_step
    else:
        fused = args.collectives == "fused"
        fused_note = None
        if fused:
            # symmetric memory needs peer access between all ranks' GPUs; where the box cannot give
            # it, every rank falls back together to NCCL around the passes (and the line says so)
            try:
                opt = amp.FusedZero1Optimizer(slots, cfg, eps=1e-8, loss_scale=loss_scale, device=dev)
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

    # m and v pre-warmed by 5 seeded steps of the implementation itself (untimed)
    for k in range(5):
        fill_grads(1000 * (k + 1) + rank + 1)
        step_fn()
    fill_grads(rank + 1)
    torch.cuda.synchronize()
    st = opt.read_state()
    if st.skipped != 0 or st.adam_t != 5:
        raise SystemExit(f"pre-warm went wrong: {st.as_dict()}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

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
            amp.pass2_f16(opt.master, opt.m, opt.v, opt.grads16, opt.weights16, opt.n, 0, opt.tensors,
                          opt.ntensors, opt.state, opt.beta1, opt.beta2, opt.eps)
            ev[k][2].record()
    elif fused:
        for k in range(args.steps):
            ev[k][0].record()
            opt._barrier("grads16")
            opt.fused_pass1()
            ev[k][1].record()
            opt._barrier("pairs")
            opt.finalize_pairs()
            ev[k][2].record()
            opt.fused_pass2()
            ev[k][3].record()
            opt._barrier("weights16")
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
    if world == 1:
        pass1_ms, pass2_ms = avg(0, 1), avg(1, 2)
        n_local = n
    elif fused:
        # each fused kernel is timed with the barrier in front of it: a rank that arrives early waits there
        phases = {"barrier_rs_pass1_ms": max_over_ranks(avg(0, 1)), "barrier_finalize_ms": max_over_ranks(avg(1, 2)),
                  "pass2_ag_ms": max_over_ranks(avg(2, 3)), "barrier_end_ms": max_over_ranks(avg(3, 4))}
        pass1_ms, pass2_ms = phases["barrier_rs_pass1_ms"], phases["pass2_ag_ms"]
        n_local = opt.n_local
        coll_bytes = (world - 1) / world * 2 * n            # per GPU per direction, each fused kernel
        phases["rs_pass1_nvlink_gbs"] = coll_bytes / (phases["barrier_rs_pass1_ms"] * 1e-3) / 1e9
        phases["pass2_ag_nvlink_gbs"] = coll_bytes / (phases["pass2_ag_ms"] * 1e-3) / 1e9
        phases["nvlink_peak_gbs"] = NVLINK_MEASURED_GBS
        phases["collectives"] = "fused into the passes: plain peer loads (rs_pass1) and peer stores (pass2_ag)"
    else:
        phases = {"reduce_scatter_ms": max_over_ranks(avg(0, 1)), "pass1_ms": max_over_ranks(avg(1, 2)),
                  "norm_gather_finalize_ms": max_over_ranks(avg(2, 3)), "pass2_ms": max_over_ranks(avg(3, 4)),
                  "all_gather_ms": max_over_ranks(avg(4, 5))}
        pass1_ms, pass2_ms = phases["pass1_ms"], phases["pass2_ms"]
        n_local = opt.n_local
        coll_bytes = (world - 1) / world * 2 * n            # per GPU per direction, each collective
        phases["reduce_scatter_gbs"] = coll_bytes / (phases["reduce_scatter_ms"] * 1e-3) / 1e9
        phases["all_gather_gbs"] = coll_bytes / (phases["all_gather_ms"] * 1e-3) / 1e9
        phases["nvlink_peak_gbs"] = NVLINK_MEASURED_GBS
        phases["collectives"] = "NCCL reduce_scatter_tensor(AVG) / all_gather_into_tensor around the passes"
        if args.collectives == "fused":
            phases["collectives"] += " (fused path unavailable on this box: %s)" % (fused_note or "a peer rank failed")
    st = opt.read_state()
    if st.skipped != 0:
        raise SystemExit("a timed step was skipped: the timing would count 2 B/param steps")

    # ------------------------------------------------------------------ end to end: host gradients in, state out
    e2e_steps = max(3, min(args.steps, 10))
    host_grads = torch.empty(n, dtype=torch.float16, pin_memory=True)
    host_grads.copy_(opt.grads16)
    host_state = torch.empty(opt.state.numel(), dtype=torch.uint8, pin_memory=True)
    torch.cuda.synchronize()

    def e2e_step():
        opt.grads16.copy_(host_grads, non_blocking=True)
        step_fn()
        host_state.copy_(opt.state, non_blocking=True)
        torch.cuda.current_stream().synchronize()       # the caller reads the state: a real host sync

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

    graph_replay = None
    if world == 1:
        # The same step as ONE CUDA-graph launch (how the reference's trainer replays it,
        # cuda/train_fast.cu:720-730): per-replay times by events, median reported.
        side = torch.cuda.Stream(device=dev)
        graph = amp.CudaGraph()
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            graph.capture(side, lambda: opt.optimizer_step(side))
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

    if world > 1:
        dist.barrier()

    peak, peak_kind = measured_hbm_peak()
    pass2_gbs = BYTES_PASS2 * n_local / (pass2_ms * 1e-3) / 1e9
    pass1_gbs = BYTES_PASS1 * n_local / (pass1_ms * 1e-3) / 1e9
    value = n_params / (ms_per_step * 1e-3) / 1e9
    hbm_gbs_step = BYTES_STEP * n_local / ((pass1_ms + pass2_ms) * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {n_params:,} params, {len(slots)} tensors, fp16 grads "
                               f"N(0,1e-3)*{int(loss_scale)}, fp32 master/m/v, m and v pre-warmed by 5 steps, "
                               "AdamW lr 6e-4 betas (0.9,0.95) eps 1e-8 wd 0.1, clip 1.0",
                   "params": n_params, "arena": n, "parallelism": "single" if world == 1 else f"zero1-dp{world}",
                   "l2": "arenas are far larger than the 126 MB L2 (no flush needed between steps)"},
        "hbm_gbs": hbm_gbs_step, "hbm_frac_of_nominal_8tbs": hbm_gbs_step / NOMINAL_HBM_GBS,
        "hbm_frac_of_measured": hbm_gbs_step / peak,
        "kernels_ms": {"pass1_finalize": pass1_ms, "pass2": pass2_ms},
        "roofline": {"bound": "hbm", "kernel": "pass2_f16_kernel", "achieved": pass2_gbs, "peak": peak,
                     "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s", "frac": pass2_gbs / peak,
                     "traffic": None, "algorithmic_bytes_per_launch": BYTES_PASS2 * n_local,
                     "pass1_achieved": pass1_gbs, "pass1_frac": pass1_gbs / peak},
        "e2e": {"value": n_params / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 2 * n, "d2h_bytes_per_step": int(opt.state.numel()), "steps": e2e_steps},
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
    line["roofline"]["traffic"] = PASS2_DRAM_BYTES_PER_PARAM_NCU * n_local
    line["roofline"]["traffic_source"] = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on the "
                                          "gpt2-small arena (profiles/), scaled by the element count")
    if world > 1 and fused:
        # A fused compute + collective kernel: its floor is the slower of the HBM time of its slice and
        # the time its bytes need on NVLink (measured peer bandwidth per direction per GPU).
        link_bytes = (world - 1) / world * 2 * n
        t_hbm = BYTES_PASS2 * n_local / (peak * 1e9)
        t_link = link_bytes / (NVLINK_MEASURED_GBS * 1e9)
        by_link = t_link > t_hbm
        achieved = (link_bytes if by_link else BYTES_PASS2 * n_local) / (pass2_ms * 1e-3) / 1e9
        bound_peak = NVLINK_MEASURED_GBS if by_link else peak
        line["roofline"].update({
            "bound": "nvlink" if by_link else "hbm", "kernel": "pass2_ag_f16_kernel", "achieved": achieved,
            "peak": bound_peak, "frac": achieved / bound_peak,
            "peak_kind": ("measured peer-copy bandwidth per direction" if by_link
                          else f"{peak_kind} copy bandwidth"),
            "floor_ms": {"hbm": t_hbm * 1e3, "nvlink": t_link * 1e3}, "traffic": None,
            "traffic_source": None, "nvlink_bytes_per_launch": link_bytes})
        line["kernels_ms"] = {"barrier+rs_pass1": pass1_ms, "pass2_ag": pass2_ms}
    if world > 1:
        dist.destroy_process_group()
    return line if rank == 0 else None


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="1.3b", choices=["debug", "readme", "gpt2-small", "1.3b"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--collectives", choices=["fused", "nccl"], default="fused",
                    help="N > 1: fold reduce-scatter / all-gather into the passes (peer loads and stores), "
                         "or call NCCL around them")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))

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
                "config": {"workload": f"{args.workload}: {n_params:,} params (timed on a bounded sample, see "
                                       "cpu_baseline.sample)", "params": n_params},
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return

    line = run_gpu(args)
    if line is None:
        return
    if args.gpus == 1 and not args.no_cpu_baseline:
        r = run_cpu_reference(args.workload, steps=5, warmup=1)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
