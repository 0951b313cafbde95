#!/usr/bin/env python
"""Benchmark of the fused decoder losses: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
                    [--workload c3_k128] [--kind hier|topk] [--dweight-mode atomic|deterministic]

A step is one forward + backward of the loss over one batch of seeded synthetic inputs
(flexsae_b200.workloads).  At N = 1 the workload is the headline set-up
F=65536, D=2304, K=128, B=4096, bf16 decoder / fp32 vals, Hierarchical loss; at N > 1 every
rank keeps B=4096 rows (weak scaling), the decoder is replicated, dweight is summed over the ranks
inside the backward kernel and the scalar loss and dbias are all-reduced each step.  `--workload
c5` (global batch 65536) splits its rows over the ranks instead (strong scaling).  Under torchrun
one process drives one GPU.

`value` is batch rows per second over all ranks with inputs resident in HBM; `e2e` is the same
through the public autograd API with the step's indices / vals / target copied from pinned host
memory and the loss read back every step.  `--impl reference` times the torch restatement of the
reference losses on the host CPU cores instead (the reference's own CPU-runnable path).

With more than one rank the run first checks the fused cross-GPU gradient sum against a plain NCCL
all-reduce of the per-rank gradients on the same inputs and refuses to print a number on a mismatch
(`"parity_checked": true` in the line).  Environment switches (all optional): FLEXSAE_OPTIONS
(`name=value,...` for flexsae_set_option), FLEXSAE_PEER_REDUCE, FLEXSAE_MULTICAST,
FLEXSAE_SYMMETRIC_DWEIGHT, FLEXSAE_FUSED_SMALL_REDUCE (0/1: flexsae_b200.distributed.config).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from flexsae_b200.workloads import CONFIGS, algorithmic_bytes, make_inputs  # noqa: E402

FALLBACK_HBM_GBS = 6650.0   # earlier measurement on this pool, used only without MEASURED_PEAKS.json
# dram__bytes_read + dram__bytes_write per launch of the dominant kernel at the headline workload,
# from the ncu launch list summarised under profiles/
NCU_TRAFFIC_BYTES_PER_LAUNCH = {("c3_k128", "hier", "atomic"): 1239.0e6}


# Exchange settings `bench.py` uses when it runs on several GPUs (each can be overridden through the
# environment, see the module docstring); they are reported in the line's "exchange" object.
SHARDED_DEFAULTS = {"symmetric_dweight": True, "fused_small_reduce": True, "options": {}}


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clocks and throttle reasons of the run's GPUs while the timed region runs (read-only).

    The samples come from one `nvidia-smi -lms` child process of rank 0, started before the warm-up
    steps; the timed region only notes its wall-clock start and end, and the samples whose time stamps
    fall between them are the ones reported.  (Sampling through NVML from a thread of the benchmark
    process itself -- one per rank, or rank 0 for all GPUs -- stalled the launch loops: every query
    cost about 0.2 ms of step time, and at 8 GPUs the forward, which ends in a cross-rank sum,
    measured 0.85 instead of 0.33 ms.)"""

    REASONS = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
               0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
               0x100: "display_clock_setting"}

    def __init__(self, indices, period_ms: int = 20):
        self.proc, self.path, self.t0, self.t1 = None, None, None, None
        self.n_gpus = len(list(indices))
        if not self.n_gpus:
            return
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        ids = []
        for index in indices:
            ids.append(visible.split(",")[index] if visible and len(visible.split(",")) > index else str(index))
        import subprocess
        import tempfile
        try:
            fd, self.path = tempfile.mkstemp(prefix="flexsae_clocks_", suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", ",".join(ids),
                 "--query-gpu=timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.active",
                 "--format=csv,noheader,nounits", "-lms", str(period_ms)], stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
            import atexit
            atexit.register(self.proc.kill)          # never outlives the benchmark, whatever way it ends
        except Exception:
            self.proc = None

    def __enter__(self):
        self.t0 = time.time()
        return self

    def __exit__(self, *exc):
        self.t1 = time.time()
        if self.proc is not None:            # the legs that follow run without it
            self.proc.terminate()

    def summary(self):
        """Reports the samples taken inside the timed region."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            with open(self.path) as f:
                text = f.read()
            os.remove(self.path)
        except Exception:
            text = ""
        out = self.parse(text, self.t0, self.t1)
        out["gpus_sampled"] = self.n_gpus
        return out

    @classmethod
    def parse(cls, text: str, t0: float, t1: float):
        """`nvidia-smi --query-gpu=timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.active
        --format=csv,noheader,nounits` lines -> the summary of those stamped between t0 and t1 (Unix
        seconds; nvidia-smi stamps a sample when it starts reading it, so samples up to 20 ms outside
        count when none lies inside, and are reported separately)."""
        import datetime
        inside, around, reasons, max_mhz = [], [], set(), None
        for line in text.splitlines():
            row = [c.strip() for c in line.split(",")]
            try:
                stamp = datetime.datetime.strptime(row[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                mhz, max_mhz, bits = int(row[1]), int(row[2]), int(row[3], 16)
            except (ValueError, IndexError):
                continue
            if t0 - 0.02 <= stamp <= t1 + 0.02:
                (inside if t0 <= stamp <= t1 else around).append(mhz)
                reasons.update(name for b, name in cls.REASONS.items() if bits & b)
        used = inside or around
        if not used:
            return {"sm_mhz": None, "sm_max_mhz": max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(used), "sm_min_mhz": min(used), "sm_max_mhz": max_mhz, "reasons": sorted(reasons),
                "samples": len(inside), "samples_within_20ms": len(around),
                "source": "nvidia-smi -lms child process of rank 0"}


def cpu_reference_rate(w, kind, budget_s: float, chunk_rows: int = 256, repeats: int = 1):
    """rows/s of the torch restatement of the reference loss (fwd + backward) on the host cores,
    on a bounded sample of the workload's rows (whole chunks until `budget_s` is spent)."""
    from oracle import torch_reference as tref
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    first = make_inputs(w, "cpu", rows=min(w.B, chunk_rows))
    full_weight = first["weight"]
    t0 = time.perf_counter()
    tref.chunked_loss_and_grads(kind, first["indices"], full_weight, first["vals"], first["bias"], first["target"],
                                chunk_rows=chunk_rows)           # warm-up chunk, also the calibration
    per_chunk = time.perf_counter() - t0
    n_chunks = max(1, min((w.B + chunk_rows - 1) // chunk_rows, int(budget_s / max(per_chunk, 1e-3))))
    rows = min(w.B, n_chunks * chunk_rows)
    x = make_inputs(w, "cpu", rows=rows, with_weight=False)
    best = None
    for _ in range(repeats):
        r = tref.chunked_loss_and_grads(kind, x["indices"], full_weight, x["vals"], x["bias"], x["target"],
                                        chunk_rows=chunk_rows)
        best = r["seconds"] if best is None else min(best, r["seconds"])
    return {"value": rows / best, "unit": "rows/s", "cores": cores, "kind": "port",
            "sample": f"first {rows} of {w.B} rows in {chunk_rows}-row chunks, {best:.2f} s; "
                      f"torch {torch.__version__} eager ops of the reference loss, {cores} threads",
            "ms_per_step_extrapolated": best / rows * w.B * 1e3}


def workload_config(w, kind, rows, global_rows, world, dweight_mode, **extra):
    """The `config` object of a bench line: the same keys for the native and the reference arm."""
    cfg = {"workload": w.name, "kind": kind, "B_per_gpu": rows, "global_B": global_rows, "K": w.K, "F": w.F, "D": w.D,
           "storage": f"{w.weight_dtype} weight/bias/target, {w.vals_dtype} vals", "accumulate": "fp32",
           "dweight_mode": dweight_mode,
           "piece_width": "by index skew (hottest decoder row's share of the batch, measured on the device every "
                          "16th backward; uniform synthetic indices keep the L2-sized pieces)" if world == 1 else
                          "fixed (the ranks of a sharded run must agree)",
           "parallelism": f"batch-sharded x{world}, decoder replicated" if world > 1 else "single GPU",
           "l2": "no flush: the decoder alone (302 MB at the headline shape) exceeds the 126 MB L2; the library's "
                 "own fp32 gradient slabs are meant to stay L2-resident between launches"}
    cfg.update(extra)
    return cfg


def run_reference(args, w, kind):
    """The reference arm: the reference's CPU path (torch eager restatement) on the host cores.

    A step is the whole per-GPU batch when `(steps + warmup)` such steps fit the time budget
    (`--reference-seconds`, 300 by default); otherwise every step is the first `sampled_rows` rows of
    the batch and `ms_per_step` is scaled up to the whole batch, and the line says so."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    chunk = 256
    from oracle import torch_reference as tref
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    probe = make_inputs(w, "cpu", rows=chunk)
    weight = probe["weight"]
    tref.chunked_loss_and_grads(kind, probe["indices"], weight, probe["vals"], probe["bias"], probe["target"], chunk_rows=chunk)
    t0 = time.perf_counter()
    tref.chunked_loss_and_grads(kind, probe["indices"], weight, probe["vals"], probe["bias"], probe["target"], chunk_rows=chunk)
    per_chunk = time.perf_counter() - t0
    n_steps = max(1, args.steps + args.warmup)
    chunks_whole = (w.B + chunk - 1) // chunk
    if per_chunk * chunks_whole * n_steps <= args.reference_seconds:
        rows = w.B
    else:
        rows = min(w.B, chunk * max(1, int(args.reference_seconds / n_steps / per_chunk)))
    x = make_inputs(w, "cpu", rows=rows, with_weight=False)
    times = []
    for i in range(args.warmup + args.steps):
        r = tref.chunked_loss_and_grads(kind, x["indices"], weight, x["vals"], x["bias"], x["target"], chunk_rows=chunk)
        if i >= args.warmup:
            times.append(r["seconds"])
    sec = sum(times) / len(times)
    value = rows / sec
    whole = rows == w.B
    sample = (f"each step = all {w.B} rows" if whole else f"each step = first {rows} of {w.B} rows") + \
             f" in {chunk}-row chunks, {cores} threads, torch {torch.__version__} eager ops of the reference loss"
    line = {
        "impl": "reference", "metric": "hier_topk_fwd_bwd_throughput" if kind == "hier" else "topk_fwd_bwd_throughput",
        "value": value, "unit": "rows/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": w.B / value * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, kind, w.B, w.B * max(1, args.gpus), max(1, args.gpus), args.dweight_mode),
        "sampled_rows": None if whole else rows,
        "note": None if whole else "ms_per_step is scaled from the sampled rows to the whole batch",
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="c3_k128", choices=sorted(CONFIGS))
    ap.add_argument("--kind", default="hier", choices=["hier", "topk"])
    ap.add_argument("--dweight-mode", default="atomic", choices=["atomic", "deterministic"])
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="CPU-baseline sample budget (0 = skip)")
    ap.add_argument("--reference-seconds", type=float, default=300.0,
                    help="--impl reference: time budget of the whole run; whole batches per step if they fit")
    ap.add_argument("--topk-steps", type=int, default=-1,
                    help="steps of the extra TopK leg that gives hier_topk_ratio (0 = skip; default: min(steps, 50))")
    ap.add_argument("--e2e-steps", type=int, default=0, help="0 = same as --steps")
    ap.add_argument("--e2e-lag", type=int, default=2, help="end-to-end loop: the host reads the loss of step i - lag at step i")
    ap.add_argument("--scaling", default="auto", choices=["auto", "weak", "strong"],
                    help="weak: every rank keeps the workload's B rows; strong: the workload's B rows are split over "
                         "the ranks; auto: strong for c5 (its B is the global batch), weak otherwise")
    args = ap.parse_args()
    w = CONFIGS[args.workload]
    kind = args.kind

    if args.impl == "reference":
        run_reference(args, w, kind)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl native needs a CUDA device (there is no CPU implementation of the fused losses)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    # one child process of rank 0 samples the clocks of every GPU of the run (local ranks 0..world-1
    # of this one node); started here so that its own start-up is long over when the timed region begins
    clocks = ClockSampler(range(world) if rank == 0 else [], 10 if world == 1 else 20)
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    import flexsae_b200 as fx
    from flexsae_b200 import _native as nv
    from flexsae_b200 import distributed as fd
    from flexsae_b200 import losses

    def env_flag(name, default):
        return os.environ.get(name, "1" if default else "0") != "0"

    fx.config.dweight_mode = args.dweight_mode
    fd.config.use_multicast = env_flag("FLEXSAE_MULTICAST", False)
    fd.config.peer_reduce = env_flag("FLEXSAE_PEER_REDUCE", True)
    # the measured-best exchange settings of a batch-sharded run (see SHARDED_DEFAULTS) unless overridden
    fd.config.symmetric_dweight = env_flag("FLEXSAE_SYMMETRIC_DWEIGHT", distributed and SHARDED_DEFAULTS["symmetric_dweight"])
    fd.config.fused_small_reduce = env_flag("FLEXSAE_FUSED_SMALL_REDUCE", distributed and SHARDED_DEFAULTS["fused_small_reduce"])
    options = dict(SHARDED_DEFAULTS["options"]) if distributed else {}
    for item in filter(None, os.environ.get("FLEXSAE_OPTIONS", "").split(",")):   # e.g. "lanes_bwd=8,segments=2"
        name, value = item.split("=")
        options[name] = int(value)
    for name, value in options.items():
        nv.set_option(name, value)
    scaling = args.scaling if args.scaling != "auto" else ("strong" if w.name == "c5" else "weak")
    if scaling == "strong":
        if w.B % world:
            raise SystemExit(f"--scaling strong: B={w.B} does not split evenly over {world} ranks")
        rows = w.B // world                        # the workload's batch is the global one
    else:
        rows = w.B                                 # per rank
    global_rows = rows * world
    wg = w.replace(B=global_rows)
    w = w.replace(B=rows)                          # what one GPU processes per step
    x = make_inputs(wg, dev, row0=rank * rows, rows=rows)
    weight = x["weight"].requires_grad_(True)
    bias = x["bias"].requires_grad_(True)
    vals = x["vals"].requires_grad_(True)
    indices, target = x["indices"], x["target"]

    def loss_function(which):
        if distributed:
            sharded = fd.sharded_hierarchical_sae_loss if which == "hier" else fd.sharded_topk_sae_loss
            return lambda i, wt, v, b, t: sharded(i, wt, v, b, t, global_rows=global_rows)
        return fx.triton_hierarchical_sae_loss if which == "hier" else fx.triton_topk_sae_loss

    loss_fn = loss_function(kind)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def step(fn=None, marks=None):
        weight.grad = vals.grad = bias.grad = None
        if marks is not None:
            e0, e1, e2 = ev(), ev(), ev()
            e0.record()
        loss = (fn or loss_fn)(indices, weight, vals, bias, target)
        if marks is not None:
            e1.record()
        loss.backward()
        if marks is not None:
            e2.record()
            marks.append((e0, e1, e2))
        return loss

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def kernels_ok() -> bool:
        """False (on every rank) if a bounded wait inside a kernel gave up on any rank."""
        try:
            losses.check_status(dev)
            ok = 1
        except RuntimeError:
            ok = 0
        if distributed:
            t = torch.tensor([ok], device=dev, dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            ok = int(t.item())
        return bool(ok)

    def timed(fn, n):
        """n steps between two events; returns (ms per step, per-step (fwd, bwd, whole) ms lists), max over ranks."""
        marks = []
        start, stop = ev(), ev()
        start.record()
        for _ in range(n):
            step(fn, marks)
        stop.record()
        barrier()
        total = start.elapsed_time(stop)
        fwd = [a.elapsed_time(b) for a, b, _ in marks]
        bwd = [b.elapsed_time(c) for _, b, c in marks]
        whole = [a.elapsed_time(c) for a, _, c in marks]
        stats = [total / n, sum(fwd) / n, sum(bwd) / n, statistics.median(whole), min(whole)]
        if distributed:
            t = torch.tensor(stats, device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            stats = [float(v) for v in t]
        return stats

    # ---- several ranks: the fused cross-GPU gradient sum against the plain collective, same inputs ----
    # The exchange settings are tried from the fastest to the plainest -- in-place dweight and the
    # library's own small sums, then the gather buffer, then NCCL for everything -- and the first one
    # whose gradients agree with "per-rank kernels + NCCL all-reduce" is the one that is timed; what was
    # dropped, and why, is reported in the line ("exchange": {"rejected": [...]}).
    parity = None
    rejected = []
    fused_exchange = distributed and fd.config.peer_reduce and args.dweight_mode == "atomic"
    if fused_exchange:
        def one_step_grads():
            """(loss, dweight, dbias, dvals) of one step, or None on every rank if any rank failed."""
            out, failed = None, 0
            try:
                loss = step()
                torch.cuda.synchronize(dev)
                out = (float(loss), weight.grad.float().clone(), bias.grad.float().clone(), vals.grad.float().clone())
            except RuntimeError as e:                       # a timed-out wait reported by the sharded loss
                sys.stderr.write(f"bench.py: rank {rank}: {e}\n")
                failed = 1
            weight.grad = vals.grad = bias.grad = None
            t = torch.tensor([failed], device=dev, dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return None if int(t.item()) else out

        ladder = [(fd.config.symmetric_dweight, fd.config.fused_small_reduce)]
        if fd.config.symmetric_dweight:
            ladder.append((False, fd.config.fused_small_reduce))
        if fd.config.fused_small_reduce:
            ladder.append((False, False))
        fd.config.peer_reduce, fd.config.symmetric_dweight, fd.config.fused_small_reduce = False, False, False
        ref = one_step_grads()                                      # per-rank kernels + NCCL all-reduce
        if ref is None or not kernels_ok():
            raise SystemExit("bench.py: the per-rank kernels + NCCL all-reduce step failed; no number is reported")
        ref_loss, ref_dw, ref_db, ref_dv = ref
        scale = float(ref_dw.abs().max())
        chosen = None
        for sym, small in ladder:
            fd.config.peer_reduce, fd.config.symmetric_dweight, fd.config.fused_small_reduce = True, sym, small
            got = one_step_grads()                                  # the path that would be timed below
            if got is not None:
                got_loss, got_dw, got_db, got_dv = got
                errs = torch.tensor([abs(got_loss - ref_loss) / abs(ref_loss), float((got_dw - ref_dw).abs().max()) / scale,
                                     float((got_db - ref_db).abs().max()) / float(ref_db.abs().max()),
                                     float((got_dv - ref_dv).abs().max()) / float(ref_dv.abs().max())],
                                    device=dev, dtype=torch.float64)
                dist.all_reduce(errs, op=dist.ReduceOp.MAX)
                parity = {"against": "per-rank kernels + NCCL all-reduce of dweight, dbias and loss, same inputs",
                          "loss_rel": float(errs[0]), "dweight_rel_of_max": float(errs[1]),
                          "dbias_rel_of_max": float(errs[2]),
                          "dvals_rel_of_max": float(errs[3])}    # per-piece dot products: the two paths cut D into different pieces
                del got, got_dw
                ok = kernels_ok() and parity["loss_rel"] < 1e-5 and parity["dweight_rel_of_max"] < 1e-2 and \
                    parity["dbias_rel_of_max"] < 1e-2 and \
                    parity["dvals_rel_of_max"] < (1e-4 if w.vals_dtype == "float32" else 1e-2)
                why = parity
            else:
                ok, why = False, "a bounded wait inside the exchange gave up"
                kernels_ok()                                        # clears the status word on every rank
            if ok:
                chosen = (sym, small)
                break
            rejected.append({"symmetric_dweight": sym, "fused_small_reduce": small, "why": why})
            parity = None
            barrier()
        del ref, ref_dw
        if chosen is None:                                          # nothing fused agrees: time the plain collective, and say so
            fused_exchange = False
            fd.config.peer_reduce, fd.config.symmetric_dweight, fd.config.fused_small_reduce = False, False, False

    dweight_sum = "in the backward kernel over peer memory" if fused_exchange else \
                  ("NCCL all-reduce after the backward" if distributed else "none (one GPU)")
    for _ in range(args.warmup):
        step()
    barrier()
    if not kernels_ok():
        raise SystemExit("bench.py: a kernel reported a timed-out wait during warm-up; no number is reported")
    losses.launch_count = 0
    with clocks:
        ms_per_step, fwd_ms, bwd_ms, median_ms, min_ms = timed(loss_fn, args.steps)
    launches = losses.launch_count
    if not kernels_ok():
        raise SystemExit("bench.py: a kernel reported a timed-out wait inside the timed region; no number is reported")
    value = global_rows / (ms_per_step * 1e-3)

    # ---- the other loss on the same inputs: the Hierarchical / TopK step-time ratio -----------------
    other = None
    other_steps = min(args.steps, 50) if args.topk_steps < 0 else args.topk_steps
    if other_steps > 0:
        other_kind = "topk" if kind == "hier" else "hier"
        other_fn = loss_function(other_kind)
        for _ in range(max(3, min(args.warmup, 10))):
            step(other_fn)
        barrier()
        o = timed(other_fn, other_steps)
        if kernels_ok():
            other = {"kind": other_kind, "ms_per_step": o[0], "fwd_ms": o[1], "bwd_ms": o[2], "steps": other_steps}

    # ---- end to end: host inputs in, loss out, every step ------------------------------------
    e2e_steps = args.e2e_steps or args.steps
    host = {k: x[k].detach().cpu().pin_memory() for k in ("indices", "vals", "target")}
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    copy_stream = torch.cuda.Stream(dev)
    bufs = [{k: torch.empty_like(x[k].detach()) for k in host} for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    lag = max(1, args.e2e_lag)     # the host reads the loss of step i - lag at step i: it may run that far ahead of the GPU
    loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(lag)]
    loss_there = [torch.cuda.Event() for _ in range(lag)]

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            for k, t in host.items():
                bufs[slot][k].copy_(t, non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_loop(n):
        """Every step: its inputs come from pinned host memory (uploaded while the previous step
        computes) and its loss goes back to the host, where it is read `lag` steps later so that the
        host can already enqueue the next steps (with several ranks a host that is not ahead of its GPU
        makes every rank wait at the cross-GPU sums)."""
        for c in consumed:
            c.record()
        upload(0)
        seen = []
        for i in range(n):
            slot = i & 1
            if i + 1 < n:
                upload(slot ^ 1)                      # next step's inputs travel while this one computes
            torch.cuda.current_stream(dev).wait_event(ready[slot])
            weight.grad = vals.grad = bias.grad = None
            v = bufs[slot]["vals"].detach().requires_grad_(True)
            loss = loss_fn(bufs[slot]["indices"], weight, v, bias, bufs[slot]["target"])
            loss.backward()
            consumed[slot].record()
            ls = i % lag
            if i >= lag:                              # the buffer about to be overwritten: read it first
                loss_there[ls].synchronize()
                seen.append(float(loss_host[ls][0]))
            loss_host[ls].copy_(loss.detach().reshape(1), non_blocking=True)    # device -> host read of the step's result
            loss_there[ls].record()
        for i in range(max(0, n - lag), n):
            loss_there[i % lag].synchronize()
            seen.append(float(loss_host[i % lag][0]))
        return seen

    e2e_loop(min(5, e2e_steps))
    barrier()
    t0 = time.perf_counter()
    seen = e2e_loop(e2e_steps)
    barrier()
    e2e_s = time.perf_counter() - t0
    if not kernels_ok():
        raise SystemExit("bench.py: a kernel reported a timed-out wait in the end-to-end loop; no number is reported")
    if len(seen) != e2e_steps or not all(v == v and v > 0 for v in seen):
        raise SystemExit("bench.py: the end-to-end loop did not read a valid loss for every step")
    if distributed:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t)
    e2e_value = global_rows * e2e_steps / e2e_s

    if rank == 0:
        peak, peak_kind = hbm_peak()
        alg = algorithmic_bytes(w)                        # per GPU per step
        sw = 2 if w.weight_dtype != "float32" else 4
        # the backward's share of the algorithmic bytes: second row gather + fp32 scatter payload,
        # dense table (clear + conversion), saved state, indices / vals / dvals
        alg_bwd = (rows * w.K * w.D * (sw + 4) + w.F * w.D * (4 + (4 + sw if sw != 4 else 0))
                   + rows * w.D * 4 + rows * w.K * (8 + 4 + 4))
        if args.dweight_mode == "deterministic":
            dominant = "decoder_loss_bwd_kernel<DET> + ordered_sum_items_kernel (one pair of launches per column piece)"
        elif distributed and fused_exchange:
            dominant = "decoder_loss_bwd_sharded_kernel (one launch per backward)"
        else:
            dominant = "decoder_loss_bwd_pipelined_kernel (one launch per backward)"
        default_build = not distributed and not os.environ.get("FLEXSAE_OPTIONS")
        line = {
            "metric": "hier_topk_fwd_bwd_throughput" if kind == "hier" else "topk_fwd_bwd_throughput",
            "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "ms_per_step_median": median_ms, "ms_per_step_min": min_ms,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(w, kind, rows, global_rows, world, args.dweight_mode),
            "exchange": {"dweight_sum": dweight_sum,
                         "loss_and_dbias_sum": ("flexsae_small_allreduce (one launch each, peer memory)"
                                                if distributed and fd.config.fused_small_reduce else
                                                ("NCCL all-reduce" if distributed else "none (one GPU)")),
                         "symmetric_dweight": bool(distributed and fd.config.symmetric_dweight),
                         "options": options},
            "hbm_gbs": alg / (ms_per_step * 1e-3) / 1e9,
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "roofline": {"bound": "hbm", "kernel": dominant,
                         "achieved": alg_bwd / (bwd_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg_bwd / (bwd_ms * 1e-3) / 1e9 / peak, "peak_source": peak_kind,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get((w.name, kind, args.dweight_mode)) if default_build else None,
                         "note": "achieved = the backward's algorithmic bytes / its CUDA-event time (bwd_ms, which also "
                                 "covers the two small finalising kernels); gathers and fp32 reductions are served by "
                                 "L2, so DRAM traffic is far below the algorithmic bytes and the binding resource is "
                                 "the L2 reduction rate (5.7 TB/s measured for red.global.add.v4.f32), not HBM"},
            "roofline_step": {"bound": "hbm", "achieved": alg / (ms_per_step * 1e-3) / 1e9, "peak": peak,
                              "unit": "GB/s", "frac": alg / (ms_per_step * 1e-3) / 1e9 / peak,
                              "algorithmic_bytes": alg},
            "e2e": {"value": e2e_value, "unit": "rows/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_s / e2e_steps * 1e3, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks.summary(),
        }
        if other is not None:
            hier_ms, topk_ms = (ms_per_step, other["ms_per_step"]) if kind == "hier" else (other["ms_per_step"], ms_per_step)
            line["hier_ms"], line["topk_ms"] = hier_ms, topk_ms
            line["hier_topk_ratio"] = hier_ms / topk_ms
            line["other_loss"] = other
        if parity is not None:
            line["parity_checked"] = True
            line["parity"] = parity
        if rejected:
            line["exchange"]["rejected"] = rejected      # faster settings whose gradients did not agree, fastest first
        if world == 1 and args.cpu_seconds > 0:
            line["cpu_baseline"] = cpu_reference_rate(w, kind, args.cpu_seconds)
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
