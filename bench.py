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
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from flexsae_b200.workloads import CONFIGS, algorithmic_bytes, make_inputs  # noqa: E402

FALLBACK_HBM_GBS = 6650.0   # earlier measurement on this pool, used only without MEASURED_PEAKS.json
# dram__bytes_read + dram__bytes_write per launch of the dominant kernel at the headline workload,
# from the ncu launch list summarised under profiles/
NCU_TRAFFIC_BYTES_PER_LAUNCH = {("c3_k128", "hier", "atomic"): 3416.0e6}


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    REASONS = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
               0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
               0x100: "display_clock_setting"}

    def __init__(self, index: int, period_s: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nvml.nvmlDeviceGetClockInfo(self.h, self.nvml.NVML_CLOCK_SM))
                bits = self.nvml.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for b, name in self.REASONS.items():
                    if bits & b:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


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


def run_reference(args, w, kind):
    """The reference arm: the reference's CPU path (torch eager restatement) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step_budget = 20.0 / max(1, args.steps + args.warmup)
    chunk = 256
    from oracle import torch_reference as tref
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    probe = make_inputs(w, "cpu", rows=chunk)
    weight = probe["weight"]
    t0 = time.perf_counter()
    tref.chunked_loss_and_grads(kind, probe["indices"], weight, probe["vals"], probe["bias"], probe["target"], chunk_rows=chunk)
    per_chunk = time.perf_counter() - t0
    rows = chunk * max(1, int(per_step_budget / per_chunk))
    rows = min(rows, w.B)
    x = make_inputs(w, "cpu", rows=rows, with_weight=False)
    times = []
    for i in range(args.warmup + args.steps):
        r = tref.chunked_loss_and_grads(kind, x["indices"], weight, x["vals"], x["bias"], x["target"], chunk_rows=chunk)
        if i >= args.warmup:
            times.append(r["seconds"])
    sec = sum(times) / len(times)
    value = rows / sec
    sample = f"each step = first {rows} of {w.B} rows per GPU-equivalent, {chunk}-row chunks, {cores} threads"
    line = {
        "impl": "reference", "metric": "hier_topk_fwd_bwd_throughput" if kind == "hier" else "topk_fwd_bwd_throughput",
        "value": value, "unit": "rows/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": w.B / value * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "kind": kind, "B_per_gpu": w.B, "K": w.K, "F": w.F, "D": w.D,
                   "storage": w.weight_dtype, "note": "ms_per_step extrapolated from the sampled rows to B rows"},
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
    ap.add_argument("--e2e-steps", type=int, default=0, help="0 = same as --steps")
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
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    import flexsae_b200 as fx
    from flexsae_b200 import _native as nv
    from flexsae_b200 import distributed as fd
    from flexsae_b200 import losses

    fx.config.dweight_mode = args.dweight_mode
    fd.config.use_multicast = os.environ.get("FLEXSAE_MULTICAST", "0") != "0"
    fd.config.peer_reduce = os.environ.get("FLEXSAE_PEER_REDUCE", "1") != "0"
    fd.config.symmetric_dweight = os.environ.get("FLEXSAE_SYMMETRIC_DWEIGHT", "0") != "0"
    for item in filter(None, os.environ.get("FLEXSAE_OPTIONS", "").split(",")):   # e.g. "lanes_bwd=8,segments=2"
        name, value = item.split("=")
        nv.set_option(name, int(value))
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

    if distributed:
        sharded = fd.sharded_hierarchical_sae_loss if kind == "hier" else fd.sharded_topk_sae_loss

        def loss_fn(i, wt, v, b, t):
            return sharded(i, wt, v, b, t, global_rows=global_rows)
    else:
        loss_fn = fx.triton_hierarchical_sae_loss if kind == "hier" else fx.triton_topk_sae_loss

    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    marks = []

    def step(record=False):
        weight.grad = vals.grad = bias.grad = None
        if record:
            e0, e1, e2 = ev(), ev(), ev()
            e0.record()
        loss = loss_fn(indices, weight, vals, bias, target)
        if record:
            e1.record()
        loss.backward()
        if record:
            e2.record()
            marks.append((e0, e1, e2))
        return loss

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def kernels_ok() -> bool:
        """False (on every rank) if a bounded wait inside a backward kernel gave up on any rank."""
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

    dweight_sum = "in the backward kernel over peer memory" if distributed and fd.config.peer_reduce else \
                  ("NCCL all-reduce after the backward" if distributed else "none (one GPU)")
    for _ in range(args.warmup):
        step()
    barrier()
    if not kernels_ok():
        if not (distributed and fd.config.peer_reduce):
            raise SystemExit("bench.py: a backward kernel reported a timed-out wait during warm-up; no number is reported")
        # the peer-memory exchange did not complete on this machine: measure with the plain collective
        fd.config.peer_reduce = False
        dweight_sum = "NCCL all-reduce after the backward (the peer-memory exchange timed out during warm-up)"
        for _ in range(args.warmup):
            step()
        barrier()
        if not kernels_ok():
            raise SystemExit("bench.py: a backward kernel reported a timed-out wait during warm-up; no number is reported")
    losses.launch_count = 0
    with ClockSampler(local_rank) as clocks:
        start, stop = ev(), ev()
        start.record()
        for _ in range(args.steps):
            step(record=True)
        stop.record()
        barrier()
    launches = losses.launch_count
    if not kernels_ok():
        raise SystemExit("bench.py: a backward kernel reported a timed-out wait inside the timed region; no number is reported")
    elapsed_ms = start.elapsed_time(stop)
    fwd_ms = sum(a.elapsed_time(b) for a, b, _ in marks) / len(marks)
    bwd_ms = sum(b.elapsed_time(c) for _, b, c in marks) / len(marks)
    if distributed:
        t = torch.tensor([elapsed_ms, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, fwd_ms, bwd_ms = (float(v) for v in t)
    ms_per_step = elapsed_ms / args.steps
    value = global_rows / (ms_per_step * 1e-3)

    # ---- end to end: host inputs in, loss out, every step ------------------------------------
    e2e_steps = args.e2e_steps or args.steps
    host = {k: x[k].detach().cpu().pin_memory() for k in ("indices", "vals", "target")}
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    copy_stream = torch.cuda.Stream(dev)
    bufs = [{k: torch.empty_like(x[k].detach()) for k in host} for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            for k, t in host.items():
                bufs[slot][k].copy_(t, non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_loop(n):
        for c in consumed:
            c.record()
        upload(0)
        last = 0.0
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
            last = loss.item()                        # device -> host read of the step's result
        return last

    e2e_loop(min(5, e2e_steps))
    barrier()
    t0 = time.perf_counter()
    e2e_loop(e2e_steps)
    barrier()
    e2e_s = time.perf_counter() - t0
    if not kernels_ok():
        raise SystemExit("bench.py: a backward kernel reported a timed-out wait in the end-to-end loop; no number is reported")
    if distributed:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t)
    e2e_value = global_rows * e2e_steps / e2e_s

    if rank == 0:
        peak, peak_kind = hbm_peak()
        alg = algorithmic_bytes(w)                        # per GPU per step
        sw = 2 if w.weight_dtype != "float32" else 4
        # backward launches of the dominant kernel: one per column piece (+ one conversion-only)
        alg_bwd = (rows * w.K * w.D * (sw + 4) + w.F * w.D * (4 + (4 + sw if sw != 4 else 0))
                   + rows * w.D * 4 + rows * w.K * (8 + 4 + 4))
        line = {
            "metric": "hier_topk_fwd_bwd_throughput" if kind == "hier" else "topk_fwd_bwd_throughput",
            "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": w.name, "kind": kind, "B_per_gpu": rows, "global_B": global_rows, "K": w.K,
                       "F": w.F, "D": w.D, "storage": f"{w.weight_dtype} weight/bias/target, {w.vals_dtype} vals",
                       "accumulate": "fp32", "dweight_mode": args.dweight_mode,
                       "parallelism": f"batch-sharded x{world}, decoder replicated" if distributed else "single GPU",
                       "dweight_sum": dweight_sum,
                       "l2": "no flush: the decoder (302 MB at the headline shape) exceeds the 126 MB L2; the "
                             "library's own fp32 gradient slabs are meant to stay L2-resident between launches"},
            "hbm_gbs": alg / (ms_per_step * 1e-3) / 1e9,
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "roofline": {"bound": "hbm", "kernel": "decoder_loss_bwd_pipelined_kernel (one launch per backward) + its two finalising kernels",
                         "achieved": alg_bwd / (bwd_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg_bwd / (bwd_ms * 1e-3) / 1e9 / peak, "peak_source": peak_kind,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get((w.name, kind, args.dweight_mode))},
            "roofline_step": {"bound": "hbm", "achieved": alg / (ms_per_step * 1e-3) / 1e9, "peak": peak,
                              "unit": "GB/s", "frac": alg / (ms_per_step * 1e-3) / 1e9 / peak,
                              "algorithmic_bytes": alg},
            "e2e": {"value": e2e_value, "unit": "rows/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_s / e2e_steps * 1e3},
            "gpu_launches": launches,
            "clocks": clocks.summary(),
        }
        if world == 1 and args.cpu_seconds > 0:
            line["cpu_baseline"] = cpu_reference_rate(w, kind, args.cpu_seconds)
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
