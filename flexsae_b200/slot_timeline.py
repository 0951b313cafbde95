"""Slot timeline of the batch-sharded backward, for tuning the cross-GPU exchange.

The sharded backward kernel works through one SLOT per column piece; in every slot its blocks play
three roles (unit blocks accumulate, converting blocks scatter the finished slab to the owners,
exchange blocks reduce and broadcast).  The tuning build of the library (``python -m
flexsae_b200.build --trace``) records, per slot and role, when the first block started and the last
one ended on the GPU's nanosecond timer.  This script runs the headline workload batch-sharded
over the ranks it is launched with, traces ONE step after warm-up and prints the table of the first
and the last rank, followed by the mean step time over ``--steps`` further steps::

    python -m flexsae_b200.build --trace
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29517 -m flexsae_b200.slot_timeline [--workload c3_k128] [--symmetric-dweight] \\
        [--options exchange_offset_pct=25,scatter_rotate=1]

Columns (microseconds since the kernel's first event on that GPU; the GPUs' timers are not
synchronised with each other): first unit block starts / last ends; converting blocks: first
enters, first starts working (after its waits), last ends; exchange blocks likewise.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys

FIELDS = ["unit_start", "unit_end", "conv_entry", "conv_start", "conv_end", "exch_entry", "exch_start", "exch_end"]
KEPT_AS_COMPLEMENT = [True, False, True, True, False, True, True, False]     # minima are stored complemented
SLOTS = 64


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--workload", default="c3_k128")
    ap.add_argument("--kind", default="hier", choices=["hier", "topk"])
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--symmetric-dweight", action="store_true")
    ap.add_argument("--options", default="", help="library options, e.g. exchange_offset_pct=25,scatter_rotate=1")
    ap.add_argument("--out", default="", help="directory for one text file per printed rank (default: stdout only)")
    args = ap.parse_args()

    from . import build as _build
    if not os.path.exists(_build.TRACE_LIB_PATH):
        raise SystemExit("build the tuning library first: python -m flexsae_b200.build --trace")
    if _build._stale(_build.TRACE_LIB_PATH) and int(os.environ.get("RANK", 0)) == 0:
        sys.stderr.write("slot_timeline: the tuning library looks older than the sources; "
                         "rebuild it with python -m flexsae_b200.build --trace\n")
    os.environ["FLEXSAE_LIB"] = _build.TRACE_LIB_PATH

    import numpy as np
    import torch
    import torch.distributed as dist

    from . import _native as nv
    from . import check_status
    from . import distributed as fd
    from .workloads import CONFIGS, make_inputs

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if world < 2:
        raise SystemExit("launch with torch.distributed.run on 2..8 GPUs: the timeline is that of the sharded backward")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    fd.config.symmetric_dweight = args.symmetric_dweight
    for item in filter(None, args.options.split(",")):
        name, value = item.split("=")
        nv.set_option(name, int(value))
    lib = nv.load()
    lib.flexsae_debug_trace_read.restype = ctypes.c_int
    lib.flexsae_debug_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]

    w = CONFIGS[args.workload]
    rows = w.B
    x = make_inputs(w.replace(B=rows * world), dev, row0=rank * rows, rows=rows)
    weight, bias, vals = (x[k].requires_grad_(True) for k in ("weight", "bias", "vals"))
    loss_fn = fd.sharded_hierarchical_sae_loss if args.kind == "hier" else fd.sharded_topk_sae_loss

    def step():
        weight.grad = vals.grad = bias.grad = None
        loss_fn(x["indices"], weight, vals, bias, x["target"], global_rows=rows * world).backward()

    table = np.zeros((SLOTS, len(FIELDS)), dtype=np.uint64)

    def read_table():
        nv.check(lib.flexsae_debug_trace_read(table.ctypes.data, table.nbytes, 1), "flexsae_debug_trace_read")

    for _ in range(args.warmup):
        step()
    read_table()                     # synchronises and clears what the warm-up recorded
    dist.barrier()
    step()
    read_table()
    check_status()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    check_status()
    mean_ms = torch.tensor([e0.elapsed_time(e1) / max(args.steps, 1)], device=dev)
    dist.all_reduce(mean_ms, op=dist.ReduceOp.MAX)

    t = table.copy()
    for f, complemented in enumerate(KEPT_AS_COMPLEMENT):
        if complemented:
            t[:, f] = np.where(table[:, f] != 0, ~table[:, f], 0)
    t0 = int(t[t != 0].min())
    lines = [f"rank {rank} of {world}  workload {w.name} {args.kind}  symmetric_dweight {int(args.symmetric_dweight)}  "
             f"options '{args.options}'  mean step {float(mean_ms):.3f} ms over {args.steps} steps (max over ranks)",
             "slot " + " ".join(f"{n:>10s}" for n in FIELDS)]
    for p in range(SLOTS):
        if t[p].any():
            lines.append(f"{p:4d} " + " ".join(f"{(int(v) - t0) / 1e3:10.1f}" if v else f"{'-':>10s}" for v in t[p]))
    text = "\n".join(lines) + "\n"
    for r in (0, world - 1):         # one after the other so that the tables do not interleave
        if rank == r:
            sys.stdout.write(text)
            sys.stdout.flush()
            if args.out:
                os.makedirs(args.out, exist_ok=True)
                with open(os.path.join(args.out, f"slot_timeline_n{world}_rank{rank}.txt"), "w") as fh:
                    fh.write(text)
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
