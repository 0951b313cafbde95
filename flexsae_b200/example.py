"""The reference's benchmark script for this library: fused loss against the torch loss on one GPU.

Same protocol as the reference's ``example.py`` (lines 30-96): fresh random parameters every
iteration (``vals = |randn|``, ``randint`` indices with duplicates, N(0,1) decoder / bias / target),
CUDA events around ``loss = f(...); loss.backward()``, 5 warm-up + 100 timed iterations, mean ± std,
a closeness check of the two losses and the speed-up.  ``--table`` prints the reference README's
table instead (README.md:163-172): ms per step and peak device memory in GiB for TopK and
HierarchicalTopK at K = 32, 64, 128 with F = 65536, D = 2304.

    python -m flexsae_b200.example                      # B=2048 K=256 F=131072 D=1024 fp32, hierarchical
    python -m flexsae_b200.example --kind topk --dtype bf16 --B 4096 --K 128 --F 65536 --D 2304
    python -m flexsae_b200.example --table --B 4096

``--reference-path DIR`` also times the reference's own Triton kernels when a copy of its package
directory (``torch-ext/flex_sae`` of corl-team/flexsae) is at hand; it is loaded from ``DIR`` under
another module name and is not part of this library.

The torch side is eager by default (``--compile`` wraps it in ``torch.compile(fullgraph=True)`` as
the reference script does); it materialises [B, K, D] in fp32, so its batch is processed in chunks
of ``--torch-chunk`` rows when that would not fit.
"""
from __future__ import annotations

import argparse
import statistics
from typing import Callable, Dict, List, Optional

import torch

from . import hierarchical_sae_loss, topk_sae_loss, triton_hierarchical_sae_loss, triton_topk_sae_loss

DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def make_parameters(B: int, K: int, F: int, D: int, dtype: torch.dtype, device: torch.device) -> Dict[str, torch.Tensor]:
    """The reference script's ``init_parameters`` (example.py:45-51); vals stay fp32 when the decoder is 16-bit."""
    return {
        "vals": torch.randn(B, K, dtype=torch.float32, device=device).abs().requires_grad_(),
        "weight": torch.randn(F, D, dtype=dtype, device=device, requires_grad=True),
        "bias": torch.randn(D, dtype=dtype, device=device, requires_grad=True),
        "target": torch.randn(B, D, dtype=dtype, device=device),
        "indices": torch.randint(0, F, (B, K), dtype=torch.long, device=device),
    }


def _drop_grads(p: Dict[str, torch.Tensor]) -> None:
    p["vals"].grad = p["weight"].grad = p["bias"].grad = None


def _step(fn: Callable, p: Dict[str, torch.Tensor]) -> torch.Tensor:
    loss = fn(p["indices"], p["weight"], p["vals"], p["bias"], p["target"])
    loss.backward()
    return loss.detach()


def _torch_step_chunked(fn: Callable, p: Dict[str, torch.Tensor], chunk: int) -> torch.Tensor:
    """The torch loss over row chunks (mean of equal-sized chunk means = the full mean; the last,
    smaller chunk is weighted by its share)."""
    B = p["indices"].shape[0]
    total = torch.zeros((), dtype=torch.float32, device=p["weight"].device)
    for r0 in range(0, B, chunk):
        r1 = min(B, r0 + chunk)
        loss = fn(p["indices"][r0:r1], p["weight"], p["vals"][r0:r1], p["bias"], p["target"][r0:r1]) * ((r1 - r0) / B)
        loss.backward()
        total += loss.detach()
    return total


def time_one(fn: Callable, B: int, K: int, F: int, D: int, dtype: torch.dtype, device: torch.device, warmup: int,
             iters: int, chunk: Optional[int] = None) -> Dict[str, float]:
    """ms per fwd+bwd step (mean, std, min), peak device memory of the steps in GiB, last loss."""
    times: List[float] = []
    loss = None
    peak = 0
    for i in range(warmup + iters):
        p = make_parameters(B, K, F, D, dtype, device)
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loss = _torch_step_chunked(fn, p, chunk) if chunk else _step(fn, p)
        e1.record()
        torch.cuda.synchronize(device)
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
            peak = max(peak, torch.cuda.max_memory_allocated(device))
        _drop_grads(p)
        del p
    return {"ms": statistics.fmean(times), "std": statistics.pstdev(times), "min": min(times),
            "gib": peak / 2 ** 30, "loss": float(loss)}


def load_reference_package(path: str):
    """The reference's ``flex_sae`` package from a directory that holds its ``__init__.py``, imported
    as ``flex_sae_reference`` (this repository ships its own ``flex_sae`` alias, so the name is taken)."""
    import importlib.util
    import os
    import sys

    init = os.path.join(path, "__init__.py")
    if not os.path.exists(init):
        raise SystemExit(f"--reference-path: {init} not found (point it at the reference's torch-ext/flex_sae directory)")
    spec = importlib.util.spec_from_file_location("flex_sae_reference", init, submodule_search_locations=[path])
    module = importlib.util.module_from_spec(spec)
    sys.modules["flex_sae_reference"] = module
    spec.loader.exec_module(module)
    return module


def compare(kind: str, B: int, K: int, F: int, D: int, dtype: torch.dtype, device: torch.device, warmup: int, iters: int,
            compile_torch: bool = False, torch_chunk: int = 0, reference=None) -> Dict[str, object]:
    """Both implementations on identical parameters once (closeness), then each timed on its own;
    with ``reference`` (the reference package) its Triton kernel is timed as well."""
    fused = triton_hierarchical_sae_loss if kind == "hier" else triton_topk_sae_loss
    plain = hierarchical_sae_loss if kind == "hier" else topk_sae_loss
    if compile_torch:
        plain = torch.compile(plain, fullgraph=True)
    chunk = torch_chunk if 0 < torch_chunk < B else None
    p = make_parameters(B, K, F, D, dtype, device)
    loss_fused = float(_step(fused, p))
    _drop_grads(p)
    loss_plain = float(_torch_step_chunked(plain, p, chunk) if chunk else _step(plain, p))
    _drop_grads(p)
    del p
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    out = {
        "close": abs(loss_fused - loss_plain) <= tol * abs(loss_plain), "loss_fused": loss_fused, "loss_torch": loss_plain,
        "fused": time_one(fused, B, K, F, D, dtype, device, warmup, iters),
        "torch": time_one(plain, B, K, F, D, dtype, device, warmup, iters, chunk),
    }
    if reference is not None:
        ref_fn = reference.triton_hierarchical_sae_loss if kind == "hier" else reference.triton_topk_sae_loss
        out["reference_triton"] = time_one(ref_fn, B, K, F, D, dtype, device, warmup, iters)
    return out


def format_table(rows: Dict[str, Dict[int, Dict[str, float]]], ks: List[int]) -> str:
    """``rows[label][K] = {"ms": ..., "gib": ...}`` -> the README-style markdown table."""
    head = "| Decoder backend | " + " | ".join(f"K={k} (ms / GiB)" for k in ks) + " |"
    rule = "| --- |" + " --- |" * len(ks)
    body = ["| " + label + " | " + " | ".join(f"{rows[label][k]['ms']:.3f} / {rows[label][k]['gib']:.2f}" for k in ks) + " |"
            for label in rows]
    return "\n".join([head, rule] + body)


def main(argv: Optional[List[str]] = None) -> Dict[str, object]:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--kind", default="hier", choices=["hier", "topk"])
    ap.add_argument("--B", type=int, default=2048)
    ap.add_argument("--K", type=int, default=256)
    ap.add_argument("--F", type=int, default=1024 * 128)
    ap.add_argument("--D", type=int, default=1024)
    ap.add_argument("--dtype", default="fp32", choices=sorted(DTYPES))
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--compile", action="store_true", help="torch.compile(fullgraph=True) around the torch loss")
    ap.add_argument("--torch-chunk", type=int, default=0, help="rows per chunk of the torch loss (0 = whole batch)")
    ap.add_argument("--table", action="store_true", help="the README table: F=65536 D=2304 K in 32,64,128, bf16 unless --dtype")
    ap.add_argument("--reference-path", default="", help="directory of the reference's flex_sae package: time its Triton kernels too")
    args = ap.parse_args(argv)
    reference = load_reference_package(args.reference_path) if args.reference_path else None
    if not torch.cuda.is_available():
        raise SystemExit("flexsae_b200.example needs a CUDA device: the fused losses have no CPU path")
    device = torch.device("cuda", torch.cuda.current_device())
    if args.table:
        dtype = DTYPES[args.dtype if args.dtype != "fp32" else "bf16"]
        ks = [32, 64, 128]
        rows: Dict[str, Dict[int, Dict[str, float]]] = {}
        for kind, name in (("topk", "TopK"), ("hier", "HierarchicalTopK")):
            for k in ks:
                r = compare(kind, args.B, k, 65536, 2304, dtype, device, args.warmup, args.iters, args.compile,
                            args.torch_chunk or 512, reference)
                rows.setdefault(f"torch {name}", {})[k] = r["torch"]
                if reference is not None:
                    rows.setdefault(f"reference Triton {name}", {})[k] = r["reference_triton"]
                rows.setdefault(f"fused (sm_100a) {name}", {})[k] = r["fused"]
        print(format_table(rows, ks))
        return {"rows": rows}
    r = compare(args.kind, args.B, args.K, args.F, args.D, DTYPES[args.dtype], device, args.warmup, args.iters,
                args.compile, args.torch_chunk, reference)
    print("outputs are close" if r["close"] else f"outputs MISMATCH: fused {r['loss_fused']} torch {r['loss_torch']}")
    f, t = r["fused"], r["torch"]
    print(f"fused kernels (ours): {f['ms']:.4f} ± {f['std']:.4f} ms   peak {f['gib']:.2f} GiB")
    print(f"torch loss:           {t['ms']:.4f} ± {t['std']:.4f} ms   peak {t['gib']:.2f} GiB")
    print(f"speed-up: {t['ms'] / f['ms']:.2f}x")
    if "reference_triton" in r:
        q = r["reference_triton"]
        print(f"reference Triton:     {q['ms']:.4f} ± {q['std']:.4f} ms   peak {q['gib']:.2f} GiB   ({q['ms'] / f['ms']:.2f}x ours)")
    return r


if __name__ == "__main__":
    main()
