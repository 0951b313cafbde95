"""The step in front of the decoder losses: encoder activations -> (indices, vals).

The reference starts from ``indices[B,K]`` and ``vals[B,K]`` and leaves their production to the
caller (its tests and example draw them at random: tests/test_all_kernels.py:20-33,
example.py:45-51); in a TopK sparse autoencoder they are the K largest encoder activations of each
row.  ``topk_activations`` selects them with one CUDA launch (``flexsae_topk_select``: exact radix
select, values in descending order, equal values by ascending index, int64 indices -- the layout
the loss kernels take), and is differentiable with respect to the activations.  ``encode_topk`` puts
the encoder's linear map (a plain library GEMM) in front of it.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _native as nv
from . import losses as _losses


def select_topk(acts: torch.Tensor, k: int, relu: bool = True,
                vals_dtype: Optional[torch.dtype] = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Runs the selection kernel (no autograd); returns ``(indices int64 [B,K], vals [B,K])``."""
    if acts.dim() != 2:
        raise ValueError("activations must be [B, F]")
    if not acts.is_cuda:
        raise RuntimeError("flexsae_b200.producer needs CUDA tensors: there is no CPU path")
    if acts.dtype not in nv.DTYPE_CODES:
        raise TypeError(f"unsupported activation dtype {acts.dtype}")
    vals_dtype = vals_dtype or acts.dtype
    B, F = acts.shape
    lib = nv.load()
    acts = acts.detach().contiguous()
    with torch.cuda.device(acts.device):
        vals = torch.empty((B, k), dtype=vals_dtype, device=acts.device)
        indices = torch.empty((B, k), dtype=torch.int64, device=acts.device)
        rc = lib.flexsae_topk_select(acts.data_ptr(), nv.DTYPE_CODES[acts.dtype], B, F, k, int(bool(relu)), vals.data_ptr(),
                                     nv.DTYPE_CODES[vals_dtype], indices.data_ptr(),
                                     torch.cuda.current_stream(acts.device).cuda_stream)
        nv.check(rc, "flexsae_topk_select")
        _losses.launch_count += lib.flexsae_last_launch_count()
    return indices, vals


class _TopKActivations(torch.autograd.Function):
    @staticmethod
    def forward(ctx, acts, k, relu, vals_dtype):
        indices, vals = select_topk(acts, k, relu, vals_dtype)
        ctx.save_for_backward(indices, vals)
        ctx.relu, ctx.shape, ctx.dtype = relu, acts.shape, acts.dtype
        ctx.mark_non_differentiable(indices)
        return indices, vals

    @staticmethod
    def backward(ctx, _grad_indices, grad_vals):
        indices, vals = ctx.saved_tensors
        g = grad_vals.to(torch.float32)
        if ctx.relu:
            g = g * (vals > 0)                     # clamped entries pass no gradient
        grad_acts = torch.zeros(ctx.shape, dtype=ctx.dtype, device=grad_vals.device)
        grad_acts.scatter_(1, indices, g.to(ctx.dtype))      # indices of a row are distinct
        return grad_acts, None, None, None


def topk_activations(acts: torch.Tensor, k: int, relu: bool = True,
                     vals_dtype: Optional[torch.dtype] = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(indices, vals)`` of the ``k`` largest activations per row, ready for
    ``triton_topk_sae_loss`` / ``triton_hierarchical_sae_loss``; ``vals`` carries gradient back to
    ``acts`` (zero for everything not selected and, with ``relu``, for values clamped at zero)."""
    return _TopKActivations.apply(acts, k, relu, vals_dtype)


def encode_topk(x: torch.Tensor, w_enc: torch.Tensor, b_enc: Optional[torch.Tensor], k: int, relu: bool = True,
                vals_dtype: Optional[torch.dtype] = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Encoder of a TopK sparse autoencoder: ``topk_activations(x @ w_enc.T + b_enc, k)`` with
    ``w_enc`` stored [F, D_in] like ``torch.nn.Linear.weight``."""
    return topk_activations(torch.nn.functional.linear(x, w_enc, b_enc), k, relu, vals_dtype)


def _main(argv=None) -> dict:
    """``python -m flexsae_b200.producer``: time the selection kernel on synthetic activations and
    print one JSON line (rows/s, achieved GB/s of algorithmic bytes: the activations read once plus
    the (index, value) pairs written)."""
    import argparse
    import json

    ap = argparse.ArgumentParser(description="time flexsae_topk_select on synthetic activations")
    ap.add_argument("--B", type=int, default=4096)
    ap.add_argument("--F", type=int, default=65536)
    ap.add_argument("--K", type=int, default=128)
    ap.add_argument("--dtype", default="bf16", choices=["fp32", "bf16", "fp16"])
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("flexsae_b200.producer needs a CUDA device")
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[args.dtype]
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)
    # two buffers larger than L2 together, used in turn, so that no step finds its rows cached
    acts = [torch.randn(args.B, args.F, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(2)]
    for i in range(args.warmup):
        select_topk(acts[i & 1], args.K)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        select_topk(acts[i & 1], args.K)
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / args.steps
    # what the reference's callers run in this place: torch.topk followed by a ReLU, same inputs
    lib_steps = max(3, args.steps // 5)
    for i in range(2):
        torch.topk(acts[i & 1], args.K, dim=1, sorted=True)
    e0.record()
    for i in range(lib_steps):
        v, _ = torch.topk(acts[i & 1], args.K, dim=1, sorted=True)
        v.clamp_min_(0)
    e1.record()
    torch.cuda.synchronize(dev)
    torch_ms = e0.elapsed_time(e1) / lib_steps
    alg = args.B * args.F * acts[0].element_size() + args.B * args.K * (8 + 4)
    # torch.topk leaves the order of equal values open (16-bit activations tie often), so compare what
    # is defined: the selected values, and that every index really holds its value
    ref_vals = torch.topk(acts[0].float(), args.K, dim=1, sorted=True).values.clamp_min(0)
    got_idx, got_vals = select_topk(acts[0], args.K)
    same = bool(torch.equal(got_vals, ref_vals)) and \
        bool(torch.equal(acts[0].float().gather(1, got_idx).clamp_min(0), got_vals))
    line = {"metric": "topk_select_throughput", "value": args.B / (ms * 1e-3), "unit": "rows/s", "ms_per_step": ms,
            "config": {"B": args.B, "F": args.F, "K": args.K, "dtype": args.dtype,
                       "l2": "two input buffers used in turn" + ("" if 2 * acts[0].numel() * acts[0].element_size() > 256e6
                                                                 else " (smaller than L2 together: cached reads)")},
            "algorithmic_bytes": alg, "achieved_gbs": alg / (ms * 1e-3) / 1e9, "matches_torch_topk": same,
            "torch_topk_ms": torch_ms}
    print(json.dumps(line))
    return line


if __name__ == "__main__":
    _main()
