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
