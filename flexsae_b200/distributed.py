"""Batch-sharded decoder losses for the GPUs of one node.

The reference is single-GPU.  Here every rank holds a shard of the batch rows
(``indices``, ``vals``, ``target``) and a full replica of the decoder (``weight``, ``bias``).
Each rank runs the ordinary fused kernels on its rows with the GLOBAL normaliser
1/(B_global*D) resp. 1/(B_global*K*D), so its loss is its additive share of the global mean and
its gradients are its additive share of the global gradients; one all-reduce(sum) of the scalar
loss in the forward and of ``dweight`` and ``dbias`` in the backward (NCCL over NVLink) gives
every rank exactly what a single GPU would have computed on the whole batch, up to summation
order.  ``dvals`` belongs to the local rows and needs no exchange.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import _native as nv
from . import losses as _losses

# (forward, backward) of one shard; replaceable so that the exchange logic can be exercised on
# CPU ranks (gloo) with any implementation of the local math.
LocalImpl = Tuple[Callable, Callable]


def _fused_local_forward(kind, indices, weight, vals, bias, target, inv_norm):
    loss, saved, (idx_c, w_c, v_c) = _losses.fused_forward(kind, indices, weight, vals, bias, target, inv_norm)
    return loss, (idx_c, w_c, v_c, saved)


def _fused_local_backward(kind, ctx_saved, grad, bias_dtype, inv_norm):
    idx_c, w_c, v_c, saved = ctx_saved
    return _losses.fused_backward(kind, idx_c, w_c, v_c, saved, grad, bias_dtype, inv_norm)


FUSED_IMPL: LocalImpl = (_fused_local_forward, _fused_local_backward)


class _ShardedDecoderLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, kind, group, impl, global_rows, indices, weight, vals, bias, target):
        B, K = indices.shape
        D = weight.shape[1]
        inv_norm = 1.0 / (float(global_rows) * D * (K if kind == nv.HIER else 1))
        fwd, _ = impl
        loss, saved = fwd(kind, indices, weight, vals, bias, target, inv_norm)
        loss = loss.clone()
        dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
        ctx.kind, ctx.group, ctx.impl, ctx.inv_norm, ctx.bias_dtype = kind, group, impl, inv_norm, bias.dtype
        ctx.saved = saved
        return loss

    @staticmethod
    def backward(ctx, grad):
        _, bwd = ctx.impl
        dweight, dvals, dbias = bwd(ctx.kind, ctx.saved, grad, ctx.bias_dtype, ctx.inv_norm)
        ctx.saved = None
        # The dense table first: it is the long transfer; the small one rides behind it.
        dist.all_reduce(dweight, op=dist.ReduceOp.SUM, group=ctx.group)
        dist.all_reduce(dbias, op=dist.ReduceOp.SUM, group=ctx.group)
        return None, None, None, None, None, dweight, dvals, dbias, None


def global_batch_rows(local_rows: int, group=None) -> int:
    """Sum of the ranks' local row counts (shards may be ragged)."""
    t = torch.tensor([local_rows], dtype=torch.int64)
    backend = dist.get_backend(group)
    if backend == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return int(t.item())


def sharded_topk_sae_loss(indices, weight, vals, bias, target, group=None, global_rows: Optional[int] = None,
                          impl: LocalImpl = FUSED_IMPL) -> torch.Tensor:
    """TopK loss of the GLOBAL batch from this rank's rows; identical on every rank."""
    if global_rows is None:
        global_rows = global_batch_rows(indices.shape[0], group)
    return _ShardedDecoderLoss.apply(nv.TOPK, group, impl, global_rows, indices, weight, vals, bias, target)


def sharded_hierarchical_sae_loss(indices, weight, vals, bias, target, group=None, global_rows: Optional[int] = None,
                                  impl: LocalImpl = FUSED_IMPL) -> torch.Tensor:
    """Hierarchical-TopK loss of the GLOBAL batch from this rank's rows; identical on every rank."""
    if global_rows is None:
        global_rows = global_batch_rows(indices.shape[0], group)
    return _ShardedDecoderLoss.apply(nv.HIER, group, impl, global_rows, indices, weight, vals, bias, target)
