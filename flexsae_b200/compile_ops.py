"""The fused losses as ``torch.library`` custom operators, so that they can sit inside
``torch.compile(fullgraph=True)`` graphs.

The reference's fused functions are plain ``autograd.Function``s around Triton launches; its
benchmark compiles only the eager torch loss (example.py:15-28).  Here the forward and the
backward are registered as opaque operators with shape-only ("fake") implementations, and
autograd is wired between them, so a compiled training step can contain the CUDA losses:

    step = torch.compile(lambda i, w, v, b, t: flexsae_b200.compile_ops.hierarchical_sae_loss(i, w, v, b, t),
                         fullgraph=True)

``flexsae_b200.triton_*_sae_loss`` switch to these operators by themselves while a graph is being
traced (``torch.compiler.is_compiling()``); eager calls keep using the ``autograd.Function``.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _native as nv
from . import losses as _losses


def _segments_for(kind: int, indices: torch.Tensor, weight: torch.Tensor) -> int:
    B, K = (int(x) for x in indices.shape)
    F, D = (int(x) for x in weight.shape)
    return nv.load().flexsae_choose_segments(kind, B, K, F, D, nv.DTYPE_CODES[weight.dtype])


def _segments_of_state(kind: int, state: torch.Tensor, indices: torch.Tensor, weight: torch.Tensor) -> int:
    """The K-segment count a saved state was written with, from its size alone."""
    rows, width = int(indices.shape[0]), int(weight.shape[1])
    per = rows * width
    n = int(state.numel())
    return 1 if (kind == nv.TOPK or n == per) else n // (2 * per)


@torch.library.custom_op("flexsae_b200::decoder_loss_fwd", mutates_args=(), device_types="cuda")
def decoder_loss_fwd(kind: int, inv_norm: float, indices: torch.Tensor, weight: torch.Tensor, vals: torch.Tensor,
                     bias: torch.Tensor, target: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    loss, (state, _segments), _ = _losses.fused_forward(kind, indices, weight, vals, bias, target, inv_norm)
    return loss, state


@decoder_loss_fwd.register_fake
def _decoder_loss_fwd_fake(kind, inv_norm, indices, weight, vals, bias, target):
    B, K = (int(x) for x in indices.shape)
    D = int(weight.shape[1])
    segments = _segments_for(kind, indices, weight)
    n = nv.load().flexsae_state_bytes(kind, B, K, D, segments) // 4
    return weight.new_empty((), dtype=torch.float32), weight.new_empty((n,), dtype=torch.float32)


@torch.library.custom_op("flexsae_b200::decoder_loss_bwd", mutates_args=(), device_types="cuda")
def decoder_loss_bwd(kind: int, inv_norm: float, indices: torch.Tensor, weight: torch.Tensor, vals: torch.Tensor,
                     bias: torch.Tensor, state: torch.Tensor,
                     grad: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    idx_c, w_c, v_c = (_losses._prep(t.detach()) for t in (indices, weight, vals))
    segments = _segments_of_state(kind, state, indices, weight)
    return _losses.fused_backward(kind, idx_c, w_c, v_c, (state, segments), grad, bias.dtype, inv_norm)


@decoder_loss_bwd.register_fake
def _decoder_loss_bwd_fake(kind, inv_norm, indices, weight, vals, bias, state, grad):
    return torch.empty_like(weight, memory_format=torch.contiguous_format), \
        torch.empty_like(vals, memory_format=torch.contiguous_format), \
        torch.empty_like(bias, memory_format=torch.contiguous_format)


def _setup_context(ctx, inputs, output):
    kind, inv_norm, indices, weight, vals, bias, _target = inputs
    _loss, state = output
    ctx.kind, ctx.inv_norm = kind, inv_norm
    ctx.save_for_backward(indices, weight, vals, bias, state)


def _backward(ctx, grad_loss, _grad_state):
    indices, weight, vals, bias, state = ctx.saved_tensors
    dweight, dvals, dbias = decoder_loss_bwd(ctx.kind, ctx.inv_norm, indices, weight, vals, bias, state, grad_loss)
    return None, None, None, dweight, dvals, dbias, None


decoder_loss_fwd.register_autograd(_backward, setup_context=_setup_context)


def topk_sae_loss(indices, weight, vals, bias, target) -> torch.Tensor:
    """Fused TopK loss through the custom operator (works in eager mode and under torch.compile)."""
    return decoder_loss_fwd(nv.TOPK, 0.0, indices, weight, vals, bias, target)[0]


def hierarchical_sae_loss(indices, weight, vals, bias, target) -> torch.Tensor:
    """Fused Hierarchical-TopK loss through the custom operator."""
    return decoder_loss_fwd(nv.HIER, 0.0, indices, weight, vals, bias, target)[0]
