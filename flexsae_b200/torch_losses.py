"""Eager torch versions of the two losses, exported because the reference package exports them
(``topk_sae_loss`` topk_kernels.py:226-237, ``hierarchical_sae_loss``
hierarchical_kernels.py:312-323).  They run on whatever device their tensors live on, build the
[B, K, D] intermediate, and are NOT used by the fused path in any way."""
from __future__ import annotations

import torch


def topk_sae_loss(indices: torch.Tensor, weight: torch.Tensor, vals: torch.Tensor, bias: torch.Tensor,
                  target: torch.Tensor) -> torch.Tensor:
    picked = weight[indices].to(torch.float32)                       # [B, K, D]
    recon = bias.to(torch.float32) + torch.einsum("bkd,bk->bd", picked, vals.to(torch.float32))
    return torch.mean(torch.square(recon - target.to(torch.float32)))


def hierarchical_sae_loss(indices: torch.Tensor, weight: torch.Tensor, vals: torch.Tensor, bias: torch.Tensor,
                          target: torch.Tensor) -> torch.Tensor:
    picked = weight[indices].to(torch.float32)                       # [B, K, D]
    prefixes = torch.cumsum(picked * vals.to(torch.float32)[..., None], dim=1) + bias.to(torch.float32)
    return torch.mean(torch.square(prefixes - target.to(torch.float32)[:, None, :]))
