"""flexsae_b200: the fused TopK / Hierarchical-TopK sparse-autoencoder decoder losses for
NVIDIA B200, with the public names of the reference package ``flex_sae``
(torch-ext/flex_sae/__init__.py:5-18), so that ``import flexsae_b200 as flex_sae`` is a drop-in.
"""
from .losses import (check_status, config, triton_hierarchical_sae_loss,  # noqa: F401
                     triton_topk_sae_loss)
from .torch_losses import hierarchical_sae_loss, topk_sae_loss  # noqa: F401

__kernel_metadata__ = {
    "license": "Apache-2.0",
    "backend": "cuda-sm_100a",
}

__all__ = [
    "__kernel_metadata__",
    "topk_sae_loss",
    "triton_topk_sae_loss",
    "hierarchical_sae_loss",
    "triton_hierarchical_sae_loss",
]
