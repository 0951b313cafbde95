"""``flex_sae``: the reference package's import name, served by ``flexsae_b200``.

Code written against the reference -- ``from flex_sae import triton_hierarchical_sae_loss``
(tests/test_all_kernels.py:7-12 of the reference), ``flex_sae.topk_sae_loss(...)`` -- runs unchanged
with this directory on ``sys.path``: the five public names of torch-ext/flex_sae/__init__.py:5-18
are re-exported from the B200 implementation.  Nothing else lives here.
"""
from flexsae_b200 import (__kernel_metadata__, hierarchical_sae_loss, topk_sae_loss,  # noqa: F401
                          triton_hierarchical_sae_loss, triton_topk_sae_loss)

__all__ = [
    "__kernel_metadata__",
    "topk_sae_loss",
    "triton_topk_sae_loss",
    "hierarchical_sae_loss",
    "triton_hierarchical_sae_loss",
]
