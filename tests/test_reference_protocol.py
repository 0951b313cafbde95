"""GPU: the reference's own acceptance test, run through the import name the reference uses.

Protocol of the reference's ``run_funcs`` (tests/test_all_kernels.py:20-50, tests/test_setup.py:3-41):
torch's own generator seeded with 1234; ``indices`` from ``randint`` (repeats allowed), ``vals`` =
|randn| in the test dtype, decoder / bias / target from ``randn`` in the test dtype, all drawn on the
GPU; the fused loss against the package's eager loss on detached copies; a random float32 upstream
gradient; ``torch.testing.assert_close`` with the reference's tolerance per dtype on the loss and on
the three gradients; no gradient for ``indices``.  26 shapes x 3 dtypes x 2 losses.
"""
import pytest
import torch

import flex_sae
from tests.test_gpu_parity import REF_PARAMS

pytestmark = pytest.mark.gpu

TOLS = {torch.float32: dict(atol=1e-4, rtol=1e-3), torch.bfloat16: dict(atol=1e-2, rtol=1e-2),
        torch.float16: dict(atol=1e-3, rtol=1e-3)}          # tests/test_setup.py:35-39
PAIRS = {"hier": (flex_sae.triton_hierarchical_sae_loss, flex_sae.hierarchical_sae_loss),
         "topk": (flex_sae.triton_topk_sae_loss, flex_sae.topk_sae_loss)}


@pytest.mark.parametrize("kind", ["hier", "topk"])
@pytest.mark.parametrize("dtype", list(TOLS), ids=lambda d: str(d).split(".")[-1])
@pytest.mark.parametrize("B,K,F,D", REF_PARAMS)
def test_fused_loss_against_eager_loss_with_the_reference_protocol(B, K, F, D, dtype, kind):
    fused, eager = PAIRS[kind]
    dev = torch.device("cuda")
    torch.manual_seed(1234)
    indices = torch.randint(0, F, (B, K), dtype=torch.long, device=dev)
    vals = torch.randn(B, K, dtype=dtype, device=dev).abs().requires_grad_()
    decoder = torch.randn(F, D, dtype=dtype, device=dev, requires_grad=True)
    bias = torch.randn(D, dtype=dtype, device=dev, requires_grad=True)
    target = torch.randn(B, D, dtype=dtype, device=dev)
    twins = [t.detach().clone().requires_grad_() for t in (decoder, vals, bias)]

    got = fused(indices, decoder, vals, bias, target)
    want = eager(indices, twins[0], twins[1], twins[2], target)
    torch.testing.assert_close(got, want, **TOLS[dtype])

    upstream = torch.randn((), device=dev, dtype=torch.float32)
    got.backward(upstream)
    want.backward(upstream.clone())
    for mine, theirs in zip((decoder, vals, bias), twins):
        torch.testing.assert_close(mine.grad, theirs.grad, **TOLS[dtype])
    assert indices.grad is None and target.grad is None
