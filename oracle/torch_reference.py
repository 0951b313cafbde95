"""The reference's eager torch losses, restated for timing and large-shape checks.
TEST / BASELINE INFRASTRUCTURE ONLY: nothing in ``flexsae_b200`` imports this file.

Same operator sequence as torch-ext/flex_sae/topk_kernels.py:226-237 and
torch-ext/flex_sae/hierarchical_kernels.py:312-323: gather ``weight[indices]``, upcast to
float32, scale by ``vals``, (cumulative) sum over K, add bias, subtract target, mean of
squares; gradients come from torch autograd.  It materialises [rows, K, D] float32 tensors
several times over, so ``chunked_loss_and_grads`` feeds it a few hundred rows at a time;
the loss is a mean, so chunk losses add up after weighting by rows/B and ``.grad`` accumulates.

``tests/test_oracle.py`` checks these functions against the golden outputs of the reference.
"""
from __future__ import annotations

import time
from typing import Dict, Optional

import torch


def topk_reference_loss(indices, weight, vals, bias, target) -> torch.Tensor:
    rows = weight[indices].float()                                   # topk_kernels.py:233
    recon = bias.float() + (rows * vals.unsqueeze(-1)).sum(dim=1)     # topk_kernels.py:234
    return (recon.float() - target.float()).pow(2).mean()            # topk_kernels.py:235-236


def hier_reference_loss(indices, weight, vals, bias, target) -> torch.Tensor:
    rows = weight[indices].float()                                          # hierarchical_kernels.py:319
    prefixes = bias.float() + (rows * vals.unsqueeze(-1)).cumsum(dim=1)      # :320
    return (prefixes.float() - target.float().unsqueeze(1)).pow(2).mean()   # :321-322


REFERENCE_LOSSES = {"topk": topk_reference_loss, "hier": hier_reference_loss}


def chunked_loss_and_grads(kind: str, indices, weight, vals, bias, target, grad_out=1.0,
                           chunk_rows: int = 256, max_rows: Optional[int] = None,
                           upcast: bool = False) -> Dict[str, object]:
    """fwd + backward of the reference loss over the batch in ``chunk_rows`` pieces.

    ``max_rows`` stops after that many rows (a bounded timing sample); the gradients then
    cover only those rows while keeping the full batch's normaliser.  ``upcast`` runs the
    float32 copy of 16-bit operands, which removes the 16-bit accumulation of
    ``weight[indices]``'s backward and is the cleaner target for a float32-accumulating kernel.
    Returns loss (float), the three gradients, the rows processed and the seconds spent.
    """
    fn = REFERENCE_LOSSES[kind]
    B = indices.shape[0]
    if upcast:
        weight, vals, bias, target = weight.float(), vals.float(), bias.float(), target.float()
    w = weight.detach().clone().requires_grad_(True)
    bs = bias.detach().clone().requires_grad_(True)
    dvals = torch.zeros_like(vals)
    loss_total = 0.0
    rows_done = 0
    go = float(grad_out)
    t0 = time.perf_counter()
    limit = B if max_rows is None else min(B, max_rows)
    for r0 in range(0, limit, chunk_rows):
        r1 = min(limit, r0 + chunk_rows)
        v = vals[r0:r1].detach().clone().requires_grad_(True)
        loss = fn(indices[r0:r1], w, v, bs, target[r0:r1])
        share = (r1 - r0) / B
        loss.backward(torch.tensor(go * share, dtype=torch.float32, device=loss.device))
        dvals[r0:r1] = v.grad
        loss_total += float(loss.detach()) * share
        rows_done = r1
    if w.device.type == "cuda":
        torch.cuda.synchronize(w.device)
    dt = time.perf_counter() - t0
    return {"loss": loss_total, "dweight": w.grad, "dvals": dvals, "dbias": bs.grad,
            "rows": rows_done, "seconds": dt}
