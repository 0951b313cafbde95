"""Writes tests/golden/<case>__<kind>.npz from the UNMODIFIED reference.

Run where the reference checkout is available (it is not on the GPU machines):

    python tests/golden/make_golden.py --reference /path/to/flexsae

It imports ``flex_sae`` from ``<reference>/torch-ext`` and runs the reference's own eager torch
losses (``topk_sae_loss`` topk_kernels.py:226-237, ``hierarchical_sae_loss``
hierarchical_kernels.py:312-323) on CPU, with torch autograd for the gradients and the same
backward call as the reference's parity harness (tests/test_all_kernels.py:42-48: a random
float32 upstream scalar).  Inputs are not stored: each file records the workload description
and the tests rebuild the tensors from it with ``flexsae_b200.workloads.make_inputs`` on CPU.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from flexsae_b200.workloads import make_inputs  # noqa: E402
from oracle.flexsae_oracle import digest  # noqa: E402
from tests.golden.cases import FULL_DWEIGHT_MAX_ELEMS, GOLDEN_CASES, KINDS  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "torch-ext"))
    import flex_sae  # the reference package

    ref_fns = {"topk": flex_sae.topk_sae_loss, "hier": flex_sae.hierarchical_sae_loss}
    torch.set_num_threads(1)          # fixed summation order inside torch's CPU kernels
    for w in GOLDEN_CASES:
        x = make_inputs(w, "cpu")
        for kind in KINDS:
            weight = x["weight"].clone().requires_grad_(True)
            vals = x["vals"].clone().requires_grad_(True)
            bias = x["bias"].clone().requires_grad_(True)
            loss = ref_fns[kind](x["indices"], weight, vals, bias, x["target"])
            loss.backward(x["grad_out"].clone())
            assert loss.dtype == torch.float32 and loss.dim() == 0
            assert weight.grad.dtype == weight.dtype and vals.grad.dtype == vals.dtype
            dW = weight.grad.float().numpy()
            out = {
                "workload": np.array(json.dumps(dataclasses.asdict(w))),
                "kind": np.array(kind),
                "grad_out": x["grad_out"].numpy(),
                "loss": loss.detach().numpy(),
                "dvals": vals.grad.float().numpy(),
                "dbias": bias.grad.float().numpy(),
            }
            out.update(digest(dW))
            if dW.size <= FULL_DWEIGHT_MAX_ELEMS:
                out["dweight"] = dW
            path = os.path.join(HERE, f"{w.name}__{kind}.npz")
            np.savez_compressed(path, **out)
            print(f"{os.path.basename(path):48s} loss={float(loss):.6f} {os.path.getsize(path)} B")


if __name__ == "__main__":
    main()
