"""CPU: the exported eager losses (``flexsae_b200.topk_sae_loss`` / ``hierarchical_sae_loss``, also
reachable as ``flex_sae.*``) against the committed outputs of the reference, and the alias package."""
import numpy as np
import pytest
import torch

import flexsae_b200 as fx
from flexsae_b200.workloads import make_inputs
from oracle import flexsae_oracle as orc
from tests.helpers import golden_files, load_golden, rel_err

EXPORTED = {"topk": fx.topk_sae_loss, "hier": fx.hierarchical_sae_loss}


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1][:-4])
def test_exported_eager_losses_match_reference_outputs(path):
    w, kind, gold = load_golden(path)
    x = make_inputs(w, "cpu")
    torch.set_num_threads(1)
    wt = x["weight"].clone().requires_grad_(True)
    v = x["vals"].clone().requires_grad_(True)
    b = x["bias"].clone().requires_grad_(True)
    loss = EXPORTED[kind](x["indices"], wt, v, b, x["target"])
    assert loss.dtype == torch.float32 and loss.dim() == 0
    loss.backward(torch.tensor(float(gold["grad_out"])))
    assert wt.grad.dtype == wt.dtype and v.grad.dtype == v.dtype and b.grad.dtype == b.dtype
    assert abs(float(loss) - float(gold["loss"])) <= 2e-6 * abs(float(gold["loss"]))
    # 16-bit decoders: the reference's own gradient is accumulated in 16 bits, in an order that
    # differs between operator spellings, hence the dtype's rounding as the tolerance
    tol = {"float32": 2e-6, "bfloat16": 2e-2, "float16": 2e-3}[w.weight_dtype]
    assert rel_err(v.grad.float().numpy(), gold["dvals"]) < tol
    assert rel_err(b.grad.float().numpy(), gold["dbias"]) < tol
    d = orc.digest(wt.grad.double().numpy())
    assert np.array_equal(d["dweight_rows_idx"], gold["dweight_rows_idx"])
    assert rel_err(d["dweight_rows"], gold["dweight_rows"]) < tol
    assert rel_err(d["dweight_rowproj"], gold["dweight_rowproj"]) < tol


def test_alias_package_exports_the_reference_names():
    import flex_sae

    for name in ("triton_topk_sae_loss", "triton_hierarchical_sae_loss", "topk_sae_loss", "hierarchical_sae_loss",
                 "__kernel_metadata__"):
        assert getattr(flex_sae, name) is getattr(fx, name)
    assert sorted(flex_sae.__all__) == sorted(fx.__all__)
