"""CPU: the oracle restatements against the committed outputs of the reference itself."""
import numpy as np
import pytest
import torch

from flexsae_b200.workloads import make_inputs
from oracle import flexsae_oracle as orc
from oracle import torch_reference as tref
from tests.helpers import golden_files, inputs_as_numpy, load_golden, rel_err

FILES = golden_files()


def test_golden_files_present():
    assert len(FILES) >= 30


@pytest.mark.parametrize("path", FILES, ids=lambda p: p.split("/")[-1][:-4])
def test_numpy_oracle_matches_reference_outputs(path):
    w, kind, gold = load_golden(path)
    x = make_inputs(w, "cpu")
    assert float(x["grad_out"]) == float(gold["grad_out"])
    got = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(gold["grad_out"]))
    # The reference evaluates in float32; for a 16-bit decoder its weight[indices] backward
    # accumulates every (row, k) contribution in 16 bits, so hot decoder rows (skewed indices)
    # carry a few per cent of accumulated rounding in the reference's own output.
    tol = {"float32": 2e-5, "bfloat16": 3e-2, "float16": 5e-3}[w.weight_dtype]
    assert abs(got["loss"] - float(gold["loss"])) <= 2e-6 * abs(float(gold["loss"]))
    assert rel_err(got["dvals"], gold["dvals"]) < tol
    assert rel_err(got["dbias"], gold["dbias"]) < tol
    d = orc.digest(got["dweight"])
    assert np.array_equal(d["dweight_rows_idx"], gold["dweight_rows_idx"])
    assert rel_err(d["dweight_rows"], gold["dweight_rows"]) < tol
    assert rel_err(d["dweight_rowproj"], gold["dweight_rowproj"]) < tol
    assert rel_err(d["dweight_colproj"], gold["dweight_colproj"]) < tol
    if "dweight" in gold:
        assert rel_err(got["dweight"], gold["dweight"]) < tol


@pytest.mark.parametrize("path", FILES[::3], ids=lambda p: p.split("/")[-1][:-4])
def test_torch_restatement_matches_reference_outputs(path):
    w, kind, gold = load_golden(path)
    x = make_inputs(w, "cpu")
    torch.set_num_threads(1)
    r = tref.chunked_loss_and_grads(kind, x["indices"], x["weight"], x["vals"], x["bias"], x["target"],
                                    grad_out=float(gold["grad_out"]), chunk_rows=max(1, w.B))
    assert abs(r["loss"] - float(gold["loss"])) <= 1e-6 * abs(float(gold["loss"]))
    tol = {"float32": 1e-6, "bfloat16": 1e-2, "float16": 1e-3}[w.weight_dtype]
    assert rel_err(r["dvals"].float().numpy(), gold["dvals"]) < tol
    assert rel_err(r["dbias"].float().numpy(), gold["dbias"]) < tol
    assert rel_err(orc.digest(r["dweight"].float().numpy())["dweight_rowproj"], gold["dweight_rowproj"]) < tol


def test_chunking_is_exact_up_to_summation_order():
    w, kind, gold = load_golden([f for f in FILES if "c1__hier" in f][0])
    x = make_inputs(w, "cpu")
    r = tref.chunked_loss_and_grads(kind, x["indices"], x["weight"], x["vals"], x["bias"], x["target"],
                                    grad_out=float(gold["grad_out"]), chunk_rows=7)
    assert abs(r["loss"] - float(gold["loss"])) <= 1e-5 * abs(float(gold["loss"]))
    assert rel_err(r["dbias"].numpy(), gold["dbias"]) < 1e-5
    assert rel_err(r["dvals"].numpy(), gold["dvals"]) < 1e-5


def test_hier_with_k1_equals_topk():
    w, _, _ = load_golden([f for f in FILES if "k1_float32__hier" in f][0])
    x = inputs_as_numpy(make_inputs(w, "cpu"))
    a, b = orc.hier_loss_and_grads(**x), orc.topk_loss_and_grads(**x)
    for k in ("loss", "dweight", "dvals", "dbias"):
        assert np.allclose(a[k], b[k], rtol=1e-12, atol=0)


def test_oracle_gradients_are_the_derivative():
    """Central differences in float64 on a tiny case: independent of any autograd."""
    rng = np.random.default_rng(0)
    B, K, F, D = 3, 4, 6, 5
    idx = rng.integers(0, F, (B, K))
    W, v, b0, t = rng.normal(size=(F, D)), np.abs(rng.normal(size=(B, K))), rng.normal(size=D), rng.normal(size=(B, D))
    for fn in orc.LOSSES.values():
        g = fn(idx, W, v, b0, t, grad_out=1.7)
        eps = 1e-6
        for name, arr, pos in (("dweight", W, (int(idx[1, 2]), 3)), ("dvals", v, (2, 1)), ("dbias", b0, (4,))):
            orig = arr[pos]
            arr[pos] = orig + eps
            up = fn(idx, W, v, b0, t)["loss"]
            arr[pos] = orig - eps
            dn = fn(idx, W, v, b0, t)["loss"]
            arr[pos] = orig
            assert abs(1.7 * (up - dn) / (2 * eps) - g[name][pos]) < 1e-7
