"""The custom-operator form of the fused losses: shape-only implementations on CPU (no GPU
needed), and -- on a GPU -- a fullgraph torch.compile of the loss against the eager call."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import flexsae_b200 as fx
from flexsae_b200 import _native as nv
from flexsae_b200 import compile_ops
from flexsae_b200.workloads import Workload, make_inputs


@pytest.mark.parametrize("kind", [nv.TOPK, nv.HIER])
@pytest.mark.parametrize("shape", [(64, 32, 4096, 256), (4096, 128, 65536, 2304)])
def test_fake_implementations_give_the_real_shapes(kind, shape):
    B, K, F, D = shape
    lib = nv.load()
    with FakeTensorMode():
        idx = torch.empty(B, K, dtype=torch.int64, device="cuda")
        w = torch.empty(F, D, dtype=torch.bfloat16, device="cuda")
        v = torch.empty(B, K, dtype=torch.float32, device="cuda")
        b = torch.empty(D, dtype=torch.bfloat16, device="cuda")
        t = torch.empty(B, D, dtype=torch.bfloat16, device="cuda")
        loss, state = torch.ops.flexsae_b200.decoder_loss_fwd(kind, 0.0, idx, w, v, b, t)
        assert loss.shape == () and loss.dtype == torch.float32 and loss.device.type == "cuda"
        seg = lib.flexsae_choose_segments(kind, B, K, F, D, nv.BF16)
        assert state.numel() * 4 == lib.flexsae_state_bytes(kind, B, K, D, seg)
        assert compile_ops._segments_of_state(kind, state, idx, w) == (seg if kind == nv.HIER else 1)
        dw, dv, db = torch.ops.flexsae_b200.decoder_loss_bwd(kind, 0.0, idx, w, v, b, state, loss)
        assert dw.shape == w.shape and dw.dtype == w.dtype
        assert dv.shape == v.shape and dv.dtype == v.dtype
        assert db.shape == b.shape and db.dtype == b.dtype


@pytest.mark.gpu
@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])     # the reference's example compiles with the default backend (example.py:15)
@pytest.mark.parametrize("kind", ["topk", "hier"])
def test_fullgraph_compile_matches_eager(kind, backend):
    w = Workload("cmp", B=96, K=32, F=1024, D=768, weight_dtype="bfloat16", indices="distinct", sort_vals=True,
                 normalise_weight=True, seed=61)
    x = make_inputs(w, "cuda")
    fn = fx.triton_hierarchical_sae_loss if kind == "hier" else fx.triton_topk_sae_loss

    def step(i, wt, v, b, t):
        return fn(i, wt, v, b, t) * 3.0

    outs = []
    for f in (step, torch.compile(step, fullgraph=True, backend=backend)):
        wt = x["weight"].clone().requires_grad_(True)
        v = x["vals"].clone().requires_grad_(True)
        b = x["bias"].clone().requires_grad_(True)
        try:
            loss = f(x["indices"], wt, v, b, x["target"])
            loss.backward()
        except torch._inductor.exc.InductorError as e:        # no working Triton / C++ toolchain for inductor's own code
            pytest.skip(f"inductor cannot generate code on this machine: {str(e)[:200]}")
        outs.append((loss.detach(), wt.grad, v.grad, b.grad))
    (l0, w0, v0, b0), (l1, w1, v1, b1) = outs
    assert torch.equal(l0, l1) and torch.equal(v0, v1) and torch.equal(b0, b1)   # fixed-order sums
    torch.testing.assert_close(w0, w1, rtol=2e-2, atol=1e-8)   # atomic dweight: order of fp32 adds varies run to run
