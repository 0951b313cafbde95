"""The producer step (top-K selection of encoder activations): oracle pinned to torch.topk on CPU,
argument checks of the C entry without a GPU, GPU parity against the oracle."""
import ctypes

import numpy as np
import pytest
import torch

from flexsae_b200 import _native as nv
from oracle import flexsae_oracle as orc


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_oracle_matches_torch_topk(seed):
    g = torch.Generator().manual_seed(seed)
    acts = torch.randn(7, 300, generator=g)
    idx, vals = orc.topk_select(acts.numpy(), 17, relu=False)
    tv, ti = torch.topk(acts, 17, dim=1, sorted=True)
    assert np.array_equal(idx, ti.numpy())                     # continuous values: no ties
    assert np.array_equal(vals.astype(np.float32), tv.numpy())


def test_oracle_orders_ties_by_index_and_clamps():
    acts = np.array([[0.5, -1.0, 0.5, 2.0, -1.0, 0.5]])
    idx, vals = orc.topk_select(acts, 5, relu=True)
    assert idx.tolist() == [[3, 0, 2, 5, 1]]
    assert vals.tolist() == [[2.0, 0.5, 0.5, 0.5, 0.0]]


def test_oracle_special_values_follow_torch_topk():
    nan, inf = float("nan"), float("inf")
    acts = np.array([[0.0, -0.0, nan, 1.0, inf, -inf, -0.0, 0.0, nan, -1.0]])
    idx, vals = orc.topk_select(acts, 8, relu=False)
    assert idx.tolist() == [[2, 8, 4, 3, 0, 1, 6, 7]]          # NaNs (by index), +inf, 1, then the four zeros by index
    tv, ti = torch.topk(torch.from_numpy(acts), 4, dim=1, sorted=True)
    assert sorted(ti[0, :2].tolist()) == [2, 8] and ti[0, 2:].tolist() == [4, 3]     # torch: NaN above +inf too
    assert np.isnan(vals[0, :2]).all() and vals[0, 2] == inf


def test_entry_rejects_bad_arguments_without_a_gpu():
    lib = nv.load()

    def call(acts=64, dt=nv.BF16, B=4, F=64, K=8, vals=64, vdt=nv.F32, idx=64):
        return lib.flexsae_topk_select(acts, dt, B, F, K, 1, vals, vdt, idx, None)

    assert call(dt=9) == -1 and b"dtype" in lib.flexsae_last_error()
    assert call(B=0) == -1 and call(K=0) == -1
    assert call(acts=None) == -1 and call(vals=None) == -1 and call(idx=None) == -1
    assert call(acts=72) == -1 and b"aligned" in lib.flexsae_last_error()
    assert call(F=60) == -3 and b"multiple of 8" in lib.flexsae_last_error()      # 16-bit rows: 8 per 16 bytes
    assert call(dt=nv.F32, F=62) == -3 and b"multiple of 4" in lib.flexsae_last_error()
    assert call(K=65) == -1 and b"exceeds" in lib.flexsae_last_error()
    assert call(F=4096, K=1025) == -3 and b"maximum" in lib.flexsae_last_error()


CASES = [  # B, F, K, dtype, kind of data
    (5, 64, 8, torch.float32, "normal"), (3, 4096, 128, torch.bfloat16, "normal"), (2, 65536, 128, torch.bfloat16, "normal"),
    (4, 1000, 33, torch.float32, "relu"), (4, 1024, 1024, torch.float16, "normal"), (3, 512, 100, torch.bfloat16, "ties"),
    (2, 131072, 64, torch.float32, "normal"), (1, 8, 1, torch.float16, "ties"), (6, 8192, 256, torch.float16, "relu"),
    (2, 8192, 16, torch.bfloat16, "const"), (2, 16384, 40, torch.float32, "ties"),      # candidate list overflows
    (2, 32768, 128, torch.float32, "normal"), (2, 131072, 64, torch.float16, "normal"),   # the largest rows whose per-vector maxima are kept
    (2, 262144, 32, torch.bfloat16, "normal"),                                            # longer: the row is read twice
    (3, 512, 12, torch.float32, "special"), (3, 1024, 20, torch.bfloat16, "special"), (2, 256, 9, torch.float16, "special"),
]


@pytest.mark.gpu
@pytest.mark.parametrize("B,F,K,dtype,data", CASES)
@pytest.mark.parametrize("relu", [False, True])
def test_gpu_selection_matches_oracle(B, F, K, dtype, data, relu):
    from flexsae_b200 import producer
    g = torch.Generator().manual_seed(B * 131 + F + K)
    if data == "const":
        acts = torch.full((B, F), 0.25).to(dtype)
    elif data == "ties":
        acts = torch.randint(-3, 4, (B, F), generator=g).to(dtype)
    elif data == "special":          # signed zeros, NaNs of both signs, infinities among small integers
        acts = torch.randint(-2, 2, (B, F), generator=g).to(torch.float32)
        acts[:, 5::37] = -0.0
        acts[:, 7::53] = float("nan")
        acts[:, 60::97] = -acts[:, 7::53][:, : acts[:, 60::97].shape[1]]     # NaN with the sign bit set
        acts[:, 11::101] = float("inf")
        acts[:, 13::89] = -float("inf")
        acts = acts.to(dtype)
    else:
        acts = torch.randn(B, F, generator=g).to(dtype)
        if data == "relu":
            acts = acts.clamp_min(0)
    want_idx, want_vals = orc.topk_select(acts.float().numpy(), K, relu)
    idx, vals = producer.select_topk(acts.cuda(), K, relu=relu, vals_dtype=torch.float32)
    assert idx.dtype == torch.int64 and idx.shape == (B, K) and vals.shape == (B, K)
    assert np.array_equal(idx.cpu().numpy(), want_idx)                      # bit-exact: integer work
    assert np.array_equal(vals.cpu().numpy(), want_vals.astype(np.float32), equal_nan=True)


@pytest.mark.gpu
def test_gpu_gradient_and_loss_chain():
    import flexsae_b200 as fx
    from flexsae_b200 import producer
    torch.manual_seed(0)
    B, Din, F, K, D = 32, 64, 512, 16, 64
    x = torch.randn(B, Din, device="cuda")
    w_enc = (torch.randn(F, Din, device="cuda") / 8).requires_grad_(True)
    b_enc = torch.zeros(F, device="cuda", requires_grad=True)
    w_dec = (torch.randn(F, D, device="cuda") / 8).requires_grad_(True)
    b_dec = torch.zeros(D, device="cuda", requires_grad=True)
    target = torch.randn(B, D, device="cuda")
    idx, vals = producer.encode_topk(x, w_enc, b_enc, K)
    loss = fx.triton_hierarchical_sae_loss(idx, w_dec, vals, b_dec, target)
    loss.backward()
    # the same graph with torch.topk and the eager loss
    w2, b2, wd2, bd2 = (t.detach().clone().requires_grad_(True) for t in (w_enc, b_enc, w_dec, b_dec))
    tv, ti = torch.topk(torch.nn.functional.linear(x, w2, b2), K, dim=1, sorted=True)
    loss2 = fx.hierarchical_sae_loss(ti, wd2, tv.clamp_min(0), bd2, target)
    loss2.backward()
    assert torch.equal(idx, ti)
    torch.testing.assert_close(loss, loss2, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(w_enc.grad, w2.grad, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(b_enc.grad, b2.grad, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(w_dec.grad, wd2.grad, rtol=1e-4, atol=1e-6)
