"""CPU: the seeded input generator and the byte model the benchmark reports against."""
import numpy as np
import torch

from flexsae_b200 import workloads as wl


def test_numpy_and_torch_generators_agree_bit_for_bit():
    a = wl.hash_bits_np(7, 3, 4096, 5)
    b = wl.hash_bits_torch(7, 3, 4096, "cpu", 5).numpy().view(np.uint64)
    assert np.array_equal(a, b)
    assert np.array_equal(wl.normal_np(1, 2, 10000), wl.normal_torch(1, 2, 10000, "cpu").numpy())
    n = wl.normal_np(1, 2, 200000)
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1.0) < 0.01


def test_shards_are_slices_of_the_whole_batch():
    w = wl.Workload("s", B=24, K=8, F=64, D=32, indices="distinct", sort_vals=True, seed=9)
    full = wl.make_inputs(w, "cpu")
    part = wl.make_inputs(w, "cpu", row0=8, rows=10)
    for k in ("indices", "vals", "target"):
        assert torch.equal(part[k], full[k][8:18])
    assert torch.equal(part["weight"], full["weight"]) and torch.equal(part["bias"], full["bias"])


def test_index_modes():
    for mode in ("distinct", "zipf"):
        w = wl.Workload("m", B=32, K=16, F=200, D=8, indices=mode, sort_vals=True, seed=3)
        x = wl.make_inputs(w, "cpu", with_weight=False)
        idx = x["indices"]
        assert idx.min() >= 0 and idx.max() < w.F
        assert all(len(set(r.tolist())) == w.K for r in idx)                  # K different features per row
        assert torch.all(x["vals"][:, :-1] >= x["vals"][:, 1:])               # sorted descending
    z = wl.make_inputs(wl.Workload("z", B=256, K=16, F=4096, D=8, indices="zipf", seed=4), "cpu", with_weight=False)
    assert (z["indices"] < 64).float().mean() > 0.5                           # a few hot decoder rows dominate
    d = wl.make_inputs(wl.Workload("d", B=64, K=64, F=16, D=8, indices="dup", seed=5), "cpu", with_weight=False)
    assert any(len(set(r.tolist())) < 64 for r in d["indices"])               # repeats allowed


def test_normalised_decoder_rows_have_unit_norm():
    w = wl.Workload("n", B=4, K=4, F=128, D=256, weight_dtype="bfloat16", normalise_weight=True, seed=6)
    x = wl.make_inputs(w, "cpu")
    assert torch.allclose(x["weight"].float().norm(dim=1), torch.ones(128), atol=5e-3)


def test_algorithmic_bytes_match_the_published_model():
    # time at 100 % of 6535.1 GB/s as tabulated for the benchmark set-ups
    for name, gb in (("c2", 7.03), ("c3_k32", 4.04), ("c3_k64", 6.46), ("c3_k128", 11.30), ("c4", 21.32)):
        assert abs(wl.algorithmic_bytes(wl.CONFIGS[name]) / 1e9 - gb) < 0.01, name
    assert abs(wl.algorithmic_bytes(wl.CONFIGS["c5"], rows=8192) / 1e9 - 40.2) < 0.1
