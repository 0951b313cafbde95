"""GPU parity of the fused CUDA losses (called through the C ABI by the autograd Functions)
against the oracle, the committed reference outputs and the reference's own parity matrix."""
import numpy as np
import pytest
import torch

import flexsae_b200 as fx
from flexsae_b200 import _native as nv
from flexsae_b200.workloads import CONFIGS, Workload, make_inputs
from oracle import flexsae_oracle as orc
from oracle import torch_reference as tref
from tests.helpers import REFERENCE_TOLS, golden_files, inputs_as_numpy, load_golden, rel_err

pytestmark = pytest.mark.gpu

FUSED = {"topk": fx.triton_topk_sae_loss, "hier": fx.triton_hierarchical_sae_loss}
# relative (max-abs-error / max-abs-value) bounds of a float32-accumulating kernel against float64
TIGHT = {"float32": 2e-5, "bfloat16": 6e-3, "float16": 8e-4}   # 16-bit: one rounding of the output


def run_fused(kind, x, dev="cuda", grad_out=None):
    idx = x["indices"].to(dev)
    w = x["weight"].to(dev).detach().clone().requires_grad_(True)
    v = x["vals"].to(dev).detach().clone().requires_grad_(True)
    b = x["bias"].to(dev).detach().clone().requires_grad_(True)
    t = x["target"].to(dev)
    loss = FUSED[kind](idx, w, v, b, t)
    go = x["grad_out"] if grad_out is None else grad_out
    loss.backward(go.to(dev))
    assert idx.grad is None and t.grad is None
    assert loss.dtype == torch.float32 and loss.dim() == 0
    assert w.grad.dtype == w.dtype and v.grad.dtype == v.dtype and b.grad.dtype == b.dtype
    return {"loss": float(loss), "dweight": w.grad.float().cpu().numpy(), "dvals": v.grad.float().cpu().numpy(),
            "dbias": b.grad.float().cpu().numpy()}


def assert_close_to_oracle(got, want, tol, loss_tol=1e-5):
    assert abs(got["loss"] - float(want["loss"])) <= loss_tol * abs(float(want["loss"]))
    for k in ("dvals", "dbias", "dweight"):
        assert rel_err(got[k], want[k]) < tol, k


@pytest.fixture(autouse=True)
def _auto_options():
    for name in ("lanes_fwd", "lanes_bwd", "segments"):
        nv.set_option(name, 0)
    nv.set_option("pipeline", 1)
    nv.set_option("direct_f32", 1)
    nv.set_option("ticket_order", 0)
    slabs, lag = nv.get_option("slabs"), nv.get_option("convert_lag")
    yield
    nv.set_option("slabs", slabs)
    nv.set_option("convert_lag", lag)
    fx.check_status()


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1][:-4])
def test_fused_matches_oracle_and_reference_outputs(path):
    w, kind, gold = load_golden(path)
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])
    # and the reference's own outputs, within the reference's own tolerances
    tols = REFERENCE_TOLS[w.weight_dtype]
    np.testing.assert_allclose(got["loss"], float(gold["loss"]), **tols)
    np.testing.assert_allclose(got["dvals"], gold["dvals"], **tols)
    np.testing.assert_allclose(got["dbias"], gold["dbias"], **tols)
    d = orc.digest(got["dweight"].astype(np.float64))
    assert np.array_equal(d["dweight_rows_idx"], gold["dweight_rows_idx"])
    np.testing.assert_allclose(d["dweight_rows"], gold["dweight_rows"], **tols)


@pytest.mark.parametrize("lanes", [8, 16, 32])
@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("name", ["ragged_rows_float32", "mixed_bf16w_f32v", "t16_16_64_512_float16"])
def test_every_lane_group_width(name, kind, lanes):
    path = [p for p in golden_files() if p.endswith(f"{name}__{kind}.npz")][0]
    w, kind, gold = load_golden(path)
    nv.set_option("lanes_fwd", lanes)
    nv.set_option("lanes_bwd", lanes)
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])


@pytest.mark.parametrize("segments", [1, 2, 3, 8])
@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("name", ["t16_64_128_1024_float32", "c1", "mixed_bf16w_f32v"])
def test_every_segment_count(name, kind, segments):
    path = [p for p in golden_files() if p.endswith(f"{name}__{kind}.npz")][0]
    w, kind, gold = load_golden(path)
    nv.set_option("segments", segments)
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])


@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("name", ["t16_64_128_1024_bfloat16", "c1", "ragged_rows_float32"])
def test_one_launch_per_piece_form(name, kind):
    """The multi-launch form of the atomic backward (the default is the single-launch pipeline)."""
    path = [p for p in golden_files() if p.endswith(f"{name}__{kind}.npz")][0]
    w, kind, gold = load_golden(path)
    nv.set_option("pipeline", 0)
    nv.set_option("lanes_bwd", 8)        # many column pieces
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])


@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("name", ["c1", "ragged_rows_float32", "t32_32_160_768_float32"])
def test_fp32_decoder_through_slab(name, kind):
    """fp32 decoders normally reduce straight into dweight; this is the slab + copy form."""
    path = [p for p in golden_files() if p.endswith(f"{name}__{kind}.npz")][0]
    w, kind, gold = load_golden(path)
    nv.set_option("direct_f32", 0)
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])


@pytest.mark.parametrize("slabs,lag", [(2, 1), (3, 1), (3, 2), (4, 1), (4, 3)])
@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("name", ["t16_64_128_1024_bfloat16", "mixed_bf16w_f32v", "t16_16_64_512_float16", "c1"])
def test_slab_rotation_and_conversion_lag(name, kind, slabs, lag):
    """The single-launch backward with 2..4 fp32 slabs in rotation and the conversion of a piece 1..3
    slots behind its accumulation."""
    path = [p for p in golden_files() if p.endswith(f"{name}__{kind}.npz")][0]
    w, kind, gold = load_golden(path)
    nv.set_option("slabs", slabs)
    nv.set_option("convert_lag", lag)
    nv.set_option("direct_f32", 0)       # fp32 decoders through the slabs too
    nv.set_option("lanes_bwd", 8)        # many column pieces
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])


@pytest.mark.parametrize("slabs,lag", [(2, 1), (3, 2)])
@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("name", ["t16_64_128_1024_bfloat16", "mixed_bf16w_f32v", "c1"])
def test_roles_by_starting_order(name, kind, slabs, lag):
    """Blocks of the single-launch backward take their roles from an atomic ticket, not from blockIdx.x."""
    path = [p for p in golden_files() if p.endswith(f"{name}__{kind}.npz")][0]
    w, kind, gold = load_golden(path)
    nv.set_option("ticket_order", 1)
    nv.set_option("slabs", slabs)
    nv.set_option("convert_lag", lag)
    nv.set_option("direct_f32", 0)
    nv.set_option("lanes_bwd", 8)
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])


EDGE = [
    Workload("k5", B=9, K=5, F=50, D=264, weight_dtype="bfloat16", indices="dup", seed=21),       # K, D odd-shaped
    Workload("k13", B=33, K=13, F=77, D=1000, indices="dup", seed=22),
    Workload("k300", B=5, K=300, F=64, D=512, indices="dup", seed=23),                           # K > F
    Workload("b1", B=1, K=2, F=3, D=4, indices="dup", seed=24),
    Workload("wide", B=4, K=8, F=32, D=8200, weight_dtype="float16", vals_dtype="float16", indices="distinct", seed=25),
]


@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("w", EDGE, ids=lambda w: w.name)
def test_edge_shapes(w, kind):
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])


# ---- the reference's own parity matrix (tests/test_setup.py:5-41, tests/test_all_kernels.py:20-50)
REF_PARAMS = [
    (16, 16, 64, 512), (16, 32, 96, 768), (16, 64, 128, 1024), (32, 16, 128, 512), (32, 32, 160, 768),
    (32, 64, 192, 1024), (48, 32, 176, 1024), (48, 64, 224, 1280), (64, 16, 192, 768), (64, 32, 224, 1024),
    (64, 128, 256, 2048), (80, 32, 240, 1280), (80, 64, 256, 1536), (96, 32, 256, 1536), (96, 64, 288, 2048),
    (96, 128, 320, 3072), (112, 64, 320, 2048), (112, 128, 352, 2560), (128, 32, 256, 1024), (128, 64, 320, 1536),
    (128, 128, 384, 3072), (160, 64, 320, 1536), (160, 128, 384, 2560), (192, 64, 384, 2048), (192, 128, 448, 3072),
    (192, 256, 512, 4096),
]


@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("B,K,F,D", REF_PARAMS)
def test_reference_parity_matrix(B, K, F, D, dtype, kind):
    """Same protocol as the reference's run_funcs: one dtype for every tensor, repeated indices,
    unsorted vals, random upstream scalar, the reference's tolerances, torch reference on the GPU."""
    w = Workload("m", B=B, K=K, F=F, D=D, weight_dtype=dtype, vals_dtype=dtype, indices="dup", seed=1234)
    x = make_inputs(w, "cuda")
    got = run_fused(kind, x)
    ref = tref.chunked_loss_and_grads(kind, x["indices"], x["weight"], x["vals"], x["bias"], x["target"],
                                      grad_out=float(x["grad_out"]), chunk_rows=B)
    tols = REFERENCE_TOLS[dtype]
    np.testing.assert_allclose(got["loss"], ref["loss"], **tols)
    np.testing.assert_allclose(got["dvals"], ref["dvals"].float().cpu().numpy(), **tols)
    np.testing.assert_allclose(got["dweight"], ref["dweight"].float().cpu().numpy(), **tols)
    np.testing.assert_allclose(got["dbias"], ref["dbias"].float().cpu().numpy(), **tols)
    # and, scale-free, against the float32-upcast reference (what fp32 accumulation should match)
    up = tref.chunked_loss_and_grads(kind, x["indices"], x["weight"], x["vals"], x["bias"], x["target"],
                                     grad_out=float(x["grad_out"]), chunk_rows=B, upcast=True)
    for k in ("dvals", "dweight", "dbias"):
        assert rel_err(got[k], up[k].float().cpu().numpy()) < max(TIGHT[dtype], 1e-4), k


def _compare_with_torch_reference_on_gpu(w: Workload, kind: str, tol: float, loss_tol: float, chunk_rows=256):
    x = make_inputs(w, "cuda")
    # a large upstream gradient undoes the 2/(B*K*D) factor, so absolute tolerances cannot pass vacuously
    go = torch.tensor(float(w.B * w.D) / 2.0 * (w.K if kind == "hier" else 1.0) * 0.37)
    got = run_fused(kind, x, grad_out=go)
    ref = tref.chunked_loss_and_grads(kind, x["indices"], x["weight"], x["vals"], x["bias"], x["target"],
                                      grad_out=float(go), chunk_rows=chunk_rows, upcast=True)
    assert abs(got["loss"] - ref["loss"]) <= loss_tol * abs(ref["loss"])
    for k in ("dvals", "dbias", "dweight"):
        want = ref[k].float().cpu().numpy()
        assert rel_err(got[k], want) < tol, k
    return got, ref


@pytest.mark.parametrize("kind", ["topk", "hier"])
def test_config1_fp32_tolerances(kind):
    """B=64 K=32 F=4096 D=256 fp32: loss within 1e-5 relative, gradients rtol 1e-4 / atol 1e-6."""
    w = CONFIGS["c1"]
    x = make_inputs(w, "cpu")
    for go in (x["grad_out"], torch.tensor(-3.0e5)):
        got = run_fused(kind, x, grad_out=go)
        want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(go))
        assert abs(got["loss"] - want["loss"]) <= 1e-5 * abs(want["loss"])
        for k in ("dvals", "dbias", "dweight"):
            if abs(float(go)) < 10:      # natural gradient scale: the stated elementwise tolerances
                np.testing.assert_allclose(got[k], want[k], rtol=1e-4, atol=1e-6)
            assert rel_err(got[k], want[k]) < 2e-5   # scale-free, bites at any gradient magnitude


@pytest.mark.parametrize("kind", ["topk", "hier"])
def test_config2_fp32_full_size(kind):
    """B=2048 K=256 F=131072 D=1024 fp32 (the reference benchmark script's shape)."""
    _compare_with_torch_reference_on_gpu(CONFIGS["c2"], kind, tol=1e-4, loss_tol=1e-5, chunk_rows=128)


@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("name", ["c3_k32", "c3_k64", "c3_k128"])
def test_config3_bf16_full_size(name, kind):
    """F=65536 D=2304 B=4096 bf16 storage, fp32 vals and accumulation: within 1e-2 relative."""
    _compare_with_torch_reference_on_gpu(CONFIGS[name], kind, tol=1e-2, loss_tol=1e-5, chunk_rows=128)


@pytest.mark.parametrize("mode", ["atomic", "deterministic"])
def test_config4_zipf_full_size_both_dweight_modes(mode):
    """F=65536 D=2304 K=64 B=16384 bf16, Zipf(1.1) indices: the hottest decoder rows receive thousands of
    contributions each, the stress case of the scatter-add and of the ordered sums' item tree."""
    fx.config.dweight_mode = mode
    try:
        got, _ = _compare_with_torch_reference_on_gpu(CONFIGS["c4"], "hier", tol=1e-2, loss_tol=1e-5, chunk_rows=128)
        if mode == "deterministic":        # bit for bit, run to run, at full size too
            x = make_inputs(CONFIGS["c4"], "cuda")
            go = torch.tensor(float(CONFIGS["c4"].B * CONFIGS["c4"].D) / 2.0 * CONFIGS["c4"].K * 0.37)
            again = run_fused("hier", x, grad_out=go)
            for k in ("dweight", "dvals", "dbias"):
                assert np.array_equal(got[k], again[k]), k
            assert got["loss"] == again["loss"]
    finally:
        fx.config.dweight_mode = "atomic"


def test_config5_one_gpu_shard_full_size():
    """F=131072 D=4096 K=128 bf16 with the 8192 rows one GPU of eight holds of the 65536-row batch:
    the widest decoder of the five set-ups (8 lanes per row, 64 column pieces)."""
    _compare_with_torch_reference_on_gpu(CONFIGS["c5"].replace(B=8192), "hier", tol=1e-2, loss_tol=1e-5, chunk_rows=64)


def test_out_of_range_index_is_reported_not_dereferenced():
    w = Workload("bad", B=8, K=4, F=16, D=256, indices="dup", seed=31)
    x = make_inputs(w, "cuda")
    x["indices"][3, 2] = 16
    x["indices"][5, 0] = -7
    loss = fx.triton_hierarchical_sae_loss(x["indices"], x["weight"], x["vals"], x["bias"], x["target"])
    torch.cuda.synchronize()
    with pytest.raises(IndexError):
        fx.check_status()
    assert torch.isfinite(loss)


def test_no_grad_and_non_contiguous_inputs():
    w = Workload("nc", B=24, K=8, F=64, D=512, indices="dup", seed=32)
    x = make_inputs(w, "cuda")
    wide = torch.zeros(w.F, 2 * w.D, device="cuda")
    wide[:, ::2] = x["weight"]
    with torch.no_grad():
        a = fx.triton_topk_sae_loss(x["indices"], wide[:, ::2], x["vals"], x["bias"], x["target"])
        b = fx.triton_topk_sae_loss(x["indices"], x["weight"], x["vals"], x["bias"], x["target"])
    assert a.requires_grad is False and float(a) == float(b)


def test_loss_is_run_to_run_reproducible():
    w = CONFIGS["c3_k32"].replace(B=512, F=8192)
    x = make_inputs(w, "cuda")
    vals = [float(fx.triton_hierarchical_sae_loss(x["indices"], x["weight"], x["vals"], x["bias"], x["target"]))
            for _ in range(3)]
    assert vals[0] == vals[1] == vals[2]


def test_rejected_arguments():
    w = Workload("rej", B=4, K=4, F=16, D=256, indices="dup", seed=33)
    x = make_inputs(w, "cuda")
    with pytest.raises(TypeError):
        fx.triton_topk_sae_loss(x["indices"].int(), x["weight"], x["vals"], x["bias"], x["target"])
    with pytest.raises(ValueError):
        fx.triton_topk_sae_loss(x["indices"], x["weight"], x["vals"][:, :2], x["bias"], x["target"])
    with pytest.raises(RuntimeError):
        fx.triton_topk_sae_loss(x["indices"].cpu(), x["weight"].cpu(), x["vals"].cpu(), x["bias"].cpu(), x["target"].cpu())
    with pytest.raises(nv.FlexSaeNativeError):     # D not a multiple of the 16-byte row piece
        fx.triton_topk_sae_loss(x["indices"], x["weight"][:, :254].contiguous(), x["vals"], x["bias"][:254].contiguous(),
                                x["target"][:, :254].contiguous())


# ---- deterministic dweight mode -----------------------------------------------------------------------
@pytest.fixture
def deterministic_mode():
    fx.config.dweight_mode = "deterministic"
    yield
    fx.config.dweight_mode = "atomic"


@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1][:-4])
def test_deterministic_mode_matches_oracle(path, deterministic_mode):
    w, kind, gold = load_golden(path)
    x = make_inputs(w, "cpu")
    got = run_fused(kind, x)
    want = orc.LOSSES[kind](**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert_close_to_oracle(got, want, TIGHT[w.weight_dtype])


DET_CASES = [
    Workload("det_uniform", B=512, K=64, F=4096, D=768, weight_dtype="bfloat16", indices="distinct", sort_vals=True,
             normalise_weight=True, seed=51),
    # a few decoder rows receive thousands of contributions: segments far longer than one 32-slot item
    Workload("det_zipf", B=2048, K=32, F=512, D=512, weight_dtype="bfloat16", indices="zipf", sort_vals=True,
             normalise_weight=True, seed=52),
    Workload("det_one_row_table", B=300, K=8, F=1, D=256, indices="dup", seed=53),     # every pair hits row 0
    Workload("det_f32_wide_table", B=64, K=16, F=70000, D=128, indices="dup", seed=54),  # three radix passes not needed, 17 bits
]


@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("w", DET_CASES, ids=lambda w: w.name)
def test_deterministic_mode_is_bitwise_reproducible_and_right(w, kind, deterministic_mode):
    x = make_inputs(w, "cuda")
    runs = []
    for _ in range(3):
        wt = x["weight"].clone().requires_grad_(True)
        v = x["vals"].clone().requires_grad_(True)
        b = x["bias"].clone().requires_grad_(True)
        loss = FUSED[kind](x["indices"], wt, v, b, x["target"])
        loss.backward(x["grad_out"])
        runs.append((loss.detach().clone(), wt.grad.clone(), v.grad.clone(), b.grad.clone()))
    for r in runs[1:]:
        for a, b_ in zip(runs[0], r):
            assert torch.equal(a, b_)            # bit for bit, run to run
    ref = tref.chunked_loss_and_grads(kind, x["indices"], x["weight"], x["vals"], x["bias"], x["target"],
                                      grad_out=float(x["grad_out"]), chunk_rows=256, upcast=True)
    assert abs(float(runs[0][0]) - ref["loss"]) <= 1e-5 * abs(ref["loss"])
    for got, name in zip(runs[0][1:], ("dweight", "dvals", "dbias")):
        assert rel_err(got.float().cpu().numpy(), ref[name].float().cpu().numpy()) < TIGHT[w.weight_dtype], name


SORT_CASES = DET_CASES + [
    Workload("sort_zipf_wide", B=4096, K=64, F=65536, D=8, weight_dtype="bfloat16", indices="zipf", seed=55),
    Workload("sort_tiny", B=1, K=1, F=1, D=8, indices="dup", seed=56),
]


@pytest.mark.parametrize("w", SORT_CASES, ids=lambda w: w.name)
def test_sort_tables_match_stable_argsort(w):
    """Integer work of the deterministic mode, bit for bit against numpy's stable argsort: the
    permutation, its inverse, the segment starts (the reference's emb_begin_pos,
    topk_kernels.py:152) and the 32-slot item table."""
    import ctypes

    lib = nv.load()
    idx = make_inputs(w, "cuda", with_weight=False)["indices"].reshape(-1).contiguous()
    n, F = idx.numel(), w.F
    if n > 8:                               # out-of-range entries count as decoder row 0, as in the losses
        idx[3], idx[n - 2] = F, -5
    ws = torch.empty(lib.flexsae_sort_workspace_bytes(n, F), dtype=torch.uint8, device="cuda")
    order, slot_of = (torch.full((n,), -1, dtype=torch.int32, device="cuda") for _ in range(2))
    seg_begin, item_begin = (torch.full((F + 1,), -1, dtype=torch.int32, device="cuda") for _ in range(2))
    rc = lib.flexsae_sort_by_decoder_row(idx.data_ptr(), n, F, ws.data_ptr(), ws.numel(), order.data_ptr(), slot_of.data_ptr(),
                                         seg_begin.data_ptr(), item_begin.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.flexsae_last_error()
    keys = idx.cpu().numpy().copy()
    keys[(keys < 0) | (keys >= F)] = 0
    want_order = np.argsort(keys, kind="stable")
    assert np.array_equal(order.cpu().numpy(), want_order)
    want_slot = np.empty(n, dtype=np.int64)
    want_slot[want_order] = np.arange(n)
    assert np.array_equal(slot_of.cpu().numpy(), want_slot)
    want_seg = np.searchsorted(keys[want_order], np.arange(F + 1), side="left")
    assert np.array_equal(seg_begin.cpu().numpy(), want_seg)
    items = np.maximum(1, (np.diff(want_seg) + 31) // 32)
    assert np.array_equal(item_begin.cpu().numpy(), np.concatenate([[0], np.cumsum(items)]))


def _index_skew_on_gpu(idx, F):
    lib = nv.load()
    B, K = idx.shape
    ws = torch.empty(lib.flexsae_index_skew_workspace_bytes(F), dtype=torch.uint8, device="cuda")
    res = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    rc = lib.flexsae_index_skew(idx.data_ptr(), B, K, F, ws.data_ptr(), ws.numel(), res.data_ptr(),
                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.flexsae_last_error()
    return tuple(int(v) for v in res.cpu())


@pytest.mark.parametrize("w", [CONFIGS["c1"], CONFIGS["c3_k128"], CONFIGS["c4"], CONFIGS["c3_k32"].replace(B=3, K=5, F=11),
                               CONFIGS["c5"].replace(B=4096)], ids=lambda w: f"{w.name}_{w.B}")
def test_index_skew_matches_oracle(w):
    """The hottest decoder row's count over the sampled positions, bit for bit against numpy; out-of-
    range entries are left out; config 4's Zipf indices are far above the wide-piece threshold,
    uniform ones far below."""
    idx = make_inputs(w, "cuda", with_weight=False)["indices"].contiguous()
    if idx.numel() > 8:
        idx.view(-1)[0], idx.view(-1)[-1] = w.F, -1
    got = _index_skew_on_gpu(idx, w.F)
    assert got == orc.index_skew(idx.cpu().numpy(), w.F)
    share = got[0] / got[1]
    if w.name == "c4":
        assert share > 2 * fx.config.skew_threshold
    if w.name == "c3_k128":
        assert share < fx.config.skew_threshold / 16         # about 8 of 65536 samples


def test_piece_width_follows_the_index_skew():
    """Zipf indices: the first backward measures, the following ones take the wide pieces; uniform
    indices on the same decoder shape turn them off again; results agree with the fixed widths."""
    from flexsae_b200 import losses

    w = CONFIGS["c4"].replace(B=2048)
    watch_key = (torch.cuda.current_device(), w.F)
    losses._skew_watches.pop(watch_key, None)
    x = make_inputs(w, "cuda")
    interval = fx.config.skew_interval
    fx.config.skew_interval = 1
    try:
        first = run_fused("hier", x)
        torch.cuda.synchronize()
        second = run_fused("hier", x)                   # reads the first measurement
        watch = losses._skew_watches[watch_key]
        assert watch.share > fx.config.skew_threshold
        fx.config.dweight_mode = "atomic_wide"
        wide = run_fused("hier", x)
        fx.config.dweight_mode = "atomic"
        for k in ("dweight", "dvals", "dbias"):
            assert rel_err(second[k], first[k]) < 6e-3, k
            assert rel_err(second[k], wide[k]) < 6e-3, k
        assert np.array_equal(second["dvals"], wide["dvals"]) or rel_err(second["dvals"], wide["dvals"]) < 1e-6
        u = make_inputs(w.replace(indices="distinct"), "cuda")
        run_fused("hier", u)
        torch.cuda.synchronize()
        run_fused("hier", u)
        assert watch.share < fx.config.skew_threshold
    finally:
        fx.config.skew_interval = interval
        fx.config.dweight_mode = "atomic"


def test_atomic_and_deterministic_modes_agree():
    w = CONFIGS["c3_k32"].replace(B=1024, F=16384)
    x = make_inputs(w, "cuda")
    out = {}
    for mode in ("atomic", "deterministic"):
        fx.config.dweight_mode = mode
        try:
            out[mode] = run_fused("hier", x)
        finally:
            fx.config.dweight_mode = "atomic"
    assert out["atomic"]["loss"] == out["deterministic"]["loss"]
    assert np.array_equal(out["atomic"]["dvals"], out["deterministic"]["dvals"])
    assert rel_err(out["atomic"]["dweight"], out["deterministic"]["dweight"]) < 6e-3   # one bf16 rounding apart at most


def test_calls_on_two_streams_do_not_share_scratch():
    """Two backward passes enqueued on different streams may overlap on the GPU: each stream has
    its own workspace, so both must give what they give alone."""
    ws = [CONFIGS["c3_k32"].replace(B=1024, F=8192, seed=71), CONFIGS["c3_k32"].replace(B=1024, F=8192, seed=72)]
    xs = [make_inputs(w, "cuda") for w in ws]
    alone = [run_fused("hier", x) for x in xs]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    params = []
    torch.cuda.synchronize()
    for x, st in zip(xs, streams):
        with torch.cuda.stream(st):
            wt = x["weight"].detach().clone().requires_grad_(True)
            v = x["vals"].detach().clone().requires_grad_(True)
            b = x["bias"].detach().clone().requires_grad_(True)
            loss = fx.triton_hierarchical_sae_loss(x["indices"], wt, v, b, x["target"])
            loss.backward(x["grad_out"])
            params.append((loss, wt, v, b))
    torch.cuda.synchronize()
    for (loss, wt, v, b), ref in zip(params, alone):
        assert float(loss) == ref["loss"]
        assert np.array_equal(v.grad.float().cpu().numpy(), ref["dvals"])
        assert rel_err(wt.grad.float().cpu().numpy(), ref["dweight"]) < 6e-3
        assert np.array_equal(b.grad.float().cpu().numpy(), ref["dbias"])
