"""The golden parity cases: small workloads whose reference outputs are committed as .npz.

Shapes follow the reference's own parity matrix (tests/test_setup.py:5-32 and its three
dtypes, tests/test_setup.py:35-41, with vals in the test dtype and repeated indices as in
tests/test_all_kernels.py:26-31) plus the CPU-runnable benchmark set-up and the edge cases the
reference's matrix leaves out: K = 1, one batch row full of repeats, 16-bit decoder with
float32 vals, a skewed index distribution.
"""
from flexsae_b200.workloads import CONFIGS, Workload

GOLDEN_CASES = [CONFIGS["c1"]]
for _dt in ("float32", "bfloat16", "float16"):
    for (_B, _K, _F, _D) in [(16, 16, 64, 512), (32, 32, 160, 768), (16, 64, 128, 1024)]:
        GOLDEN_CASES.append(Workload(f"t{_B}_{_K}_{_F}_{_D}_{_dt}", B=_B, K=_K, F=_F, D=_D,
                                     weight_dtype=_dt, vals_dtype=_dt, indices="dup", seed=1234))
GOLDEN_CASES += [
    Workload("k1_float32", B=8, K=1, F=32, D=256, indices="dup", seed=11),
    Workload("onerow_repeats_float32", B=1, K=64, F=16, D=256, indices="dup", seed=12),
    Workload("mixed_bf16w_f32v", B=32, K=32, F=512, D=768, weight_dtype="bfloat16",
             indices="distinct", sort_vals=True, normalise_weight=True, seed=13),
    Workload("zipf_bf16", B=64, K=16, F=256, D=512, weight_dtype="bfloat16", indices="zipf",
             sort_vals=True, normalise_weight=True, seed=14),
    Workload("ragged_rows_float32", B=13, K=8, F=40, D=384, indices="dup", seed=15),
]
KINDS = ("topk", "hier")
FULL_DWEIGHT_MAX_ELEMS = 40000
