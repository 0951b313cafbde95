"""Shared helpers of the parity tests: golden-file loading and gradient comparison."""
from __future__ import annotations

import glob
import json
import os
from typing import Dict

import numpy as np
import torch

from flexsae_b200.workloads import Workload, make_inputs

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(path: str):
    z = np.load(path, allow_pickle=False)
    w = Workload(**json.loads(str(z["workload"])))
    return w, str(z["kind"]), {k: z[k] for k in z.files if k not in ("workload", "kind")}


def inputs_as_numpy(x: Dict[str, torch.Tensor]) -> Dict[str, np.ndarray]:
    """Upcasts the (possibly 16-bit) tensors exactly to float64 arrays for the numpy oracle."""
    out = {"indices": x["indices"].cpu().numpy()}
    for k in ("weight", "vals", "bias", "target"):
        out[k] = x[k].detach().cpu().double().numpy()
    return out


# tolerances of the reference's own parity harness (tests/test_setup.py:35-39)
REFERENCE_TOLS = {
    "float32": dict(atol=1e-4, rtol=1e-3),
    "bfloat16": dict(atol=1e-2, rtol=1e-2),
    "float16": dict(atol=1e-3, rtol=1e-3),
}


def rel_err(a, b) -> float:
    """max |a-b| / max |b|: a scale-free error that cannot pass vacuously on tiny gradients."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = float(np.max(np.abs(b)))
    return float(np.max(np.abs(a - b))) / (den if den > 0 else 1.0)
