"""CPU oracle for the two sparse-autoencoder decoder losses.  TEST INFRASTRUCTURE ONLY.

This module restates, in float64 numpy with hand-derived gradients, what the reference's torch
losses compute:

* ``topk_sae_loss``          torch-ext/flex_sae/topk_kernels.py:226-237
* ``hierarchical_sae_loss``  torch-ext/flex_sae/hierarchical_kernels.py:312-323

and what autograd returns for them (the gradient contract of
torch-ext/flex_sae/hierarchical_kernels.py:288-299 and topk_kernels.py:200-210: gradients for
weight, vals and bias, none for indices and target, everything scaled by the upstream scalar).

It is a checker, never a product path: only the tests, the smoke entry and the CPU-baseline leg
of the benchmark may import it.  Nothing in ``flexsae_b200`` does.

Parity is pinned: ``tests/golden/*.npz`` hold outputs of the reference's own functions (run on
CPU through torch autograd by ``tests/golden/make_golden.py``) and ``tests/test_oracle.py``
checks this restatement against every one of them.

The reference upcasts every operand to float32 before any arithmetic
(hierarchical_kernels.py:319-321), so its result is the float32 evaluation of an exact
real-valued formula of the stored (possibly 16-bit) inputs; float64 here is that formula with
less rounding, which is what a float32-accumulating kernel should be compared with.
"""
from __future__ import annotations

from typing import Dict

import numpy as np


def _as64(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.float64))


def topk_loss_and_grads(indices, weight, vals, bias, target, grad_out: float = 1.0,
                        norm_rows: int | None = None) -> Dict[str, np.ndarray]:
    """loss = mean_{b,d} (bias + sum_k vals[b,k] * weight[indices[b,k]] - target[b])^2.

    Follows topk_kernels.py:233-236.  ``norm_rows`` replaces B in the mean's denominator
    (a batch shard of a larger batch); the default is the number of rows given.
    """
    idx = np.asarray(indices, dtype=np.int64)
    W, v, b0, t = _as64(weight), _as64(vals), _as64(bias), _as64(target)
    B, K = idx.shape
    D = W.shape[1]
    denom = float((B if norm_rows is None else norm_rows) * D)
    dW = np.zeros_like(W)
    dv = np.zeros_like(v)
    db = np.zeros_like(b0)
    total = 0.0
    for b in range(B):
        rows = W[idx[b]]                                  # [K, D]  (topk_kernels.py:233)
        recon = b0 + (rows * v[b][:, None]).sum(axis=0)   # (topk_kernels.py:234)
        diff = recon - t[b]                               # (topk_kernels.py:235)
        total += float(np.dot(diff, diff))
        g = (2.0 * grad_out / denom) * diff               # d loss / d recon
        db += g
        dv[b] = rows @ g
        np.add.at(dW, idx[b], v[b][:, None] * g[None, :])
    return {"loss": np.float64(total / denom), "dweight": dW, "dvals": dv, "dbias": db}


def hier_loss_and_grads(indices, weight, vals, bias, target, grad_out: float = 1.0,
                        norm_rows: int | None = None) -> Dict[str, np.ndarray]:
    """loss = mean_{b,k,d} (bias + sum_{i<=k} vals[b,i] * weight[indices[b,i]] - target[b])^2.

    Follows hierarchical_kernels.py:319-322: the k-th reconstruction is the running prefix
    (``cumsum(dim=1)``) and every prefix is penalised.  The gradient with respect to the k-th
    gathered row is vals[b,k] times the SUFFIX sum over j >= k of the per-prefix residual
    gradients, which is also what the reference's fused backward walks
    (hierarchical_kernels.py:147-173).
    """
    idx = np.asarray(indices, dtype=np.int64)
    W, v, b0, t = _as64(weight), _as64(vals), _as64(bias), _as64(target)
    B, K = idx.shape
    D = W.shape[1]
    denom = float((B if norm_rows is None else norm_rows) * K * D)
    dW = np.zeros_like(W)
    dv = np.zeros_like(v)
    db = np.zeros_like(b0)
    total = 0.0
    for b in range(B):
        rows = W[idx[b]]                                            # [K, D]
        recon = b0 + np.cumsum(rows * v[b][:, None], axis=0)        # [K, D] prefixes
        diff = recon - t[b]
        total += float(np.sum(diff * diff))
        g = (2.0 * grad_out / denom) * diff                         # per-prefix residual grads
        suffix = np.cumsum(g[::-1], axis=0)[::-1]                   # S_k = sum_{j>=k} g_j
        db += suffix[0]
        dv[b] = np.einsum("kd,kd->k", rows, suffix)
        np.add.at(dW, idx[b], v[b][:, None] * suffix)
    return {"loss": np.float64(total / denom), "dweight": dW, "dvals": dv, "dbias": db}


LOSSES = {"topk": topk_loss_and_grads, "hier": hier_loss_and_grads}


def digest(dweight: np.ndarray, n_rows: int = 4) -> Dict[str, np.ndarray]:
    """Small fingerprints of a dense [F, D] gradient, used where a golden file cannot afford to
    store the whole table: its projections on two fixed pseudo-random vectors (any error that is
    not orthogonal to both shows up) and its first ``n_rows`` non-zero rows."""
    F, D = dweight.shape
    u = np.cos(1.0 + 0.61803398875 * np.arange(D, dtype=np.float64) ** 1.5)
    w = np.cos(2.0 + 0.41421356237 * np.arange(F, dtype=np.float64) ** 1.5)
    touched = np.flatnonzero(np.abs(dweight).sum(axis=1) > 0)[:n_rows]
    return {
        "dweight_rowproj": dweight.astype(np.float64) @ u,      # [F]
        "dweight_colproj": w @ dweight.astype(np.float64),      # [D]
        "dweight_rows_idx": touched.astype(np.int64),
        "dweight_rows": dweight[touched].astype(np.float64),
    }


def topk_select(acts, k: int, relu: bool = True):
    """The producer step in front of the losses: per row the ``k`` largest activations, values in
    descending order, equal values by ascending index (what ``torch.topk(acts, k, sorted=True)``
    returns up to the order of ties, which torch leaves open; like torch.topk, a NaN counts as larger
    than every number, and -0.0 equals +0.0).  The reference has no such function
    (its tests draw indices and vals at random, tests/test_all_kernels.py:20-33), so this one is
    pinned to torch.topk itself in ``tests/test_producer.py`` rather than to a golden file.
    Returns ``(indices int64 [B,k], vals float64 [B,k])``."""
    a = _as64(acts)
    nan = np.isnan(a)
    key = np.where(nan, np.inf, a) + 0.0                    # + 0.0 turns -0.0 into +0.0
    order = np.lexsort((-key, ~nan), axis=1)[:, :k]         # NaN first, then descending value, then ascending index
    vals = np.take_along_axis(a, order, axis=1)
    if relu:
        vals = np.maximum(vals, 0.0)
    return order.astype(np.int64), vals


def index_skew(indices, F: int, max_samples: int = 65536):
    """The statistic ``flexsae_index_skew`` computes: up to ``max_samples`` positions of the
    flattened ``indices[B,K]`` at an odd stride, counted per decoder row (entries outside [0, F) are
    left out); returns (largest count, positions taken).  The reference has no counterpart (its
    tile sizes are literals, torch-ext/flex_sae/hierarchical_kernels.py:263-267); this restates the
    library's own definition for the tests."""
    flat = np.asarray(indices).reshape(-1)
    n = flat.size
    stride = max(1, n // max_samples) | 1
    samples = min((n + stride - 1) // stride, max_samples)
    taken = flat[np.arange(samples, dtype=np.int64) * stride]
    taken = taken[(taken >= 0) & (taken < F)]
    hottest = int(np.bincount(taken, minlength=1).max()) if taken.size else 0
    return hottest, samples

