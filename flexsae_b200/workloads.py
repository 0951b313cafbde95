"""Seeded synthetic inputs for the decoder-loss hot path.

The reference draws its inputs with ``torch.randn`` / ``torch.randint``
(tests/test_all_kernels.py:24-31, example.py:45-51).  Those streams differ between devices
and torch versions, so this module uses a counter-based generator instead: every element is a
pure function of ``(seed, stream, position)`` built from the splitmix64 finaliser.  The same
tensors can therefore be produced with numpy on a CPU box and with torch integer ops on the
GPU, bit for bit, which is what lets committed golden outputs be checked on another machine.

Only shapes, dtypes and value distributions follow the reference's benchmark set-ups:

* ``dup``      indices = uniform draws from [0, F) with repeats (tests/test_all_kernels.py:26)
* ``distinct`` K different features per row, uniform
* ``zipf``     K different features per row, drawn without replacement from Zipf(s) over F
               (Gumbel top-K on ``-s*log(rank)``), so a few decoder rows are hit by most rows
* vals = |N(0,1)|, optionally sorted descending per row
* weight ~ N(0,1), optionally scaled by 1/sqrt(D) and row-normalised; bias, target ~ N(0,1)
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, Optional

import numpy as np
import torch

_MASK64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_C1 = 0xBF58476D1CE4E5B9
_C2 = 0x94D049BB133111EB


def _s64(x: int) -> int:
    """Python int (mod 2**64) -> the int64 with the same bit pattern."""
    x &= _MASK64
    return x - (1 << 64) if x >= (1 << 63) else x


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical shift right of an int64 tensor holding uint64 bit patterns."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def _mix_torch(x: torch.Tensor) -> torch.Tensor:
    x = (x ^ _lsr(x, 30)) * _s64(_C1)
    x = (x ^ _lsr(x, 27)) * _s64(_C2)
    return x ^ _lsr(x, 31)


def _mix_np(x: np.ndarray) -> np.ndarray:
    x = (x ^ (x >> np.uint64(30))) * np.uint64(_C1)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(_C2)
    return x ^ (x >> np.uint64(31))


def _key(seed: int, stream: int) -> int:
    return ((seed * 0xD1342543DE82EF95 + stream * 0xA0761D6478BD642F + 0x2545F4914F6CDD1D) & _MASK64)


def hash_bits_torch(seed: int, stream: int, n: int, device, offset: int = 0) -> torch.Tensor:
    """n 64-bit hashes (as int64 bit patterns) of positions offset..offset+n-1."""
    ctr = torch.arange(offset, offset + n, dtype=torch.int64, device=device)
    return _mix_torch(_mix_torch(ctr * _s64(_GOLDEN) + _s64(_key(seed, stream))))


def hash_bits_np(seed: int, stream: int, n: int, offset: int = 0) -> np.ndarray:
    with np.errstate(over="ignore"):
        ctr = np.arange(offset, offset + n, dtype=np.uint64)
        return _mix_np(_mix_np(ctr * np.uint64(_GOLDEN) + np.uint64(_key(seed, stream))))


def uniform_torch(seed: int, stream: int, n: int, device, offset: int = 0) -> torch.Tensor:
    """float64 uniforms in (0, 1): (top 53 bits + 0.5) / 2**53."""
    h = hash_bits_torch(seed, stream, n, device, offset)
    return (_lsr(h, 11).to(torch.float64) + 0.5) * (1.0 / (1 << 53))


def uniform_np(seed: int, stream: int, n: int, offset: int = 0) -> np.ndarray:
    h = hash_bits_np(seed, stream, n, offset)
    return ((h >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / (1 << 53))


def normal_torch(seed: int, stream: int, n: int, device, offset: int = 0) -> torch.Tensor:
    """float32 N(0,1) by Box-Muller on two independent uniform streams (computed in float64)."""
    u1 = uniform_torch(seed, 2 * stream, n, device, offset)
    u2 = uniform_torch(seed, 2 * stream + 1, n, device, offset)
    return (torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * math.pi) * u2)).to(torch.float32)


def normal_np(seed: int, stream: int, n: int, offset: int = 0) -> np.ndarray:
    u1 = uniform_np(seed, 2 * stream, n, offset)
    u2 = uniform_np(seed, 2 * stream + 1, n, offset)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos((2.0 * math.pi) * u2)).astype(np.float32)


# stream ids (kept apart so that changing one tensor's shape never shifts another's values)
_S_INDICES, _S_VALS, _S_WEIGHT, _S_BIAS, _S_TARGET, _S_GRAD = 1, 2, 3, 4, 5, 6


@dataclasses.dataclass(frozen=True)
class Workload:
    """One benchmark / parity configuration of the decoder-loss path."""

    name: str
    B: int
    K: int
    F: int
    D: int
    weight_dtype: str = "float32"      # dtype of weight, bias and target
    vals_dtype: str = "float32"
    indices: str = "dup"               # "dup" | "distinct" | "zipf"
    sort_vals: bool = False
    normalise_weight: bool = False     # weight ~ N(0,1)/sqrt(D), rows L2-normalised
    zipf_s: float = 1.1
    seed: int = 0

    def replace(self, **kw) -> "Workload":
        return dataclasses.replace(self, **kw)


# The five set-ups the headline metric and its parity cases are quoted on.
CONFIGS: Dict[str, Workload] = {
    "c1": Workload("c1", B=64, K=32, F=4096, D=256, indices="distinct", sort_vals=True, seed=0),
    "c2": Workload("c2", B=2048, K=256, F=131072, D=1024, indices="dup", seed=2),
    "c3_k32": Workload("c3_k32", B=4096, K=32, F=65536, D=2304, weight_dtype="bfloat16",
                       indices="distinct", sort_vals=True, normalise_weight=True, seed=3),
    "c3_k64": Workload("c3_k64", B=4096, K=64, F=65536, D=2304, weight_dtype="bfloat16",
                       indices="distinct", sort_vals=True, normalise_weight=True, seed=3),
    "c3_k128": Workload("c3_k128", B=4096, K=128, F=65536, D=2304, weight_dtype="bfloat16",
                        indices="distinct", sort_vals=True, normalise_weight=True, seed=3),
    "c4": Workload("c4", B=16384, K=64, F=65536, D=2304, weight_dtype="bfloat16",
                   indices="zipf", sort_vals=True, normalise_weight=True, seed=4),
    "c5": Workload("c5", B=65536, K=128, F=131072, D=4096, weight_dtype="bfloat16",
                   indices="distinct", sort_vals=True, normalise_weight=True, seed=5),
}

TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _indices_torch(w: Workload, device, row0: int, rows: int) -> torch.Tensor:
    """indices[row0:row0+rows, :] as int64."""
    if w.indices == "dup":
        u = uniform_torch(w.seed, _S_INDICES, rows * w.K, device, offset=row0 * w.K)
        return torch.clamp((u * w.F).to(torch.int64), max=w.F - 1).view(rows, w.K)
    out = torch.empty(rows, w.K, dtype=torch.int64, device=device)
    chunk = max(1, min(rows, (1 << 25) // w.F))
    log_rank = None
    if w.indices == "zipf":
        log_rank = -w.zipf_s * torch.log(torch.arange(1, w.F + 1, dtype=torch.float64, device=device))
    for r in range(0, rows, chunk):
        n = min(chunk, rows - r)
        u = uniform_torch(w.seed, _S_INDICES, n * w.F, device, offset=(row0 + r) * w.F).view(n, w.F)
        if w.indices == "distinct":
            score = u                                           # K largest of F iid uniforms
        else:
            score = log_rank - torch.log(-torch.log(u))         # Gumbel top-K
        out[r:r + n] = torch.topk(score, w.K, dim=1, largest=True, sorted=True).indices
    return out


def make_inputs(w: Workload, device="cpu", row0: int = 0, rows: Optional[int] = None,
                with_weight: bool = True) -> Dict[str, torch.Tensor]:
    """Builds the tensors of ``w`` on ``device``; ``row0/rows`` selects a batch shard.

    Every rank of a batch-sharded run calls this with its own ``row0`` and gets exactly the
    rows the single-process run would have, together with the full (replicated) decoder.
    """
    rows = w.B - row0 if rows is None else rows
    wd, vd = TORCH_DTYPES[w.weight_dtype], TORCH_DTYPES[w.vals_dtype]
    out: Dict[str, torch.Tensor] = {}
    out["indices"] = _indices_torch(w, device, row0, rows)
    v = normal_torch(w.seed, _S_VALS, rows * w.K, device, offset=row0 * w.K).abs().view(rows, w.K)
    if w.sort_vals:
        v = torch.sort(v, dim=1, descending=True).values
    out["vals"] = v.to(vd).contiguous()
    if with_weight:
        wt = torch.empty(w.F, w.D, dtype=wd, device=device)
        chunk = max(1, (1 << 24) // w.D)
        for f0 in range(0, w.F, chunk):
            n = min(chunk, w.F - f0)
            x = normal_torch(w.seed, _S_WEIGHT, n * w.D, device, offset=f0 * w.D).view(n, w.D)
            if w.normalise_weight:
                x = x / math.sqrt(w.D)
                x = x / x.norm(dim=1, keepdim=True)
            wt[f0:f0 + n] = x.to(wd)
        out["weight"] = wt
    out["bias"] = normal_torch(w.seed, _S_BIAS, w.D, device).to(wd)
    out["target"] = normal_torch(w.seed, _S_TARGET, rows * w.D, device, offset=row0 * w.D).view(rows, w.D).to(wd)
    out["grad_out"] = normal_torch(w.seed, _S_GRAD, 1, device).reshape(())
    return out


def algorithmic_bytes(w: Workload, rows: Optional[int] = None) -> int:
    """Bytes one fwd+bwd step has to move if every operand crossed HBM exactly as often as the
    arithmetic needs it: two row gathers, the fp32 scatter payload, the dense gradient table
    (zero-fill, and the fp32 -> storage-dtype conversion when the decoder is 16-bit), target and
    saved row state in both passes, indices / vals / dvals."""
    B = w.B if rows is None else rows
    sw = torch.empty((), dtype=TORCH_DTYPES[w.weight_dtype]).element_size()
    sv = torch.empty((), dtype=TORCH_DTYPES[w.vals_dtype]).element_size()
    n = 2 * B * w.K * w.D * sw + B * w.K * w.D * 4 + w.F * w.D * 4
    if sw != 4:
        n += w.F * w.D * (4 + sw)
    n += 2 * B * w.D * sw + 2 * B * w.D * 4 + 2 * B * w.K * (8 + sv) + B * w.K * 4
    return n
