"""ctypes binding of ``libflexsae_b200.so`` (declared in ``include/flexsae_b200.h``).

There is no fallback: if the library is missing or a call is rejected, an exception is raised.

Environment: ``FLEXSAE_LIB`` (path of a library built elsewhere), ``FLEXSAE_NO_BUILD=1`` (never invoke
nvcc), ``FLEXSAE_OPTIONS="name=value,..."`` (``flexsae_set_option`` calls made once when the library is
loaded, e.g. ``wait_limit_ms=60000`` for a job whose ranks may drift far apart).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

F32, BF16, F16 = 0, 1, 2
TOPK, HIER = 0, 1
DW_ATOMIC, DW_DETERMINISTIC, DW_ATOMIC_SHARDED, DW_ATOMIC_WIDE = 0, 1, 2, 3
STATUS_BAD_INDEX = 1
STATUS_PIPELINE_TIMEOUT = 2

DTYPE_CODES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_c_i64, _c_int, _c_vp, _c_sz, _c_dbl = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_double

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "flexsae_version": (_c_int, []),
    "flexsae_last_error": (ctypes.c_char_p, []),
    "flexsae_last_launch_count": (_c_int, []),
    "flexsae_set_option": (_c_int, [ctypes.c_char_p, _c_i64]),
    "flexsae_get_option": (_c_i64, [ctypes.c_char_p]),
    "flexsae_fwd_workspace_bytes": (_c_sz, [_c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_int]),
    "flexsae_bwd_workspace_bytes": (_c_sz, [_c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_int]),
    "flexsae_choose_segments": (_c_int, [_c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_int]),
    "flexsae_state_bytes": (_c_sz, [_c_int, _c_i64, _c_i64, _c_i64, _c_int]),
    "flexsae_loss_fwd": (_c_int, [_c_int] + [_c_vp] * 7 + [_c_int, _c_vp, _c_sz] + [_c_i64] * 4 + [_c_int] * 4
                         + [_c_dbl, _c_vp, _c_vp]),
    "flexsae_shard_buffer_bytes": (_c_int, [_c_i64, _c_i64, _c_int, _c_int, _c_vp, _c_vp, _c_vp]),
    "flexsae_shard_slots": (_c_int, [_c_i64, _c_i64, _c_int]),
    "flexsae_loss_bwd_sharded": (_c_int, [_c_int] + [_c_vp] * 4 + [_c_int] + [_c_vp] * 5 + [_c_sz] + [_c_i64] * 4
                                 + [_c_int] * 3 + [_c_dbl, _c_vp, _c_vp] + [_c_int] * 3 + [_c_vp] * 6),
    "flexsae_topk_select": (_c_int, [_c_vp, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_vp, _c_int, _c_vp, _c_vp]),
    "flexsae_small_allreduce_bytes": (_c_int, [_c_int, _c_i64, _c_vp]),
    "flexsae_small_allreduce": (_c_int, [_c_vp, _c_vp, _c_i64, _c_int, _c_int, _c_int, _c_int, _c_vp, _c_i64, _c_vp, _c_vp]),
    "flexsae_sort_workspace_bytes": (_c_sz, [_c_i64, _c_i64]),
    "flexsae_sort_by_decoder_row": (_c_int, [_c_vp, _c_i64, _c_i64, _c_vp, _c_sz, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp]),
    "flexsae_index_skew_workspace_bytes": (_c_sz, [_c_i64]),
    "flexsae_index_skew": (_c_int, [_c_vp, _c_i64, _c_i64, _c_i64, _c_vp, _c_sz, _c_vp, _c_vp]),
    "flexsae_loss_fwd_static_scratch": (_c_int, [_c_int] + [_c_vp] * 7 + [_c_int] + [_c_i64] * 4 + [_c_int] * 4
                                        + [_c_dbl, _c_vp, _c_vp]),
    "flexsae_loss_bwd": (_c_int, [_c_int] + [_c_vp] * 4 + [_c_int] + [_c_vp] * 5 + [_c_sz] + [_c_i64] * 4
                         + [_c_int] * 3 + [_c_dbl, _c_int, _c_vp, _c_vp]),
}

_lib: Optional[ctypes.CDLL] = None


class FlexSaeNativeError(RuntimeError):
    pass


def lib_path() -> str:
    return _build.LIB_PATH


def load() -> ctypes.CDLL:
    """Loads the shared library (building it first if nvcc is present and sources are newer)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    override = os.environ.get("FLEXSAE_LIB")        # a library built elsewhere (tuning variants)
    if override:
        path = override
    elif os.environ.get("FLEXSAE_NO_BUILD", "0") != "1":
        try:
            path = _build.build()
        except RuntimeError:
            if not os.path.exists(path):
                raise
    if not os.path.exists(path):
        raise FlexSaeNativeError(
            f"{path} is missing: build it with `python -m flexsae_b200.build` (needs nvcc); "
            "flexsae_b200 has no non-CUDA implementation of the fused losses")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    for item in filter(None, os.environ.get("FLEXSAE_OPTIONS", "").split(",")):
        name, _, value = item.partition("=")
        check(lib.flexsae_set_option(name.strip().encode(), int(value)), f"FLEXSAE_OPTIONS: {item}")
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().flexsae_last_error().decode("utf-8", "replace")
        raise FlexSaeNativeError(f"{what} failed (code {rc}): {msg}")


def set_option(name: str, value: int) -> None:
    check(load().flexsae_set_option(name.encode(), int(value)), f"set_option({name}={value})")


def get_option(name: str) -> int:
    return int(load().flexsae_get_option(name.encode()))
