"""The two fused decoder losses as ``torch.autograd.Function``s over the CUDA library.

Public signature and autograd behaviour are those of ``flex_sae.triton_topk_sae_loss``
(torch-ext/flex_sae/topk_kernels.py:213-223) and ``flex_sae.triton_hierarchical_sae_loss``
(torch-ext/flex_sae/hierarchical_kernels.py:302-309):

    loss = f(indices[B,K] int64, weight[F,D], vals[B,K], bias[D], target[B,D])   # 0-dim float32

differentiable with respect to weight, vals and bias (gradients arrive in each parameter's own
dtype), ``None`` for indices and target (hierarchical_kernels.py:299), any upstream scalar.
Differences a caller can see: the loss value is run-to-run reproducible (the reference sums it
with float atomics, hierarchical_kernels.py:80-85), inputs are validated, and the upstream
gradient is applied inside the kernels instead of by three ``mul_`` passes
(hierarchical_kernels.py:294-297).
"""
from __future__ import annotations

import threading
from typing import Dict, Optional, Tuple

import torch

from . import _native as nv

_tls = threading.local()

#: kernels enqueued by the fused losses since the counter was last reset (benchmark accounting)
launch_count = 0


class config:
    """Process-wide switches of the fused losses."""

    #: "atomic" (vectorised fp32 reductions resolved in L2; the piece width follows the index
    #: distribution, see ``adaptive_pieces``), "atomic_wide" (the same with the widest column pieces
    #: always) or "deterministic" (sorted, fixed-order sums: bitwise reproducible dweight)
    dweight_mode: str = "atomic"
    #: check the device status word after every forward (forces a host sync; for debugging)
    check_indices: bool = False
    #: let the atomic backward follow the index distribution: every ``skew_interval``-th backward of
    #: a decoder shape measures how much of the batch its hottest decoder row takes (one tiny launch,
    #: read back without a synchronisation), and later backwards take the widest column pieces while
    #: that share is above ``skew_threshold`` (Zipf-like activations: up to 20 % faster), the
    #: L2-sized ones otherwise.  Measured at F=65536, D=2304 bf16, narrow / wide pieces in ms per
    #: step: share 0.0042 (Zipf 0.6, B=16384, K=64) 2.49 / 2.68; 0.0081 (Zipf 1.1, B=4096, K=128)
    #: 1.65 / 1.61; 0.0123 (Zipf 0.8, K=64) 3.30 / 2.92; 0.0154 (Zipf 1.1, K=64) 3.71 / 2.98.  Single-GPU backward only: the ranks of a sharded run must agree on the piece
    #: width, and each sees different indices.
    adaptive_pieces: bool = True
    skew_interval: int = 16
    skew_threshold: float = 1.0 / 144.0


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _prep(t: torch.Tensor) -> torch.Tensor:
    """Dense row-major, 16-byte aligned view of ``t`` (copies only when it has to)."""
    if not t.is_contiguous():
        t = t.contiguous()
    if t.data_ptr() % 16 != 0:
        t = t.clone(memory_format=torch.contiguous_format)
    return t


def _validate(indices, weight, vals, bias, target) -> Tuple[int, int, int, int]:
    if indices.dim() != 2 or weight.dim() != 2 or vals.dim() != 2 or bias.dim() != 1 or target.dim() != 2:
        raise ValueError("expected indices[B,K], weight[F,D], vals[B,K], bias[D], target[B,D]")
    B, K = indices.shape
    F, D = weight.shape
    if tuple(vals.shape) != (B, K) or tuple(bias.shape) != (D,) or tuple(target.shape) != (B, D):
        raise ValueError(f"shape mismatch: indices {tuple(indices.shape)}, weight {tuple(weight.shape)}, "
                         f"vals {tuple(vals.shape)}, bias {tuple(bias.shape)}, target {tuple(target.shape)}")
    if indices.dtype != torch.int64:
        raise TypeError(f"indices must be int64, got {indices.dtype}")
    for name, t in (("weight", weight), ("vals", vals), ("bias", bias), ("target", target)):
        if t.dtype not in nv.DTYPE_CODES:
            raise TypeError(f"{name} must be float32, bfloat16 or float16, got {t.dtype}")
    dev = weight.device
    if dev.type != "cuda":
        raise RuntimeError("the fused decoder losses run on CUDA tensors only "
                           "(use topk_sae_loss / hierarchical_sae_loss for the eager torch path)")
    for name, t in (("indices", indices), ("vals", vals), ("bias", bias), ("target", target)):
        if t.device != dev:
            raise RuntimeError(f"{name} is on {t.device}, weight is on {dev}")
    return B, K, F, D


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """A scratch buffer per (device, stream) that is kept between calls (so that the fp32 gradient
    slabs keep their L2 lines warm) and only ever grows.  Calls enqueued on different streams get
    different buffers, so they may overlap on the GPU; calls on one stream are ordered by it."""
    cache: Dict[tuple, torch.Tensor] = _tls.__dict__.setdefault("ws", {})
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    key = (index, torch.cuda.current_stream(dev).cuda_stream)
    buf = cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        cache[key] = buf
    return buf


def _status_word(dev: torch.device) -> torch.Tensor:
    cache: Dict[int, torch.Tensor] = _tls.__dict__.setdefault("status", {})
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in cache:
        cache[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return cache[key]


def check_status(device=None) -> None:
    """Raises if any fused-loss kernel on ``device`` met an out-of-range index since the last
    check (such an index is read as row 0 instead of being dereferenced)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_word(dev)
    bits = int(word.item())
    if bits:
        word.zero_()
        if bits & nv.STATUS_PIPELINE_TIMEOUT:
            raise RuntimeError("flexsae_b200: a bounded wait inside the single-launch backward gave up; "
                               "the gradients of that call are invalid")
        if bits & nv.STATUS_BAD_INDEX:
            raise IndexError("flexsae_b200: indices outside [0, F) were passed to a fused loss")


class _SkewWatch:
    """Per (device, F): the share of sampled positions held by the hottest decoder row, measured
    on the device every few backwards and read on the host only once the copy has arrived."""

    def __init__(self, dev: torch.device, F: int, lib) -> None:
        self.hist = torch.empty(lib.flexsae_index_skew_workspace_bytes(F), dtype=torch.uint8, device=dev)
        self.result = torch.zeros(2, dtype=torch.int32, device=dev)
        self.host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self.arrived: Optional[torch.cuda.Event] = None
        self.calls = 0
        self.share = 0.0

    def wide(self, lib, indices: torch.Tensor, F: int, stream) -> bool:
        """True when the next backward should take wide pieces; launches a measurement when due."""
        global launch_count
        if self.arrived is not None and self.arrived.query():
            self.arrived = None
            hottest, samples = int(self.host[0]), int(self.host[1])
            self.share = hottest / samples if samples else 0.0
        due = self.calls % max(1, config.skew_interval) == 0
        self.calls += 1
        if due and self.arrived is None:
            B, K = indices.shape
            nv.check(lib.flexsae_index_skew(_ptr(indices), B, K, F, _ptr(self.hist), self.hist.numel(),
                                            _ptr(self.result), stream), "flexsae_index_skew")
            launch_count += lib.flexsae_last_launch_count()
            self.host.copy_(self.result, non_blocking=True)
            self.arrived = torch.cuda.Event()
            self.arrived.record()
        return self.share > config.skew_threshold


_skew_watches: Dict[tuple, _SkewWatch] = {}     # process-wide: backwards run on autograd's threads
_skew_lock = threading.Lock()


def _skew_watch(dev: torch.device, F: int, lib) -> _SkewWatch:
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), F)
    with _skew_lock:
        if key not in _skew_watches:
            _skew_watches[key] = _SkewWatch(dev, F, lib)
        return _skew_watches[key]


def fused_forward(kind: int, indices, weight, vals, bias, target, inv_norm: float = 0.0):
    """Runs the forward kernels; returns (loss 0-dim float32, (state, segments), prepared inputs)."""
    B, K, F, D = _validate(indices, weight, vals, bias, target)
    lib = nv.load()
    indices, weight, vals, bias, target = (_prep(t.detach()) for t in (indices, weight, vals, bias, target))
    dev = weight.device
    wdt = nv.DTYPE_CODES[weight.dtype]
    with torch.cuda.device(dev):
        need = lib.flexsae_fwd_workspace_bytes(kind, B, K, F, D, wdt)
        if need == 0:
            raise nv.FlexSaeNativeError("flexsae_loss_fwd: " + lib.flexsae_last_error().decode())
        ws = _workspace(dev, need)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        segments = lib.flexsae_choose_segments(kind, B, K, F, D, wdt)
        state = torch.empty(lib.flexsae_state_bytes(kind, B, K, D, segments) // 4, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = lib.flexsae_loss_fwd(kind, _ptr(indices), _ptr(weight), _ptr(vals), _ptr(bias), _ptr(target),
                                  _ptr(loss), _ptr(state), segments, _ptr(ws), ws.numel(), B, K, F, D, wdt,
                                  nv.DTYPE_CODES[vals.dtype], nv.DTYPE_CODES[bias.dtype],
                                  nv.DTYPE_CODES[target.dtype], float(inv_norm), _ptr(_status_word(dev)), stream)
        nv.check(rc, "flexsae_loss_fwd")
        global launch_count
        launch_count += lib.flexsae_last_launch_count()
    if config.check_indices:
        check_status(dev)
    return loss, (state, segments), (indices, weight, vals)


def fused_backward(kind: int, indices, weight, vals, saved, grad_out, bias_dtype, inv_norm: float = 0.0,
                   dweight_mode: Optional[str] = None, peers=None):
    """Runs the backward kernels; returns (dweight, dvals, dbias) in the parameters' dtypes.
    With ``peers`` (a ``distributed.PeerExchange``) dweight is summed over the ranks in-kernel."""
    B, K = indices.shape
    F, D = weight.shape
    state, segments = saved
    lib = nv.load()
    dev = weight.device
    wdt = nv.DTYPE_CODES[weight.dtype]
    mode = {"atomic": nv.DW_ATOMIC, "atomic_wide": nv.DW_ATOMIC_WIDE,
            "deterministic": nv.DW_DETERMINISTIC}[dweight_mode or config.dweight_mode]
    with torch.cuda.device(dev):
        if (mode == nv.DW_ATOMIC and peers is None and config.adaptive_pieces
                and not torch.cuda.is_current_stream_capturing()
                and _skew_watch(dev, F, lib).wide(lib, indices, F, torch.cuda.current_stream(dev).cuda_stream)):
            mode = nv.DW_ATOMIC_WIDE
        go = grad_out.detach().to(device=dev, dtype=torch.float32).reshape(1).contiguous()
        need = lib.flexsae_bwd_workspace_bytes(kind, B, K, F, D, wdt, nv.DW_ATOMIC_SHARDED if peers is not None else mode)
        if need == 0:
            raise nv.FlexSaeNativeError("flexsae_loss_bwd: " + lib.flexsae_last_error().decode())
        ws = _workspace(dev, need)
        dw_ptrs = None
        if peers is not None and getattr(peers, "dweight", None) is not None:
            dweight, dw_ptrs = peers.take_dweight()      # every rank's table is peer-mapped: reduced rows land in place
        else:
            dweight = torch.empty((F, D), dtype=weight.dtype, device=dev)
        dvals = torch.empty((B, K), dtype=vals.dtype, device=dev)
        dbias = torch.empty((D,), dtype=bias_dtype, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        if peers is not None:
            rc = lib.flexsae_loss_bwd_sharded(kind, _ptr(indices), _ptr(weight), _ptr(vals), _ptr(state), segments,
                                              _ptr(go), _ptr(dweight), _ptr(dvals), _ptr(dbias), _ptr(ws), ws.numel(),
                                              B, K, F, D, wdt, nv.DTYPE_CODES[vals.dtype], nv.DTYPE_CODES[bias_dtype],
                                              float(inv_norm), _ptr(_status_word(dev)), stream, peers.world,
                                              peers.rank, peers.next_seq(), peers.x, peers.y, peers.flags,
                                              peers.mc_x, peers.mc_y, dw_ptrs)
        else:
            rc = lib.flexsae_loss_bwd(kind, _ptr(indices), _ptr(weight), _ptr(vals), _ptr(state), segments, _ptr(go),
                                      _ptr(dweight), _ptr(dvals), _ptr(dbias), _ptr(ws), ws.numel(), B, K, F, D, wdt,
                                      nv.DTYPE_CODES[vals.dtype], nv.DTYPE_CODES[bias_dtype], float(inv_norm), mode,
                                      _ptr(_status_word(dev)), stream)
        nv.check(rc, "flexsae_loss_bwd")
        global launch_count
        launch_count += lib.flexsae_last_launch_count()
    return dweight, dvals, dbias


class _FusedDecoderLoss(torch.autograd.Function):
    """Shared autograd glue; ``kind`` selects TopK or Hierarchical.  Plays the role of
    HierarchicalSAELossFunction (hierarchical_kernels.py:273-299) and of xFormersEmbeddingBag
    plus the eager tail around it (topk_kernels.py:188-223)."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, kind, inv_norm, indices, weight, vals, bias, target):
        loss, (state, segments), (idx_c, w_c, v_c) = fused_forward(kind, indices, weight, vals, bias, target, inv_norm)
        ctx.kind, ctx.inv_norm, ctx.bias_dtype, ctx.segments = kind, inv_norm, bias.dtype, segments
        ctx.save_for_backward(idx_c, w_c, v_c, state)
        return loss

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad):
        idx_c, w_c, v_c, state = ctx.saved_tensors
        dweight, dvals, dbias = fused_backward(ctx.kind, idx_c, w_c, v_c, (state, ctx.segments), grad, ctx.bias_dtype,
                                               ctx.inv_norm)
        return None, None, None, dweight, dvals, dbias, None


def triton_topk_sae_loss(indices: torch.Tensor, weight: torch.Tensor, vals: torch.Tensor, bias: torch.Tensor,
                         target: torch.Tensor) -> torch.Tensor:
    """Fused TopK decoder loss; drop-in for ``flex_sae.triton_topk_sae_loss`` (the name is kept
    for callers; no Triton is involved)."""
    if torch.compiler.is_compiling():
        from . import compile_ops
        return compile_ops.topk_sae_loss(indices, weight, vals, bias, target)
    return _FusedDecoderLoss.apply(nv.TOPK, 0.0, indices, weight, vals, bias, target)


def triton_hierarchical_sae_loss(indices: torch.Tensor, weight: torch.Tensor, vals: torch.Tensor,
                                 bias: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Fused Hierarchical-TopK decoder loss; drop-in for ``flex_sae.triton_hierarchical_sae_loss``."""
    if torch.compiler.is_compiling():
        from . import compile_ops
        return compile_ops.hierarchical_sae_loss(indices, weight, vals, bias, target)
    return _FusedDecoderLoss.apply(nv.HIER, 0.0, indices, weight, vals, bias, target)
