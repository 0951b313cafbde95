"""Batch-sharded decoder losses for the GPUs of one node.

The reference is single-GPU.  Here every rank holds a shard of the batch rows
(``indices``, ``vals``, ``target``) and a full replica of the decoder (``weight``, ``bias``).
Each rank runs the ordinary fused kernels on its rows with the GLOBAL normaliser
1/(B_global*D) resp. 1/(B_global*K*D), so its loss is its additive share of the global mean and
its gradients are its additive share of the global gradients.  The scalar loss and ``dbias`` (D
values) are summed over the ranks by NCCL or, with ``config.fused_small_reduce``, by the library's own
single-launch exchange.  The dense ``dweight`` table is summed over the ranks INSIDE the backward
kernel: its converting blocks push each finished column piece to the ranks that own its rows and the
owners push the reduced rows back, all as posted NVLink peer STORES (no remote loads), while the next
pieces are still being accumulated (``flexsae_loss_bwd_sharded``), so no separate all-reduce of the
[F, D] gradient is exposed.  ``config.peer_reduce = False`` falls back to an NCCL all-reduce of
``dweight`` after the backward.  ``dvals`` belongs to the local rows and needs no exchange.

The in-kernel exchange makes the ranks wait for one another on the GPU, with a time limit
(``flexsae_set_option("wait_limit_ms")``, 5 s by default).  A rank whose backward is enqueued later
than that after the others' makes them give up: they set ``FLEXSAE_STATUS_PIPELINE_TIMEOUT`` in their
status word and their gradients of that step are INVALID.  The sharded losses look at the status word
of the previous step at the start of every call (an asynchronous copy to pinned memory, no
synchronisation) and raise ``RuntimeError`` when the bit is set, so a bad step is reported one step
late at the latest; ``flexsae_b200.check_status()`` reports it at once, at the price of a
synchronisation.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import _native as nv
from . import losses as _losses

# (forward, backward) of one shard; replaceable so that the exchange logic can be exercised on
# CPU ranks (gloo) with any implementation of the local math.
LocalImpl = Tuple[Callable, Callable]


class config:
    #: sum dweight over the ranks inside the backward kernel (NVLink peer memory) instead of an
    #: NCCL all-reduce afterwards
    peer_reduce: bool = True
    #: let the NVSwitch do the sum and the broadcast (multimem) when the exchange buffers could be
    #: bound to a multicast object; otherwise, or when False, plain peer stores.  Off by default:
    #: measured on 2 GPUs it is 7 % slower than peer stores (it saves bytes only from 4 ranks up)
    use_multicast: bool = False
    #: keep ``weight.grad`` of the sharded losses in one persistent peer-mapped table per decoder
    #: shape, so that the reduced rows are stored straight into every rank's gradient (no gather
    #: buffer, no copy pass).  The gradient a backward returns is then a view of that table and the
    #: NEXT sharded backward of the same shape overwrites it: consume it (optimizer step) and drop
    #: it (``grad = None`` / ``zero_grad(set_to_none=True)``) before then, on the same stream.  A
    #: backward that finds the previous gradient still referenced raises instead of overwriting it.
    symmetric_dweight: bool = False
    #: sum the scalar loss and dbias over the ranks with the library's own single-launch exchange
    #: over peer memory (``flexsae_small_allreduce``) instead of two NCCL all-reduces, whose latency
    #: is a visible share of a 2 ms step (falls back to NCCL where symmetric memory is unavailable)
    fused_small_reduce: bool = True


class PeerExchange:
    """Symmetric exchange buffers of one (process group, device, decoder shape, dtype): every
    rank's X / Y / flag buffers mapped into every process, plus the running sequence number."""

    def __init__(self, group, device: torch.device, F: int, D: int, dtype: torch.dtype):
        import torch.distributed._symmetric_memory as symm_mem

        lib = nv.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        wdt = nv.DTYPE_CODES[dtype]
        xb, yb, fb = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_size_t()
        nv.check(lib.flexsae_shard_buffer_bytes(F, D, wdt, self.world, ctypes.byref(xb), ctypes.byref(yb),
                                                ctypes.byref(fb)), "flexsae_shard_buffer_bytes")
        self.slots = lib.flexsae_shard_slots(F, D, wdt)
        with torch.cuda.device(device):
            self.buffer = symm_mem.empty(xb.value + yb.value + fb.value, dtype=torch.uint8, device=device)
            self.buffer.zero_()
            self.handle = symm_mem.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
            torch.cuda.synchronize(device)
        dist.barrier(group)            # every rank's flags are zero before anyone can publish
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        arr = ctypes.c_void_p * self.world
        self.x = arr(*ptrs)
        self.y = arr(*[p + xb.value for p in ptrs])
        self.flags = arr(*[p + xb.value + yb.value for p in ptrs])
        self.flag_words = self.buffer[xb.value + yb.value:xb.value + yb.value + fb.value]
        mc = 0
        if config.use_multicast:
            try:
                mc = int(self.handle.multicast_ptr or 0)
            except Exception:
                mc = 0
        self.multicast = mc != 0
        self.mc_x = ctypes.c_void_p(mc) if mc else None
        self.mc_y = ctypes.c_void_p(mc + xb.value) if mc else None
        self.seq = 1
        self.dweight = None
        if config.symmetric_dweight and not self.multicast:
            with torch.cuda.device(device):
                flat = symm_mem.empty(F * D, dtype=dtype, device=device)
                self.dweight_handle = symm_mem.rendezvous(flat, group if group is not None else dist.group.WORLD)
                self.dweight = flat.view(F, D)
                del flat
            self.dweight_ptrs = arr(*[int(p) for p in self.dweight_handle.buffer_ptrs])
            self._dweight_refs = _storage_refs(self.dweight)

    def take_dweight(self):
        """A fresh view of the persistent gradient table plus every rank's address of it."""
        if _storage_refs(self.dweight) > self._dweight_refs:
            raise RuntimeError("flexsae_b200: the weight gradient of the previous sharded backward is still referenced and "
                               "this backward would overwrite it; drop it first (grad = None) or set "
                               "flexsae_b200.distributed.config.symmetric_dweight = False")
        return self.dweight.view(self.dweight.shape), self.dweight_ptrs

    #: the flag values count up from call to call as C ints; long before they would overflow, all
    #: ranks start again from 1 on zeroed flags
    SEQ_RESTART = (1 << 31) - (1 << 20)

    def next_seq(self) -> int:
        if self.seq + 2 * self.slots >= self.SEQ_RESTART:
            self._restart()
        seq = self.seq
        self.seq += self.slots
        return seq

    def _restart(self) -> None:
        """Collective (every rank gets here at the same call, because all ranks count alike): nobody is
        inside a kernel that uses the flags, then zero them and count from 1 again."""
        torch.cuda.synchronize(self.buffer.device)
        dist.barrier(self.group)
        self.flag_words.zero_()
        torch.cuda.synchronize(self.buffer.device)
        dist.barrier(self.group)
        self.seq = 1


def _storage_refs(t: torch.Tensor) -> int:
    """How many tensors (and storage handles) share ``t``'s memory."""
    counter = getattr(torch._C, "_storage_Use_Count", None)
    if counter is None:
        raise RuntimeError("flexsae_b200.distributed.config.symmetric_dweight needs torch._C._storage_Use_Count "
                           "(to refuse overwriting a gradient that is still referenced); this torch build lacks it")
    return counter(t.untyped_storage()._cdata)


_exchanges: Dict[tuple, PeerExchange] = {}


def peer_exchange(group, device: torch.device, F: int, D: int, dtype: torch.dtype) -> Optional[PeerExchange]:
    """The exchange buffers for this shape, created on first use (a collective: every rank of the
    group must get here together, which they do when they run the same training step).  ``None``
    when symmetric memory cannot be set up on this machine (agreed on by all ranks)."""
    key = (id(group) if group is not None else 0, device.index, F, D, dtype,
           nv.get_option("lanes_bwd"), nv.get_option("lanes_sharded"), nv.get_option("l2_budget_mb"), nv.get_option("slabs"),
           config.use_multicast,
           config.symmetric_dweight)
    if key not in _exchanges:
        ex, problem = None, None
        try:
            ex = PeerExchange(group, device, F, D, dtype)
        except Exception as e:  # no symmetric memory / no peer access on this machine
            problem = e
        ok = torch.tensor([0 if ex is None else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)      # all ranks take the same path
        if int(ok.item()) == 0:
            import warnings
            warnings.warn(f"flexsae_b200: peer-memory exchange unavailable ({problem}); "
                          "dweight will be all-reduced with NCCL after the backward")
            ex = None
        _exchanges[key] = ex
    return _exchanges[key]


class SmallExchange:
    """Symmetric buffer and running sequence number of ``flexsae_small_allreduce`` for one (process
    group, device): sums short vectors (up to ``CAPACITY`` values) over the ranks in one launch."""

    CAPACITY = 16384

    def __init__(self, group, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        lib = nv.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        nbytes = ctypes.c_size_t()
        nv.check(lib.flexsae_small_allreduce_bytes(self.world, self.CAPACITY, ctypes.byref(nbytes)),
                 "flexsae_small_allreduce_bytes")
        with torch.cuda.device(device):
            self.buffer = symm_mem.empty(nbytes.value, dtype=torch.uint8, device=device)
            self.buffer.zero_()
            self.handle = symm_mem.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
            torch.cuda.synchronize(device)
        dist.barrier(group)            # every rank's flags are zero before anyone can announce
        self.ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self.handle.buffer_ptrs])
        self.seq = 0

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum of ``t`` over the ranks, on the current stream."""
        if not (t.is_cuda and t.is_contiguous() and 1 <= t.numel() <= self.CAPACITY and t.dtype in nv.DTYPE_CODES):
            raise ValueError("SmallExchange.all_reduce_ takes a contiguous fp32/bf16/fp16 CUDA tensor of at most "
                             f"{self.CAPACITY} values")
        lib = nv.load()
        if self.seq >= PeerExchange.SEQ_RESTART:      # same collective restart as PeerExchange._restart
            torch.cuda.synchronize(t.device)
            dist.barrier(self.group)
            self.buffer.zero_()
            torch.cuda.synchronize(t.device)
            dist.barrier(self.group)
            self.seq = 0
        self.seq += 1
        with torch.cuda.device(t.device):
            rc = lib.flexsae_small_allreduce(t.data_ptr(), t.data_ptr(), t.numel(), nv.DTYPE_CODES[t.dtype], self.world,
                                             self.rank, self.seq, self.ptrs, self.CAPACITY,
                                             _losses._ptr(_losses._status_word(t.device)),
                                             torch.cuda.current_stream(t.device).cuda_stream)
        nv.check(rc, "flexsae_small_allreduce")
        _losses.launch_count += lib.flexsae_last_launch_count()
        return t


_small_exchanges: Dict[tuple, Optional[SmallExchange]] = {}


def small_exchange(group, device: torch.device) -> Optional[SmallExchange]:
    """The small-vector exchange of this (group, device), created on first use (a collective);
    ``None`` when symmetric memory cannot be set up here (agreed on by all ranks)."""
    key = (id(group) if group is not None else 0, device.index)
    if key not in _small_exchanges:
        ex = None
        try:
            ex = SmallExchange(group, device)
        except Exception:  # no symmetric memory / no peer access on this machine
            ex = None
        ok = torch.tensor([0 if ex is None else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        _small_exchanges[key] = ex if int(ok.item()) == 1 else None
    return _small_exchanges[key]


def _sum_over_ranks_(t: torch.Tensor, group, fused: bool) -> torch.Tensor:
    """In-place sum of a small tensor over the group: own exchange when asked for and possible, else NCCL / gloo."""
    if fused and t.is_cuda and t.numel() <= SmallExchange.CAPACITY and 2 <= dist.get_world_size(group) <= 8:
        ex = small_exchange(group, t.device)
        if ex is not None:
            return ex.all_reduce_(t if t.is_contiguous() else t.contiguous())
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


class _StatusWatch:
    """Pinned host mirror of one device's status word.  ``post`` enqueues a copy of the word behind
    the work already on the current stream; ``poll`` looks at the last copy that has arrived, without
    waiting for anything."""

    def __init__(self):
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event: Optional[torch.cuda.Event] = None

    def post(self, dev: torch.device) -> None:
        self.host.copy_(_losses._status_word(dev), non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record(torch.cuda.current_stream(dev))

    def poll(self) -> int:
        if self.event is None or not self.event.query():
            return 0
        return int(self.host[0])


_watches: Dict[int, _StatusWatch] = {}


def _raise_if_previous_step_timed_out(dev: torch.device) -> None:
    watch = _watches.get(dev.index)
    if watch is not None and watch.poll() & nv.STATUS_PIPELINE_TIMEOUT:
        watch.event = None
        raise RuntimeError(
            "flexsae_b200: an earlier batch-sharded backward on this GPU gave up waiting for another rank "
            "(FLEXSAE_STATUS_PIPELINE_TIMEOUT): the gradients of that step are invalid and must not be applied. "
            "A rank enqueued its backward more than wait_limit_ms after the others, or died. "
            "flexsae_b200.check_status() clears the flag.")


def _post_status(dev: torch.device) -> None:
    _watches.setdefault(dev.index, _StatusWatch()).post(dev)


def _fused_local_forward(kind, indices, weight, vals, bias, target, inv_norm):
    loss, saved, (idx_c, w_c, v_c) = _losses.fused_forward(kind, indices, weight, vals, bias, target, inv_norm)
    return loss, (idx_c, w_c, v_c, saved)


def _fused_local_backward(kind, ctx_saved, grad, bias_dtype, inv_norm):
    idx_c, w_c, v_c, saved = ctx_saved
    return _losses.fused_backward(kind, idx_c, w_c, v_c, saved, grad, bias_dtype, inv_norm)


FUSED_IMPL: LocalImpl = (_fused_local_forward, _fused_local_backward)


def _fused_backward_with_peer_reduce(kind, ctx_saved, grad, bias_dtype, inv_norm, group):
    """Backward of this rank's shard; dweight comes back already summed over the group."""
    idx_c, w_c, v_c, saved = ctx_saved
    ex = peer_exchange(group, w_c.device, w_c.shape[0], w_c.shape[1], w_c.dtype)
    out = _losses.fused_backward(kind, idx_c, w_c, v_c, saved, grad, bias_dtype, inv_norm, dweight_mode="atomic",
                                 peers=ex)
    if ex is None:  # no peer memory here: the plain collective instead
        dist.all_reduce(out[0], op=dist.ReduceOp.SUM, group=group)
    return out


class _ShardedDecoderLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, kind, group, impl, global_rows, indices, weight, vals, bias, target):
        B, K = indices.shape
        D = weight.shape[1]
        inv_norm = 1.0 / (float(global_rows) * D * (K if kind == nv.HIER else 1))
        fwd, _ = impl
        if impl is FUSED_IMPL:
            _raise_if_previous_step_timed_out(weight.device)
        loss, saved = fwd(kind, indices, weight, vals, bias, target, inv_norm)
        loss = _sum_over_ranks_(loss.clone(), group, impl is FUSED_IMPL and config.fused_small_reduce)
        ctx.kind, ctx.group, ctx.impl, ctx.inv_norm, ctx.bias_dtype = kind, group, impl, inv_norm, bias.dtype
        ctx.saved = saved
        return loss

    @staticmethod
    def backward(ctx, grad):
        _, bwd = ctx.impl
        world = dist.get_world_size(ctx.group)
        fused_peer = (ctx.impl is FUSED_IMPL and config.peer_reduce and 2 <= world <= 8
                      and _losses.config.dweight_mode in ("atomic", "atomic_wide"))   # the sharded kernel has its own piece width
        if fused_peer:
            dweight, dvals, dbias = _fused_backward_with_peer_reduce(ctx.kind, ctx.saved, grad, ctx.bias_dtype,
                                                                     ctx.inv_norm, ctx.group)
        else:
            dweight, dvals, dbias = bwd(ctx.kind, ctx.saved, grad, ctx.bias_dtype, ctx.inv_norm)
            dist.all_reduce(dweight, op=dist.ReduceOp.SUM, group=ctx.group)
        ctx.saved = None
        dbias = _sum_over_ranks_(dbias, ctx.group, ctx.impl is FUSED_IMPL and config.fused_small_reduce)
        if ctx.impl is FUSED_IMPL:
            _post_status(dweight.device)
        return None, None, None, None, None, dweight, dvals, dbias, None


def global_batch_rows(local_rows: int, group=None) -> int:
    """Sum of the ranks' local row counts (shards may be ragged)."""
    t = torch.tensor([local_rows], dtype=torch.int64)
    backend = dist.get_backend(group)
    if backend == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return int(t.item())


def sharded_topk_sae_loss(indices, weight, vals, bias, target, group=None, global_rows: Optional[int] = None,
                          impl: LocalImpl = FUSED_IMPL) -> torch.Tensor:
    """TopK loss of the GLOBAL batch from this rank's rows; identical on every rank."""
    if global_rows is None:
        global_rows = global_batch_rows(indices.shape[0], group)
    return _ShardedDecoderLoss.apply(nv.TOPK, group, impl, global_rows, indices, weight, vals, bias, target)


def sharded_hierarchical_sae_loss(indices, weight, vals, bias, target, group=None, global_rows: Optional[int] = None,
                                  impl: LocalImpl = FUSED_IMPL) -> torch.Tensor:
    """Hierarchical-TopK loss of the GLOBAL batch from this rank's rows; identical on every rank."""
    if global_rows is None:
        global_rows = global_batch_rows(indices.shape[0], group)
    return _ShardedDecoderLoss.apply(nv.HIER, group, impl, global_rows, indices, weight, vals, bias, target)
