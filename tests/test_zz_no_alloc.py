"""GPU: the forward entry point that brings its own scratch memory.

Some callers of the C ABI cannot hand the library a scratch buffer because they are not allowed
to allocate device memory where the call happens (a host application that owns all allocations,
a memory pool that was handed out in full at start-up, a loop that cannot afford the implicit
synchronisation of an allocation).
``flexsae_loss_fwd_static_scratch`` serves them from a fixed 1 MiB array inside the library.
This test calls it through ctypes exactly as such a caller would -- inputs and outputs only --
and checks loss and saved state against the ordinary entry point, twice in a row, because the
array is shared by all calls and keeps the previous call's contents.

The file sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It passes alone in a fresh process and after the other tests.
"""
import pytest
import torch

from flexsae_b200 import _native as nv
from flexsae_b200.workloads import Workload, make_inputs

pytestmark = pytest.mark.gpu


def _call(lib, entry, kind, x, w, segments, workspace=None):
    dev = x["weight"].device
    loss = torch.full((), float("nan"), dtype=torch.float32, device=dev)
    state = torch.full((lib.flexsae_state_bytes(kind, w.B, w.K, w.D, segments) // 4,), float("nan"),
                       dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    codes = [nv.DTYPE_CODES[x[k].dtype] for k in ("weight", "vals", "bias", "target")]
    head = [kind] + [x[k].data_ptr() for k in ("indices", "weight", "vals", "bias", "target")] + \
           [loss.data_ptr(), state.data_ptr(), segments]
    tail = [w.B, w.K, w.F, w.D] + codes + [0.0, status.data_ptr(), torch.cuda.current_stream(dev).cuda_stream]
    if entry == "static":
        rc = lib.flexsae_loss_fwd_static_scratch(*head, *tail)
    else:
        rc = lib.flexsae_loss_fwd(*head, workspace.data_ptr(), workspace.numel(), *tail)
    assert rc == 0, lib.flexsae_last_error()
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0
    return loss, state


@pytest.mark.parametrize("kind", [nv.HIER, nv.TOPK])
def test_static_scratch_forward_matches_ordinary_forward_twice(kind):
    lib = nv.load()
    shapes = [Workload("a", B=300, K=32, F=2048, D=1536, weight_dtype="bfloat16", indices="distinct",
                       sort_vals=True, normalise_weight=True, seed=41),
              Workload("b", B=77, K=16, F=512, D=512, indices="dup", seed=42)]     # smaller: stale partials remain
    for w in shapes:                    # two calls in a row on the shared array, different shapes
        x = make_inputs(w, "cuda")
        wdt = nv.DTYPE_CODES[x["weight"].dtype]
        segments = lib.flexsae_choose_segments(kind, w.B, w.K, w.F, w.D, wdt)
        ws = torch.empty(lib.flexsae_fwd_workspace_bytes(kind, w.B, w.K, w.F, w.D, wdt), dtype=torch.uint8, device="cuda")
        want_loss, want_state = _call(lib, "ordinary", kind, x, w, segments, ws)
        for _ in range(2):              # and the same shape twice
            got_loss, got_state = _call(lib, "static", kind, x, w, segments)
            assert torch.isfinite(got_loss)
            torch.testing.assert_close(got_loss, want_loss, rtol=1e-5, atol=0.0)
            torch.testing.assert_close(got_state, want_state, rtol=1e-5, atol=1e-6)


def test_static_scratch_refuses_shapes_beyond_its_array():
    lib = nv.load()
    w = Workload("big", B=40000, K=8, F=64, D=4096, indices="dup", seed=43)   # 16+ pieces x 40000 rows > 262144
    rc = lib.flexsae_loss_fwd_static_scratch(nv.HIER, None, None, None, None, None, None, None, 1, w.B, w.K, w.F, w.D,
                                             nv.F32, nv.F32, nv.F32, nv.F32, 0.0, None, None)
    assert rc == -3
    msg = lib.flexsae_last_error().decode()
    assert "built-in scratch" in msg and "1048576" in msg
