"""GPU, one device, no fault: a wait inside a kernel that nothing will ever satisfy must end by
itself, report through the status word and leave the GPU usable.

``flexsae_small_allreduce`` is called as rank 0 of a 2-rank group whose "rank 1" never runs (both
exchange buffers are ordinary local memory): the kernel stores its values, announces itself and then
waits for rank 1's announcement, which never comes.  With ``wait_limit_ms`` set to 50 the wait gives
up after 50 ms on the GPU's timer, the kernel returns normally, the status word carries
FLEXSAE_STATUS_PIPELINE_TIMEOUT, ``check_status`` raises, and so does the check the batch-sharded
losses make at the start of their next step.  Nothing traps, nothing spins without a limit."""
import ctypes
import time

import numpy as np
import pytest
import torch

import flexsae_b200 as fx
from flexsae_b200 import _native as nv
from flexsae_b200 import distributed as fd
from flexsae_b200 import losses
from flexsae_b200.workloads import Workload, make_inputs
from oracle import flexsae_oracle as orc
from tests.helpers import inputs_as_numpy, rel_err

pytestmark = pytest.mark.gpu


def test_wait_for_a_rank_that_never_comes_gives_up_and_reports():
    lib = nv.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    fx.check_status()                                   # start from a clean status word
    before = nv.get_option("wait_limit_ms")
    nv.set_option("wait_limit_ms", 50)
    try:
        nbytes = ctypes.c_size_t()
        assert lib.flexsae_small_allreduce_bytes(2, 1024, ctypes.byref(nbytes)) == 0
        mine, absent = (torch.zeros(nbytes.value, dtype=torch.uint8, device=dev) for _ in range(2))
        ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
        src = torch.arange(8, dtype=torch.float32, device=dev)
        out = torch.empty_like(src)
        status = losses._status_word(dev)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        rc = lib.flexsae_small_allreduce(src.data_ptr(), out.data_ptr(), 8, nv.F32, 2, 0, 1, ptrs, 1024, status.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.flexsae_last_error()
        torch.cuda.synchronize()                        # returns: the wait was bounded
        waited = time.perf_counter() - t0
        assert 0.04 <= waited < 5.0, waited
        assert int(status.item()) & nv.STATUS_PIPELINE_TIMEOUT

        # the check the sharded losses make without synchronising: copy posted, then polled
        fd._post_status(dev)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="gave up waiting for another rank"):
            fd._raise_if_previous_step_timed_out(dev)
        with pytest.raises(RuntimeError, match="gave up"):
            fx.check_status()
        fx.check_status()                               # cleared by the report
    finally:
        nv.set_option("wait_limit_ms", before)

    # the device is in working order: an ordinary fused step still matches the oracle
    w = Workload("after", B=24, K=8, F=64, D=512, indices="dup", seed=91)
    x = make_inputs(w, "cuda")
    wt, v, b = (x[k].clone().requires_grad_(True) for k in ("weight", "vals", "bias"))
    loss = fx.triton_hierarchical_sae_loss(x["indices"], wt, v, b, x["target"])
    loss.backward(x["grad_out"])
    want = orc.hier_loss_and_grads(**inputs_as_numpy(x), grad_out=float(x["grad_out"]))
    assert abs(float(loss) - want["loss"]) <= 1e-5 * abs(want["loss"])
    assert rel_err(wt.grad.cpu().numpy(), want["dweight"]) < 2e-5
    fx.check_status()

