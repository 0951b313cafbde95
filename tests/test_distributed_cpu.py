"""CPU, world_size 2 over gloo: the batch-sharded wrapper's exchange logic against the
single-process oracle, with the oracle standing in for the per-shard kernels."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_impl():
    from flexsae_b200 import _native as nv
    from oracle import flexsae_oracle as orc

    def fwd(kind, indices, weight, vals, bias, target, inv_norm):
        fn = orc.hier_loss_and_grads if kind == nv.HIER else orc.topk_loss_and_grads
        B, K = indices.shape
        D = weight.shape[1]
        norm_rows = round(1.0 / (inv_norm * D * (K if kind == nv.HIER else 1)))
        out = fn(indices.numpy(), weight.double().numpy(), vals.double().numpy(), bias.double().numpy(),
                 target.double().numpy(), grad_out=1.0, norm_rows=norm_rows)
        return torch.tensor(out["loss"], dtype=torch.float32), out

    def bwd(kind, saved, grad, bias_dtype, inv_norm):
        g = float(grad)
        return (torch.from_numpy(saved["dweight"] * g).float(), torch.from_numpy(saved["dvals"] * g).float(),
                torch.from_numpy(saved["dbias"] * g).to(bias_dtype))

    return fwd, bwd


def _worker(rank, world, port, kind, rows, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flexsae_b200 import distributed as fd
        from flexsae_b200.workloads import Workload, make_inputs
        w = Workload("shard", B=sum(rows), K=8, F=48, D=64, indices="dup", seed=77)
        row0 = sum(rows[:rank])
        x = make_inputs(w, "cpu", row0=row0, rows=rows[rank])
        weight = x["weight"].clone().requires_grad_(True)
        vals = x["vals"].clone().requires_grad_(True)
        bias = x["bias"].clone().requires_grad_(True)
        fn = fd.sharded_hierarchical_sae_loss if kind == "hier" else fd.sharded_topk_sae_loss
        loss = fn(x["indices"], weight, vals, bias, x["target"], impl=_oracle_impl())
        loss.backward(torch.tensor(-1.5))
        q.put((rank, float(loss), weight.grad.numpy(), vals.grad.numpy(), bias.grad.numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["topk", "hier"])
@pytest.mark.parametrize("rows", [(6, 6), (9, 3)])
def test_two_rank_shards_match_single_process(kind, rows):
    sys.path.insert(0, ROOT)
    from flexsae_b200.workloads import Workload, make_inputs
    from oracle import flexsae_oracle as orc
    from tests.helpers import inputs_as_numpy

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 200) + (0 if kind == "topk" else 1) * 201 + rows[0]
    procs = [ctx.Process(target=_worker, args=(r, 2, port, kind, rows, q)) for r in range(2)]
    for p in procs:
        p.start()
    outs = sorted([q.get(timeout=120) for _ in procs], key=lambda o: o[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0

    w = Workload("shard", B=sum(rows), K=8, F=48, D=64, indices="dup", seed=77)
    want = orc.LOSSES[kind](**inputs_as_numpy(make_inputs(w, "cpu")), grad_out=-1.5)
    row0 = 0
    for rank, loss, dW, dv, db in outs:
        assert abs(loss - want["loss"]) < 1e-6 * abs(want["loss"])          # same global loss on every rank
        np.testing.assert_allclose(dW, want["dweight"], rtol=1e-5, atol=1e-9)  # reduced over ranks
        np.testing.assert_allclose(db, want["dbias"], rtol=1e-5, atol=1e-9)
        np.testing.assert_allclose(dv, want["dvals"][row0:row0 + rows[rank]], rtol=1e-5, atol=1e-9)  # local rows only
        row0 += rows[rank]


def test_persistent_gradient_table_is_not_overwritten_while_referenced():
    """symmetric_dweight hands out views of one persistent table; a backward must refuse to overwrite
    it while an earlier gradient is still alive (here without any GPU: only the bookkeeping)."""
    import torch

    from flexsae_b200 import distributed as fd

    ex = object.__new__(fd.PeerExchange)
    ex.dweight = torch.zeros(4, 8)
    ex.dweight_ptrs = None
    ex._dweight_refs = fd._storage_refs(ex.dweight)
    grad, _ = ex.take_dweight()
    assert grad.data_ptr() == ex.dweight.data_ptr() and grad.shape == (4, 8)
    with pytest.raises(RuntimeError, match="still referenced"):
        ex.take_dweight()
    holder = torch.nn.Parameter(torch.zeros(4, 8))
    holder.grad = grad
    del grad
    with pytest.raises(RuntimeError, match="still referenced"):      # held as somebody's .grad
        ex.take_dweight()
    holder.grad = None
    again, _ = ex.take_dweight()
    assert again.data_ptr() == ex.dweight.data_ptr()


def test_flag_sequence_restarts_before_a_c_int_would_overflow():
    """The flag values of the in-kernel exchange count up from call to call and are passed as C ints:
    long before INT32_MAX every rank restarts them collectively (zeroed flags, sequence 1)."""
    from flexsae_b200.distributed import PeerExchange

    ex = object.__new__(PeerExchange)          # no GPU, no symmetric memory: only the counting
    ex.slots = 23
    ex.seq = PeerExchange.SEQ_RESTART - 3 * ex.slots
    restarts = []

    def fake_restart():
        restarts.append(ex.seq)
        ex.seq = 1

    ex._restart = fake_restart
    seen = [ex.next_seq() for _ in range(6)]
    assert len(restarts) == 1
    assert all(1 <= s and s + ex.slots < 2 ** 31 for s in seen)
    assert seen[seen.index(1):] == [1 + i * ex.slots for i in range(len(seen) - seen.index(1))]   # contiguous again after it
    assert seen[:seen.index(1)] == sorted(seen[:seen.index(1)])
