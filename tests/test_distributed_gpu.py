"""GPU, 2 ranks (and, when the box has more, as many ranks as GPUs) over NVLink: batch-sharded
fused losses against the single-GPU fused result on the whole batch.  Skipped with one GPU."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, kind, q, mode):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import flexsae_b200 as fx
        from flexsae_b200 import distributed as fd
        from flexsae_b200.workloads import CONFIGS, make_inputs
        fd.config.peer_reduce = mode != "nccl"
        fd.config.use_multicast = mode == "multicast"
        fd.config.symmetric_dweight = mode in ("inplace", "inplace_small", "inplace_lag2")
        fd.config.fused_small_reduce = mode == "inplace_small"
        if mode in ("lag2", "inplace_lag2"):        # three slabs in rotation, scatter two slots behind the accumulation
            fx._native.set_option("slabs", 3 if mode == "lag2" else 4)
            fx._native.set_option("convert_lag", 2 if mode == "lag2" else 3)
        if mode in ("inplace", "inplace_small", "inplace_lag2"):       # together with the other non-default exchange settings
            for name, value in (("exchange_offset_pct", 25), ("scatter_rotate", 1), ("flag_fan_out", 1)):
                fx._native.set_option(name, value)
        w = CONFIGS["c3_k32"].replace(B=768, F=8190)       # F not a multiple of the world size
        rows = w.B // world
        x = make_inputs(w, f"cuda:{rank}", row0=rank * rows, rows=rows)
        weight = x["weight"].requires_grad_(True)
        vals = x["vals"].requires_grad_(True)
        bias = x["bias"].requires_grad_(True)
        fn = fd.sharded_hierarchical_sae_loss if kind == "hier" else fd.sharded_topk_sae_loss
        for _ in range(3):          # several steps in a row on the same exchange buffers
            weight.grad = vals.grad = bias.grad = None
            loss = fn(x["indices"], weight, vals, bias, x["target"])
            loss.backward(x["grad_out"])
        torch.cuda.synchronize()
        fx.check_status()
        out = (rank, float(loss), weight.grad.float().cpu(), vals.grad.float().cpu(), bias.grad.float().cpu())
        if fd.config.symmetric_dweight:       # the gradient is a view of the persistent table: a backward that would
            loss = fn(x["indices"], weight, vals, bias, x["target"])   # overwrite it while it is held must refuse
            with pytest.raises(RuntimeError, match="still referenced"):
                loss.backward(x["grad_out"])
            torch.cuda.synchronize()
        q.put(out)
    finally:
        dist.destroy_process_group()


def _worlds():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return sorted({2, min(n, 8)}) if n > 2 else [2]


@pytest.mark.parametrize("world", _worlds())
@pytest.mark.parametrize("peer_reduce", ["multicast", "stores", "inplace", "nccl", "inplace_small", "lag2", "inplace_lag2"])
@pytest.mark.parametrize("kind", ["topk", "hier"])
def test_gpu_shards_match_one_gpu(kind, peer_reduce, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    import flexsae_b200 as fx
    from flexsae_b200.workloads import CONFIGS, make_inputs
    from tests.helpers import rel_err

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + os.getpid() % 100 + (7 if kind == "hier" else 0)
    port += {"multicast": 13, "stores": 5, "inplace": 17, "inplace_small": 19, "lag2": 21, "inplace_lag2": 23,
             "nccl": 0}[peer_reduce] + 29 * world
    procs = [ctx.Process(target=_worker, args=(r, world, port, kind, q, peer_reduce)) for r in range(world)]
    for p in procs:
        p.start()
    outs = sorted([q.get(timeout=300) for _ in procs], key=lambda o: o[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0

    w = CONFIGS["c3_k32"].replace(B=768, F=8190)
    x = make_inputs(w, "cuda:0")
    weight = x["weight"].requires_grad_(True)
    vals = x["vals"].requires_grad_(True)
    bias = x["bias"].requires_grad_(True)
    fn = fx.triton_hierarchical_sae_loss if kind == "hier" else fx.triton_topk_sae_loss
    loss = fn(x["indices"], weight, vals, bias, x["target"])
    loss.backward(x["grad_out"])
    rows = w.B // world
    for rank, l, dW, dv, db in outs:
        assert abs(l - float(loss)) <= 1e-6 * abs(float(loss))
        assert rel_err(dW.numpy(), weight.grad.float().cpu().numpy()) < 1e-2      # bf16 sum of bf16 shards
        assert rel_err(db.numpy(), bias.grad.float().cpu().numpy()) < 1e-2
        assert torch.equal(dv, vals.grad.float().cpu()[rank * rows:(rank + 1) * rows])


def _small_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import flexsae_b200 as fx
        from flexsae_b200 import distributed as fd
        ex = fd.small_exchange(None, torch.device("cuda", rank))
        assert ex is not None
        worst = 0.0
        same = True
        for step, (n, dtype) in enumerate([(1, torch.float32), (7, torch.float32), (2304, torch.bfloat16), (16384, torch.float32),
                                           (1, torch.float32), (2305, torch.float16), (33, torch.float32)] * 3):
            g = torch.Generator(device="cpu").manual_seed(1000 * step + rank)
            t = torch.randn(n, generator=g).to(device=f"cuda:{rank}", dtype=dtype)
            want = t.float().clone()
            dist.all_reduce(want)
            got = ex.all_reduce_(t.clone()).float()
            tol = 1e-6 if dtype == torch.float32 else 1e-2
            worst = max(worst, float(((got - want).abs() / (want.abs() + 1.0)).max()) / tol)
            every = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(every, got)
            same = same and all(torch.equal(every[0], e) for e in every)      # identical bits on every rank
        torch.cuda.synchronize()
        fx.check_status()
        q.put((rank, worst, same))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", _worlds())
def test_small_allreduce_matches_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 100 + 3 * world
    procs = [ctx.Process(target=_small_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    outs = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, worst, same in outs:
        assert worst <= 1.0, (rank, worst)
        assert same
