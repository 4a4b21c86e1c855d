"""One-shot push all-reduce between two GPUs of one node (skipped with fewer than two GPUs)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from eptq_b200.comm import PushAllReduce
    comm = PushAllReduce(dist.group.WORLD, 8192, dev)
    ok = True
    for it, n in enumerate([4096, 8192, 8, 4096, 4096, 1024]):
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = torch.randn(n, generator=g, device=dev).half()
        want = x.clone()
        dist.all_reduce(want)
        got = comm.all_reduce_(x.clone())
        ok &= bool(float((got.float() - want.float()).abs().max()) <= 2e-3 * float(want.float().abs().max()))
    res = torch.randn(4096, generator=torch.Generator(device=dev).manual_seed(5), device=dev).half()
    part = torch.full((4096,), 0.5 * (rank + 1), device=dev).half()
    want = res + sum(0.5 * (r + 1) for r in range(world))
    got = comm.all_reduce_(part, residual=res.clone())
    ok &= bool(float((got.float() - want.float()).abs().max()) <= 2e-3 * float(want.float().abs().max()))
    # replayed from a CUDA graph: the call counters advance on the device
    x = torch.full((4096,), float(rank + 1), device=dev).half()
    buf = x.clone()
    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        comm.all_reduce_(buf.copy_(x))
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            buf.copy_(x)
            comm.all_reduce_(buf)
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    ok &= bool((buf == sum(range(1, world + 1))).all())
    comm.check()
    results[rank] = ok
    dist.barrier()
    dist.destroy_process_group()


def test_push_allreduce_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(2, 29641, results), nprocs=2, join=True)
        assert results.get(0) is True and results.get(1) is True
