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


def test_push_allreduce_wait_runs_out_on_one_gpu():
    """Bounded device-side wait: rank 0 of a two-rank reduction whose second 'peer' is a local buffer that
    nothing writes.  With the limit set to a few milliseconds the kernel gives up, records EPTQ_ERR_TIMEOUT in
    the status word and leaves `out` alone; the context stays usable and an ordinary call passes afterwards."""
    import ctypes as C
    from eptq_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    n, ranks = 4096, 2
    data = [torch.zeros(lib.eptq_allreduce_data_bytes(ranks, n), dtype=torch.uint8, device=dev) for _ in range(ranks)]
    flags = [torch.zeros(lib.eptq_allreduce_flag_bytes(ranks), dtype=torch.uint8, device=dev) for _ in range(ranks)]
    dp = (C.c_void_p * ranks)(*[t.data_ptr() for t in data])
    fp = (C.c_void_p * ranks)(*[t.data_ptr() for t in flags])
    x = torch.ones(n, device=dev, dtype=torch.float16)
    out = torch.full((n,), 7.0, device=dev, dtype=torch.float16)
    stream = torch.cuda.current_stream(dev).cuda_stream
    lib.eptq_allreduce_set_wait_ns(5_000_000)                       # 5 ms
    try:
        assert lib.eptq_allreduce_push(x.data_ptr(), out.data_ptr(), None, n, dp, fp, 0, ranks, n, stream) == 0
        torch.cuda.synchronize(dev)
    finally:
        lib.eptq_allreduce_set_wait_ns(0)
    status = int(flags[0].view(torch.int32)[2 * ranks * 8 + 8].item())
    assert status == 8                                              # EPTQ_ERR_TIMEOUT
    assert bool((out == 7.0).all())                                 # nothing was written
    # an ordinary one-rank reduction on the same GPU afterwards
    d1 = torch.zeros(lib.eptq_allreduce_data_bytes(1, n), dtype=torch.uint8, device=dev)
    f1 = torch.zeros(lib.eptq_allreduce_flag_bytes(1), dtype=torch.uint8, device=dev)
    y = torch.arange(n, device=dev).half()
    res = y.clone()
    assert lib.eptq_allreduce_push(res.data_ptr(), res.data_ptr(), None, n, (C.c_void_p * 1)(d1.data_ptr()),
                                   (C.c_void_p * 1)(f1.data_ptr()), 0, 1, n, stream) == 0
    torch.cuda.synchronize(dev)
    assert torch.equal(res, y)
    assert int(f1.view(torch.int32)[2 * 1 * 8 + 8].item()) == 0
