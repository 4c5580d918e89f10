"""PeerAllReduce across real GPUs (skipped with fewer than two): one process per GPU, buffers mapped through CUDA IPC,
results compared bit for bit with the host sum in rank order and between ranks, sizes from 16 bytes to 1 MiB, with
and without the fused residual, interleaved with messages the kernel does not take (they go to NCCL)."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from nanovllm_jax_b200 import _lib
    from nanovllm_jax_b200.comm import PeerAllReduce
    ar = PeerAllReduce(1 << 20)
    ok, worst = True, 0.0
    for step, count in enumerate([8, 4096, 128 * 4096, 8 * 1000, 128 * 4096, 64, 524288, 4096 * 3]):
        gens = [np.random.Generator(np.random.PCG64(1000 * step + r)) for r in range(world)]
        xs = [torch.from_numpy(g.standard_normal(count, dtype=np.float32)).bfloat16() for g in gens]
        res = torch.from_numpy(np.random.Generator(np.random.PCG64(77 + step)).standard_normal(count, dtype=np.float32)).bfloat16()
        acc = torch.zeros(count, dtype=torch.float32)
        for x in xs:
            acc = acc + x.float()
        use_res = step % 2 == 1
        want = (acc + res.float()).bfloat16() if use_res else acc.bfloat16()
        mine = xs[rank].to(dev)
        ar.all_reduce_(mine, residual=res.to(dev) if use_res else None)
        torch.cuda.synchronize()
        ok = ok and torch.equal(mine.cpu(), want)
        worst = max(worst, float((mine.cpu().float() - want.float()).abs().max()))
        if step == 3:  # a message the kernel does not take: fp32 goes through the process group
            y = torch.full((16,), float(rank + 1), device=dev)
            ar.all_reduce_(y)
            ok = ok and bool((y == world * (world + 1) / 2).all())
    status = _lib.device_status()
    ar.close()
    q.put((rank, ok, worst, status))
    dist.destroy_process_group()


@pytest.mark.skipif(_gpus() < 2, reason="needs at least two GPUs")
def test_peer_allreduce_matches_the_host_sum_on_every_rank():
    import torch.multiprocessing as mp
    world = min(_gpus(), 8)
    while 8 % world:
        world -= 1
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok, worst, status in got:
        assert ok and status == 0, (rank, worst, status)
