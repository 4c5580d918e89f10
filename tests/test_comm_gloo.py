"""Host side of PeerAllReduce (nanovllm_jax_b200/comm.py) on CPU with two gloo ranks: the ranks exchange their 64-byte
handles through torch.distributed, each opens every peer's handle exactly once and keeps the pointers in rank order.
The C library is replaced by a fake that hands out recognisable handles (no GPU here)."""
import ctypes
import os
import sys

import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _FakeLib:
    """Stands in for libnvllm_b200_attn.so: alloc returns address 0x1000 * (rank + 1) and a handle naming the rank."""

    def __init__(self, rank):
        self.rank, self.opened, self.calls = rank, [], []

    def nvllm_b200_comm_alloc(self, max_bytes, buf_ref, handle):
        buf_ref._obj.value = 0x1000 * (self.rank + 1)
        handle.raw = (b"rank%d" % self.rank).ljust(64, b"\0")
        return 0

    def nvllm_b200_comm_open(self, handle, buf_ref):
        peer = int(bytes(handle.raw).rstrip(b"\0")[4:])
        self.opened.append(peer)
        buf_ref._obj.value = 0x1000 * (peer + 1) + 0x100000  # "mapped" address differs from the owner's
        return 0

    def nvllm_b200_comm_close(self, p):
        self.calls.append(("close", p.value))
        return 0

    def nvllm_b200_comm_free(self, p):
        self.calls.append(("free", p.value))
        return 0


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nanovllm_jax_b200 import _lib, comm
    fake = _FakeLib(rank)
    _lib.load = lambda: fake
    _lib.check = lambda rc: None
    torch.cuda.current_device = lambda: 0
    torch.cuda.synchronize = lambda *a, **k: None

    class _NoDev:
        def __init__(self, *a, **k): pass
        def __enter__(self): return self
        def __exit__(self, *a): return False
    torch.cuda.device = _NoDev
    ar = comm.PeerAllReduce(1 << 20, device="cpu")
    ptrs = [int(ar._ptrs[r] or 0) for r in range(world)]
    # a message the kernel does not take (fp32) goes to the process group's all-reduce, residual added afterwards
    x = torch.full((8,), float(rank + 1))
    ar.all_reduce_(x, residual=torch.ones(8))
    ar.close()
    q.put((rank, ptrs, sorted(fake.opened), x.tolist(), fake.calls))
    dist.destroy_process_group()


def test_two_ranks_exchange_handles_and_map_each_other():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ptrs, opened, x, calls in got:
        assert opened == [1 - rank], "each rank maps its one peer exactly once"
        assert ptrs[rank] == 0x1000 * (rank + 1) and ptrs[1 - rank] == 0x1000 * (2 - rank) + 0x100000
        assert x == [4.0] * 8  # 1 + 2 over the ranks, + residual
        assert [c[0] for c in calls] == ["close", "free"]
