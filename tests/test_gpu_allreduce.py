"""One-shot all-reduce kernel (csrc/allreduce.cu) on ONE GPU: the ranks of a world are emulated by one cooperative
launch over all ranks' data (kernels that wait on one another must not run as separate launches on one device), and the
result is checked against the host sum in rank order, bit for bit.  A second test makes the wait for a peer run out --
a flag that nothing sets, a small poll limit -- and checks that the kernel returns with the status bit raised and the
context still usable (no trap, no hang)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _bf16_round(x):
    from oracle import reference_attention as ref
    return ref.bf16_bits_to_f32(ref.f32_to_bf16_bits(x.astype(np.float32)))


def _alloc(lib, max_bytes):
    import torch
    n = int(lib.nvllm_b200_comm_buffer_bytes(max_bytes))
    return torch.zeros(n, dtype=torch.uint8, device="cuda")  # same layout as comm_alloc's buffer, owned by torch


@pytest.mark.parametrize("world,count,with_residual", [(2, 8, False), (2, 128 * 4096, True), (4, 37 * 1024, False),
                                                       (4, 128 * 4096, True), (3, 5000 * 8, True)])
def test_emulated_world_matches_the_host_sum_bit_for_bit(world, count, with_residual):
    import torch
    from nanovllm_jax_b200 import _lib
    lib = _lib.load()
    max_bytes = 1 << 20  # (worlds beyond 4 do not fit one device as co-resident blocks: they run on real GPUs instead)
    rng = np.random.Generator(np.random.PCG64(800 + world + count))
    xs = [_bf16_round(rng.standard_normal(count)) for _ in range(world)]
    res = [_bf16_round(rng.standard_normal(count)) for _ in range(world)] if with_residual else None
    bufs = [_alloc(lib, max_bytes) for _ in range(world)]
    ins = [torch.from_numpy(x).cuda().bfloat16() for x in xs]
    outs = [torch.full((count,), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    rs = [torch.from_numpy(r).cuda().bfloat16() for r in res] if res else None
    arr = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
    stream = torch.cuda.current_stream().cuda_stream
    for epoch in (1, 2, 3):  # three calls in a row: both staging slots, and a slot reused
        _lib.check(lib.nvllm_b200_allreduce_sum_emulated(arr(ins), arr(outs), arr(rs) if rs else None, arr(bufs), world,
                                                         count, max_bytes, epoch, 1 << 22, stream))
        torch.cuda.synchronize()
        acc = np.zeros(count, np.float32)
        for x in xs:  # rank order, fp32 accumulation: what the kernel does
            acc = acc + x
        for r in range(world):
            want = _bf16_round(acc + res[r]) if res else _bf16_round(acc)
            got = outs[r].float().cpu().numpy()
            assert np.array_equal(got, want), (world, count, epoch, r, np.abs(got - want).max())
        # next call sums the previous outputs of rank 0 on every rank: inputs change, so stale staging would show
        xs = [_bf16_round(x * np.float32(0.5) + np.float32(r)) for r, x in enumerate(xs)]
        for t, x in zip(ins, xs):
            t.copy_(torch.from_numpy(x).cuda().bfloat16())
    assert _lib.device_status() == 0


def test_calls_numbered_on_the_device():
    """epoch 0: the kernel takes the call number from the counter in each rank's buffer, so the very same launch
    parameters (what a CUDA-graph replay re-issues) make a new call every time."""
    import torch
    from nanovllm_jax_b200 import _lib
    lib = _lib.load()
    world, count, max_bytes = 3, 6 * 4096, 1 << 18
    bufs = [_alloc(lib, max_bytes) for _ in range(world)]
    ins = [torch.zeros(count, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    outs = [torch.zeros(count, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    arr = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
    a_in, a_out, a_buf = arr(ins), arr(outs), arr(bufs)
    for call in range(1, 6):
        for r, t in enumerate(ins):
            t.fill_(float(call * (r + 1)))
        _lib.check(lib.nvllm_b200_allreduce_sum_emulated(a_in, a_out, None, a_buf, world, count, max_bytes, 0, 1 << 22,
                                                         torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        for o in outs:
            assert bool((o == float(6 * call)).all()), call
    assert _lib.device_status() == 0


def test_in_place_and_size_limits():
    import torch
    from nanovllm_jax_b200 import _lib
    lib = _lib.load()
    world, count, max_bytes = 2, 4096, 8192
    bufs = [_alloc(lib, max_bytes) for _ in range(world)]
    xs = [torch.arange(count, device="cuda").float().mul(0.001 * (r + 1)).bfloat16() for r in range(world)]
    want = (xs[0].float() + xs[1].float()).bfloat16()
    arr = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
    _lib.check(lib.nvllm_b200_allreduce_sum_emulated(arr(xs), arr(xs), None, arr(bufs), world, count, max_bytes, 1,
                                                     1 << 22, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(xs[0], want) and torch.equal(xs[1], want)
    rc = lib.nvllm_b200_allreduce_sum_emulated(arr(xs), arr(xs), None, arr(bufs), world, 8192, max_bytes, 2, 1 << 22, None)
    assert rc == _lib.EWORKSPACE
    rc = lib.nvllm_b200_allreduce_sum_emulated(arr(xs), arr(xs), None, arr(bufs), world, 4, max_bytes, 2, 1 << 22, None)
    assert rc == _lib.EUNSUPPORTED


def test_a_peer_that_never_signals_ends_in_a_status_bit_not_a_hang():
    """Rank 0 of a world of 2 runs alone: the flag of rank 1 is never written.  With a small poll limit the kernel gives
    up within milliseconds, raises bit 6, writes nothing, and the device keeps working."""
    import torch
    from nanovllm_jax_b200 import _lib
    lib = _lib.load()
    world, count, max_bytes = 2, 64 * 1024, 1 << 20
    bufs = [_alloc(lib, max_bytes) for _ in range(world)]
    x = torch.ones(count, dtype=torch.bfloat16, device="cuda")
    out = torch.full_like(x, 7.0)
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    try:
        _lib.check(lib.nvllm_b200_allreduce_sum(x.data_ptr(), out.data_ptr(), None, ptrs, 0, world, count, max_bytes, 1,
                                                2000, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert _lib.device_status() & 64
        assert bool((out == 7.0).all()), "nothing may be reduced from a peer that never delivered"
        assert float((x * 2).sum()) == 2.0 * count  # the context is alive
    finally:
        _lib.device_status_reset()
    assert _lib.device_status() == 0
