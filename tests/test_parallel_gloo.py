"""World-size-2 (and 4) gloo runs on CPU of the head-parallel host logic: each rank takes its kv-head shard,
computes attention on it (with the CPU oracle standing in for the kernels, which need a GPU), and the gathered
result must equal the unsharded answer; the o_proj partial sums must all-reduce to the full product."""
import math
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nanovllm_jax_b200 import parallel, workloads
        from oracle import reference_attention as ref
        w = workloads.make_decode_workload("gloo", seed=31, batch=5, num_heads=16, num_kv_heads=4, num_blocks=24,
                                           block_size=64, ctx_lo=1, ctx_hi=300, max_blocks=5)
        t = workloads.decode_tensors_numpy(w)
        full = ref.paged_decode_attention_vectorized(t["q"], t["k_cache"], t["v_cache"], w.block_tables, w.context_lens,
                                                     w.scale, w.block_size)
        sh = parallel.head_shard(rank, world, w.num_heads, w.num_kv_heads)
        q = parallel.shard_heads(torch.from_numpy(t["q"]), sh.q_lo, sh.q_hi)
        kc = parallel.shard_heads(torch.from_numpy(t["k_cache"]), sh.kv_lo, sh.kv_hi)
        vc = parallel.shard_heads(torch.from_numpy(t["v_cache"]), sh.kv_lo, sh.kv_hi)
        local = ref.paged_decode_attention_vectorized(q.numpy(), kc.numpy(), vc.numpy(), w.block_tables, w.context_lens,
                                                      w.scale, w.block_size)
        gathered = parallel.gather_heads(torch.from_numpy(local)).numpy()
        ok_attn = np.allclose(gathered, full, atol=1e-6, rtol=1e-6)
        # row-parallel o_proj: each rank multiplies its head slice, the sum over ranks is the full product
        rng = np.random.Generator(np.random.PCG64(5))
        wo = rng.standard_normal((w.num_heads * 128, 64)).astype(np.float32)
        part = torch.from_numpy(local.reshape(w.batch, -1) @ wo[sh.q_lo * 128:sh.q_hi * 128])
        total = parallel.all_reduce_sum(part).numpy()
        ok_proj = np.allclose(total, full.reshape(w.batch, -1) @ wo, atol=1e-3, rtol=1e-4)
        ret[rank] = (bool(ok_attn), bool(ok_proj), sh.num_heads, sh.num_kv_heads)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_head_shards_gather_to_unsharded_result(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29610 + world
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        ok_attn, ok_proj, h, kvh = ret[r]
        assert ok_attn and ok_proj and h == 16 // world and kvh == 4 // world


def test_head_shard_arithmetic():
    from nanovllm_jax_b200 import parallel
    s = parallel.head_shard(3, 4, 32, 8)
    assert (s.q_lo, s.q_hi, s.kv_lo, s.kv_hi) == (24, 32, 6, 8)
    covered = [parallel.head_shard(r, 8, 64, 8) for r in range(8)]
    assert [c.kv_lo for c in covered] == list(range(8)) and covered[-1].q_hi == 64
    for c in covered:  # every q head of a shard reads a kv head of the same shard
        assert all(c.kv_lo <= h // 8 < c.kv_hi for h in range(c.q_lo, c.q_hi))
    with pytest.raises(ValueError):
        parallel.head_shard(0, 3, 32, 8)
    with pytest.raises(ValueError):
        parallel.head_shard(8, 8, 64, 8)
