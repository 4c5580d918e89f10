"""Head-parallel sharding of the attention path across the GPUs of one node.

The reference splits attention by KV head (QKVParallelLinear.load_weights, layers/linear.py:339-381; KV cache
sharded on its head axis, engine/model_runner.py:178-188): rank r of tp owns KV heads
[r*KVH/tp, (r+1)*KVH/tp) and the query heads that read them, every index tensor (slot_mapping, block_tables,
context_lens, cu_seqlens) is replicated, and attention itself needs no communication.  The one exchange of the
layer is the sum over ranks after the row-parallel o_proj GEMM (layers/linear.py:497-503), which is outside the
attention path; ``all_reduce_sum`` is that collective over torch.distributed (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

from typing import NamedTuple

import torch
import torch.distributed as dist


class HeadShard(NamedTuple):
    q_lo: int
    q_hi: int
    kv_lo: int
    kv_hi: int

    @property
    def num_heads(self) -> int:
        return self.q_hi - self.q_lo

    @property
    def num_kv_heads(self) -> int:
        return self.kv_hi - self.kv_lo


def head_shard(rank: int, tp: int, num_heads: int, num_kv_heads: int) -> HeadShard:
    """Heads owned by ``rank``.  tp must divide both head counts (the reference asserts tp in [1, 8], config.py:39)."""
    if tp <= 0 or not 0 <= rank < tp:
        raise ValueError(f"rank {rank} outside tensor-parallel size {tp}")
    if num_kv_heads % tp or num_heads % tp or num_heads % num_kv_heads:
        raise ValueError(f"{num_heads} q heads / {num_kv_heads} kv heads cannot be split {tp} ways")
    hq, hk = num_heads // tp, num_kv_heads // tp
    return HeadShard(rank * hq, (rank + 1) * hq, rank * hk, (rank + 1) * hk)


def shard_heads(x: torch.Tensor, lo: int, hi: int, head_dim_index: int = -2) -> torch.Tensor:
    """Contiguous copy of heads [lo, hi) of a [..., heads, head_dim] tensor (q, k, v or a cache)."""
    return x.narrow(head_dim_index if head_dim_index >= 0 else x.dim() + head_dim_index, lo, hi - lo).contiguous()


def gather_heads(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate the ranks' [T, H/tp, D] outputs into [T, H, D] (used by tests; a model feeds the local heads
    straight into its row-parallel o_proj instead)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def all_reduce_sum(x: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over the tensor-parallel group: the collective that follows o_proj / down_proj."""
    dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    return x
