"""Seeded synthetic workloads for the attention hot path.

The shapes, length distributions and paging follow the five benchmark
configurations of this project (Qwen3-0.6B / 8B / 32B attention shapes, KV
block size 256).  Metadata (context lengths, block tables, slot mappings,
cu_seqlens) is always built on the host with ``numpy.random.Generator(PCG64)``
exactly the way the reference's model runner builds it
(engine/model_runner.py:225-246, 300-309, 357-361); tensors are N(0,1) draws
rounded to bf16, produced either with NumPy (small cases, bit-reproducible on
any machine) or directly on a CUDA device with a seeded torch generator (large
cases, where a host-side draw of several GB would dominate the run).

Seeds: ``1000 * config + trial``.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np


@dataclasses.dataclass
class DecodeWorkload:
    name: str
    batch: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    block_size: int
    num_blocks: int
    context_lens: np.ndarray  # [B] int32, already counts the token stored this step
    block_lists: list  # ragged physical block ids per sequence
    block_tables: np.ndarray  # [B, MB] int32, -1 padded
    slot_mapping: np.ndarray  # [B] int32, slot of the newest token
    scale: float
    seed: int

    @property
    def max_blocks(self) -> int:
        return int(self.block_tables.shape[1])

    def kv_bytes(self, num_kv_heads: int | None = None) -> int:
        """Algorithmic HBM bytes of one decode-attention call.

        sum_b ctx_b * KVH * D * 2 (K and V) * 2 B  +  q and out (B*H*D*2 B each)
        + the int32 metadata actually dereferenced.  Split-K scratch traffic is
        deliberately not counted.
        """
        kvh = self.num_kv_heads if num_kv_heads is None else num_kv_heads
        h = self.num_heads * kvh // self.num_kv_heads
        ctx = int(self.context_lens.astype(np.int64).sum())
        used_blocks = int(sum(-(-int(c) // self.block_size) for c in self.context_lens))
        return (ctx * kvh * self.head_dim * 2 * 2
                + 2 * self.batch * h * self.head_dim * 2
                + 4 * (used_blocks + self.batch))


@dataclasses.dataclass
class PrefillWorkload:
    name: str
    num_heads: int
    num_kv_heads: int
    head_dim: int
    block_size: int
    num_blocks: int
    seq_lens: np.ndarray  # [B]
    cu_seqlens: np.ndarray  # [B+1] int32 (q and k identical)
    block_lists: list
    slot_mapping: np.ndarray  # [T] int32
    scale: float
    seed: int

    @property
    def batch(self) -> int:
        return int(len(self.seq_lens))

    @property
    def total_tokens(self) -> int:
        return int(self.cu_seqlens[-1])

    def flops(self, num_heads: int | None = None) -> int:
        """Causal QK^T + PV flops: 4 * D * H * sum_b L_b (L_b + 1) / 2 (softmax excluded)."""
        h = self.num_heads if num_heads is None else num_heads
        l = self.seq_lens.astype(np.int64)
        return int(4 * self.head_dim * h * int((l * (l + 1) // 2).sum()))

    def store_bytes(self, num_kv_heads: int | None = None) -> int:
        """store_kvcache bytes: T * KVH * D * 2 B * 2 tensors * (read + write) + 4 T."""
        kvh = self.num_kv_heads if num_kv_heads is None else num_kv_heads
        return self.total_tokens * (kvh * self.head_dim * 2 * 2 * 2 + 4)


def _deal_blocks(rng: np.random.Generator, num_blocks: int, need_per_seq):
    """Non-overlapping random physical blocks: one permutation of the pool dealt in order."""
    total = int(sum(need_per_seq))
    if total > num_blocks:
        raise ValueError(f"pool of {num_blocks} blocks cannot hold {total}")
    perm = rng.permutation(num_blocks).astype(np.int32)
    lists, pos = [], 0
    for n in need_per_seq:
        lists.append(perm[pos:pos + n].tolist())
        pos += n
    return lists


def _pad_tables(block_lists, max_blocks=None):
    mb = max(len(b) for b in block_lists) if max_blocks is None else max_blocks
    mb = max(mb, 1)
    out = np.full((len(block_lists), mb), -1, dtype=np.int32)
    for i, bl in enumerate(block_lists):
        out[i, : len(bl)] = bl
    return out


def make_decode_workload(name, *, seed, batch, num_heads, num_kv_heads, head_dim=128, block_size=256,
                         num_blocks, ctx_lo, ctx_hi, log_uniform=False, max_blocks=None) -> DecodeWorkload:
    rng = np.random.Generator(np.random.PCG64(seed))
    if log_uniform:
        ctx = np.rint(np.exp(rng.uniform(math.log(ctx_lo), math.log(ctx_hi), size=batch))).astype(np.int32)
        ctx = np.clip(ctx, ctx_lo, ctx_hi)
    else:
        ctx = rng.integers(ctx_lo, ctx_hi + 1, size=batch).astype(np.int32)
    need = [-(-int(c) // block_size) for c in ctx]
    lists = _deal_blocks(rng, num_blocks, need)
    tables = _pad_tables(lists, max_blocks)
    slots = np.array([bl[-1] * block_size + (int(c) - (len(bl) - 1) * block_size) - 1
                      for bl, c in zip(lists, ctx)], dtype=np.int32)
    return DecodeWorkload(name, batch, num_heads, num_kv_heads, head_dim, block_size, num_blocks, ctx, lists,
                          tables, slots, 1.0 / math.sqrt(head_dim), seed)


def make_prefill_workload(name, *, seed, batch, num_heads, num_kv_heads, head_dim=128, block_size=256,
                          len_lo, len_hi, num_blocks=None, seq_lens=None) -> PrefillWorkload:
    rng = np.random.Generator(np.random.PCG64(seed))
    if seq_lens is None:
        lens = rng.integers(len_lo, len_hi + 1, size=batch).astype(np.int32)
    else:
        lens = np.asarray(seq_lens, dtype=np.int32)
    need = [-(-int(n) // block_size) for n in lens]
    if num_blocks is None:
        num_blocks = int(sum(need)) + 8
    lists = _deal_blocks(rng, num_blocks, need)
    cu = np.zeros(len(lens) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(lens)
    parts = []
    for bl, n in zip(lists, lens):
        for i, blk in enumerate(bl):
            ln = block_size if i != len(bl) - 1 else int(n) - (len(bl) - 1) * block_size
            parts.append(np.arange(blk * block_size, blk * block_size + ln, dtype=np.int32))
    slots = np.concatenate(parts) if parts else np.zeros(0, np.int32)
    return PrefillWorkload(name, num_heads, num_kv_heads, head_dim, block_size, num_blocks, lens, cu, lists, slots,
                           1.0 / math.sqrt(head_dim), seed)


# ---- the named configurations -------------------------------------------------


def config1(trial: int = 0) -> DecodeWorkload:
    """Qwen3-0.6B shapes: 16 q heads / 8 kv heads, batch 8, ctx U[64,1024], pool of 64 blocks."""
    return make_decode_workload("cfg1-qwen3-0.6b-b8", seed=1000 + trial, batch=8, num_heads=16, num_kv_heads=8,
                                num_blocks=64, ctx_lo=64, ctx_hi=1024, max_blocks=4)


def config2(trial: int = 0, num_blocks: int = 4096) -> DecodeWorkload:
    """Qwen3-8B shapes: 32 q heads / 8 kv heads, batch 64, ctx U[512,8192], pool of 4096 blocks.

    ``num_blocks`` shrinks the physical pool (same sequences, same lengths) for profiler captures that
    must hold little device memory."""
    return make_decode_workload("cfg2-qwen3-8b-b64", seed=2000 + trial, batch=64, num_heads=32, num_kv_heads=8,
                                num_blocks=num_blocks, ctx_lo=512, ctx_hi=8192, max_blocks=32)


def config3(trial: int = 0, num_blocks: int = 8192) -> DecodeWorkload:
    """Qwen3-32B shapes: 64 q heads / 8 kv heads, batch 256, ctx log-U[16,32768], pool of 8192 blocks."""
    return make_decode_workload("cfg3-qwen3-32b-b256", seed=3000 + trial, batch=256, num_heads=64, num_kv_heads=8,
                                num_blocks=num_blocks, ctx_lo=16, ctx_hi=32768, log_uniform=True, max_blocks=128)


def config4(trial: int = 0) -> PrefillWorkload:
    """Qwen3-8B prefill: 16 packed sequences, L U[128,4096], cu_seqlens_q == cu_seqlens_k."""
    return make_prefill_workload("cfg4-qwen3-8b-prefill16", seed=4000 + trial, batch=16, num_heads=32,
                                 num_kv_heads=8, len_lo=128, len_hi=4096)


# ---- tensors ------------------------------------------------------------------


def normal_bf16_numpy(rng: np.random.Generator, shape):
    """N(0,1) fp32 draws rounded to bf16; returns (fp32 values that are exactly bf16, uint16 bit patterns)."""
    x = rng.standard_normal(size=shape, dtype=np.float32)
    u = x.view(np.uint32)
    bits = ((u + (((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF))) >> np.uint32(16)).astype(np.uint16)
    vals = (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)
    return vals, bits


def decode_tensors_numpy(w: DecodeWorkload):
    """q, new k/v, and both caches as bf16 bit patterns (uint16) + fp32 views, all from the workload seed."""
    rng = np.random.Generator(np.random.PCG64(w.seed + 500))
    out = {}
    for name, shape in (("q", (w.batch, w.num_heads, w.head_dim)),
                        ("k_new", (w.batch, w.num_kv_heads, w.head_dim)),
                        ("v_new", (w.batch, w.num_kv_heads, w.head_dim)),
                        ("k_cache", (w.num_blocks, w.block_size, w.num_kv_heads, w.head_dim)),
                        ("v_cache", (w.num_blocks, w.block_size, w.num_kv_heads, w.head_dim))):
        vals, bits = normal_bf16_numpy(rng, shape)
        out[name] = vals
        out[name + "_bits"] = bits
    return out


def prefill_tensors_numpy(w: PrefillWorkload):
    rng = np.random.Generator(np.random.PCG64(w.seed + 500))
    out = {}
    t = w.total_tokens
    for name, shape in (("q", (t, w.num_heads, w.head_dim)),
                        ("k", (t, w.num_kv_heads, w.head_dim)),
                        ("v", (t, w.num_kv_heads, w.head_dim))):
        vals, bits = normal_bf16_numpy(rng, shape)
        out[name] = vals
        out[name + "_bits"] = bits
    return out
