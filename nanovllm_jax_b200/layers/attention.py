"""Attention layer with a paged KV cache -- the reference's call surface over the sm_100a kernels.

Mirrors, name for name, what the model and the model runner of nanovllm_jax touch
(layers/attention.py:31-77, 135-148, 282-480 and layers/pallas_attention.py:465-474, 557-564):

    KVCache, store_kv_to_cache, variable_length_attention_prefill,
    paged_attention, paged_prefill_attention, PALLAS_AVAILABLE,
    Attention(num_heads, head_dim, scale, num_kv_heads, block_size=256)
        .set_kv_cache(k_cache, v_cache)     # [num_blocks, block_size, num_kv_heads, head_dim] bf16
        .__call__(q, k, v, context) -> o    # same shape and dtype as q

Arrays are torch CUDA tensors.  Head counts are per rank, as in the reference
(models/qwen3.py:63-69, 114-120): a tensor-parallel rank constructs the layer with its own
H/tp query heads and KVH/tp kv heads and its own cache shard, and no communication happens here.

Differences from the reference, all deliberate:
  * the caches are updated IN PLACE (the reference donates and rebinds them, :42, :470-475);
    ``store_kv_to_cache`` still returns the pair so call sites read the same;
  * a negative slot is skipped, as documented at :57-58 (the reference code writes slot 0);
  * there is no gather fallback (:399-434): without the CUDA library every call raises;
  * a prefill context that carries block_tables (a prefix-cache hit, engine/model_runner.py:311-314) attends the
    cached prefix too, through the pages; the reference ignores the tables there (:351-364).
"""
from __future__ import annotations

from typing import NamedTuple

import torch

from .. import ops
from ..utils.context import AttentionContext

# The reference exports this flag from its Pallas module (layers/attention.py:21-28); callers test it before
# taking the paged path.  Here the paged kernels are the only path.
PALLAS_AVAILABLE = True


class KVCache(NamedTuple):
    """Per-layer cache pair, each [num_blocks, block_size, num_kv_heads, head_dim] (reference :31-39)."""
    k_cache: torch.Tensor
    v_cache: torch.Tensor


def store_kv_to_cache(key, value, k_cache, v_cache, slot_mapping):
    """Scatter this step's K/V rows into the flat cache [num_slots, KVH, D]; returns (k_cache, v_cache)."""
    ops.store_kvcache(key.contiguous(), value.contiguous(), k_cache, v_cache, slot_mapping)
    return k_cache, v_cache


def paged_attention(q, k_cache, v_cache, block_tables, context_lens, scale: float, block_size: int):
    """Decode attention over the block-table cache (reference layers/pallas_attention.py:465-507)."""
    return ops.paged_decode(q.contiguous(), k_cache, v_cache, block_tables, context_lens, scale, block_size)


def variable_length_attention_prefill(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int,
                                      num_heads: int, num_kv_heads: int, scale: float, batch_size: int,
                                      cu_seqlens_host=None):
    """Causal attention over packed sequences (reference layers/attention.py:135-279)."""
    if q.shape[1] != num_heads or k.shape[1] != num_kv_heads:
        raise ValueError("head counts do not match the tensors")
    if cu_seqlens_q.shape[0] != batch_size + 1:
        raise ValueError("cu_seqlens_q must have batch_size + 1 entries")
    return ops.varlen_prefill(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens_q,
                              max(max_seqlen_q, max_seqlen_k), scale, cu_seqlens_host=cu_seqlens_host,
                              cu_seqlens_k=cu_seqlens_k)


def paged_prefill_attention(q, k, v, cu_seqlens, max_seqlen: int, scale: float):
    """Reference layers/pallas_attention.py:557-608 (cu_seqlens_q == cu_seqlens_k)."""
    return ops.varlen_prefill(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens, max_seqlen, scale)


class Attention:
    """Multi-head attention with a paged KV cache (reference layers/attention.py:282-480)."""

    def __init__(self, num_heads: int, head_dim: int, scale: float, num_kv_heads: int, block_size: int = 256):
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.block_size = block_size
        self.k_cache = None
        self.v_cache = None

    def set_kv_cache(self, k_cache, v_cache):
        """Called by the model runner after it allocates the cache (reference :326-329)."""
        self.k_cache = k_cache
        self.v_cache = v_cache

    def _prefill_attention(self, q, k, v, context: AttentionContext):
        batch_size = context.cu_seqlens_q.shape[0] - 1
        if context.block_tables is not None:
            # Prefix-cache hit: the model runner attaches the tables exactly when cu_seqlens_k > cu_seqlens_q
            # (engine/model_runner.py:311-314).  The reference drops them here (:351-364) and attends the new tokens
            # only; this layer reads the whole sequence, cached prefix included, from the pages (the new tokens'
            # rows were stored by __call__ just before).
            if self.k_cache is None or self.v_cache is None:
                raise RuntimeError("prefill over a cached prefix needs the KV cache: call set_kv_cache first")
            return ops.paged_prefill(q.to(self.k_cache.dtype).contiguous(), self.k_cache, self.v_cache,
                                     context.block_tables, context.cu_seqlens_q, context.cu_seqlens_k,
                                     context.max_seqlen_q, self.scale, self.block_size,
                                     cu_seqlens_host=getattr(context, "cu_seqlens_host", None))
        if context.max_seqlen_k != context.max_seqlen_q:
            raise ValueError("cu_seqlens_k differs from cu_seqlens_q (a cached prefix) but the context carries no "
                             "block_tables to read the prefix from")
        return variable_length_attention_prefill(
            q=q, k=k, v=v, cu_seqlens_q=context.cu_seqlens_q, cu_seqlens_k=context.cu_seqlens_k,
            max_seqlen_q=context.max_seqlen_q, max_seqlen_k=context.max_seqlen_k, num_heads=self.num_heads,
            num_kv_heads=self.num_kv_heads, scale=self.scale, batch_size=batch_size,
            cu_seqlens_host=getattr(context, "cu_seqlens_host", None))

    def _decode_attention(self, q, context: AttentionContext):
        if self.k_cache is None or self.v_cache is None:
            raise RuntimeError("decode attention needs the KV cache: call set_kv_cache first")
        q = q.to(self.k_cache.dtype)  # reference :386-387
        return paged_attention(q=q, k_cache=self.k_cache, v_cache=self.v_cache, block_tables=context.block_tables,
                               context_lens=context.context_lens, scale=self.scale, block_size=self.block_size)

    def __call__(self, q, k, v, context: AttentionContext):
        """q [T, H, D]; k, v [T, KVH, D]; returns [T, H, D].  Stores k/v first, then attends (reference :436-480)."""
        if not context.is_prefill and self.k_cache is not None and self.v_cache is not None:
            # decode: the scatter of the step's K/V rows and the attention over the pages go down as one C call
            # (same result as the two calls of the reference, :465-467 then :476-478)
            return ops.decode_step(q.to(self.k_cache.dtype).contiguous(), k.contiguous(), v.contiguous(),
                                   self.k_cache, self.v_cache, context.slot_mapping, context.block_tables,
                                   context.context_lens, self.scale, self.block_size)
        if self.k_cache is not None and self.v_cache is not None:
            num_blocks = self.k_cache.shape[0]
            flat = (num_blocks * self.block_size, self.num_kv_heads, self.head_dim)
            store_kv_to_cache(k, v, self.k_cache.view(flat), self.v_cache.view(flat), context.slot_mapping)
        if context.is_prefill:
            return self._prefill_attention(q, k, v, context)
        return self._decode_attention(q, context)

    forward = __call__
