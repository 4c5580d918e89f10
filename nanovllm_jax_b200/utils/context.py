"""AttentionContext: the per-step metadata handed to the attention layer.

Field names, meanings and the two builders mirror the reference's utils/context.py:35-190 so that
code written against it (engine/model_runner.py:323-330, 370-374) needs no change.  The arrays here
are torch int32 tensors on the attention device (the reference holds jnp arrays); the three static
fields are plain Python values.  The JAX PyTree registration of the reference (:88-126) lives with the
jax.ffi glue, which keeps the reference's own class.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional


def _bucket_to_power_of_2(value: int, min_bucket: int = 16, max_bucket: int = 8192) -> int:
    """Round up to a power of two within [min_bucket, max_bucket] (reference utils/context.py:18-32).

    The reference needs this to limit XLA recompilation; the CUDA kernels here take the lengths at run
    time, so the bucketed value only serves as an upper bound for grid sizing.
    """
    if value <= min_bucket:
        return min_bucket
    if value >= max_bucket:
        return max_bucket
    return min(1 << (int(value) - 1).bit_length(), max_bucket)


@dataclasses.dataclass
class AttentionContext:
    is_prefill: bool = False
    # prefill: packed variable-length sequences
    cu_seqlens_q: Optional[Any] = None   # [num_seqs + 1] int32
    cu_seqlens_k: Optional[Any] = None   # [num_seqs + 1] int32
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    # decode: one token per sequence
    context_lens: Optional[Any] = None   # [batch] int32, counts the token stored this step
    # shared
    slot_mapping: Optional[Any] = None   # [num_tokens] int32 flat cache slot; negative = do not store
    block_tables: Optional[Any] = None   # [batch, max_blocks] int32, -1 padded
    last_token_indices: Optional[Any] = None  # [batch] index of each sequence's last token (LM head)
    # Optional host copy of cu_seqlens_q (numpy / CPU tensor).  Not in the reference; when present the
    # prefill kernel sizes its grid exactly instead of from max_seqlen_q.
    cu_seqlens_host: Optional[Any] = None


def create_prefill_context(cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, slot_mapping,
                           block_tables=None, cu_seqlens_host=None) -> AttentionContext:
    """Reference utils/context.py:129-166."""
    return AttentionContext(
        is_prefill=True,
        cu_seqlens_q=cu_seqlens_q,
        cu_seqlens_k=cu_seqlens_k,
        max_seqlen_q=_bucket_to_power_of_2(max_seqlen_q),
        max_seqlen_k=_bucket_to_power_of_2(max_seqlen_k),
        slot_mapping=slot_mapping,
        block_tables=block_tables,
        last_token_indices=cu_seqlens_q[1:] - 1,
        cu_seqlens_host=cu_seqlens_host,
    )


def create_decode_context(context_lens, slot_mapping, block_tables) -> AttentionContext:
    """Reference utils/context.py:169-190."""
    return AttentionContext(is_prefill=False, context_lens=context_lens, slot_mapping=slot_mapping,
                            block_tables=block_tables, last_token_indices=None)
