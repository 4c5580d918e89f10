"""torch-CPU restatement of the reference's jnp path, op for op, for the timed CPU baseline.

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.  PARITY UNPINNED (same reason).

The NumPy module next to this one is the checker; this one exists because the reference runs its
jnp code through XLA, which uses every host core, and torch's CPU operators do too.  It keeps the
reference's op sequence -- including the padded gather of all ``max_blocks`` pages, the GQA
``repeat`` and the fp32 widening (layers/pallas_attention.py:185-238) -- so its cost is the cost of
the reference's algorithm, not of a cleverer one.  The CPU test-suite checks it against the NumPy
oracle.
"""
from __future__ import annotations

import torch


def store_kv_to_cache(key, value, k_cache, v_cache, slot_mapping):
    """layers/attention.py:63-77 on torch CPU tensors; returns updated copies (functional, like the original)."""
    valid = slot_mapping >= 0
    safe = torch.where(valid, slot_mapping, torch.zeros_like(slot_mapping)).long()
    keep = safe < k_cache.shape[0]
    key = key.to(k_cache.dtype)
    value = value.to(v_cache.dtype)
    k_cache = k_cache.clone()
    v_cache = v_cache.clone()
    k_cache[safe[keep]] = key[keep]
    v_cache[safe[keep]] = value[keep]
    return k_cache, v_cache


def paged_decode_attention_vectorized(q, k_cache, v_cache, block_tables, context_lens, scale, block_size):
    """layers/pallas_attention.py:176-238 with torch CPU ops; q/k_cache/v_cache may be bf16 or fp32."""
    batch, num_heads, head_dim = q.shape
    nb, _, num_kv_heads, _ = k_cache.shape
    max_blocks = block_tables.shape[1]
    max_ctx = max_blocks * block_size
    g = num_heads // num_kv_heads
    safe = block_tables.long().clamp(0, nb - 1)                                    # :185
    k_flat = k_cache[safe].reshape(batch, max_ctx, num_kv_heads, head_dim)         # :188-192
    v_flat = v_cache[safe].reshape(batch, max_ctx, num_kv_heads, head_dim)
    k_exp = k_flat.repeat_interleave(g, dim=2)                                     # :197
    v_exp = v_flat.repeat_interleave(g, dim=2)                                     # :198
    q32, k32, v32 = q.float(), k_exp.float(), v_exp.float()                        # :201-203
    k_t = k32.permute(0, 2, 1, 3)                                                  # :209
    scores = torch.matmul(q32[:, :, None, :], k_t.transpose(-1, -2)) * scale       # :212
    scores = scores.squeeze(2)                                                     # :213
    mask = torch.arange(max_ctx)[None, None, :] < context_lens.long()[:, None, None]   # :216-217
    scores = torch.where(mask, scores, torch.tensor(-1e9, dtype=torch.float32))    # :220
    smax = scores.max(dim=-1, keepdim=True).values                                 # :223
    e = torch.exp(scores - smax)                                                   # :224
    e = torch.where(mask, e, torch.zeros((), dtype=torch.float32))                 # :225
    w = e / (e.sum(dim=-1, keepdim=True) + 1e-9)                                   # :226-227
    v_t = v32.permute(0, 2, 1, 3)                                                  # :232
    out = (w[:, :, :, None] * v_t).sum(dim=2)                                      # :236
    return out.to(q.dtype)                                                         # :238


def variable_length_attention_prefill(q, k, v, cu_seqlens, num_heads, num_kv_heads, scale):
    """layers/attention.py:165-279 per sequence (no [B,1,S,S] mask), fp32 math, GQA by kv-head broadcast."""
    total, h, d = q.shape
    g = num_heads // num_kv_heads
    out = torch.zeros_like(q)
    cu = [int(x) for x in cu_seqlens]
    for b in range(len(cu) - 1):
        s0, s1 = cu[b], cu[b + 1]
        n = s1 - s0
        if n <= 0:
            continue
        qb = q[s0:s1].float().view(n, num_kv_heads, g, d).permute(1, 2, 0, 3)      # [KVH, G, n, d]
        kb = k[s0:s1].float().permute(1, 0, 2)[:, None]                             # [KVH, 1, n, d]
        vb = v[s0:s1].float().permute(1, 0, 2)[:, None]
        s = torch.matmul(qb, kb.transpose(-1, -2)) * scale
        causal = torch.ones(n, n, dtype=torch.bool).tril()
        s = s.masked_fill(~causal, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.matmul(p, vb)                                                     # [KVH, G, n, d]
        out[s0:s1] = o.permute(2, 0, 1, 3).reshape(n, h, d).to(q.dtype)
    return out
