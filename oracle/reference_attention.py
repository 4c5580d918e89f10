"""NumPy restatement of the reference's jnp attention path (fp32 math).

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.  PARITY UNPINNED (no
golden vectors exist in the reference; JAX is not importable here).

Each function names the reference lines it follows (paths are relative to the
reference project root):

* ``store_kv_to_cache``                   <- layers/attention.py:42-77
* ``paged_decode_attention_vectorized``   <- layers/pallas_attention.py:146-238
* ``paged_decode_attention_streamed``     same arithmetic, one sequence at a time
* ``variable_length_attention_prefill``   <- layers/attention.py:135-279
* ``make_decode_metadata`` / ``make_prefill_slot_mapping``
                                          <- engine/model_runner.py:225-246,
                                             300-309, 357-361

bf16 values are carried as ``uint16`` bit patterns (NumPy has no bfloat16);
``f32_to_bf16_bits`` rounds to nearest-even exactly like an XLA ``convert``.
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------
# bf16 <-> fp32 bit conversions
# --------------------------------------------------------------------------


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round fp32 to bf16 (round-to-nearest-even); returns uint16 bit patterns.

    NaN inputs map to a quiet NaN that keeps the sign bit, which is what both
    XLA's convert and CUDA's ``__float2bfloat16_rn`` produce for canonical NaNs.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    r = ((u + bias) >> np.uint32(16)).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, ((u >> np.uint32(16)).astype(np.uint16) | np.uint16(0x0040)), r)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    """Exact widening of bf16 bit patterns (uint16) to fp32."""
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 -> fp32 (the value a bf16 tensor would hold)."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# --------------------------------------------------------------------------
# K1: store_kv_to_cache   (layers/attention.py:42-77)
# --------------------------------------------------------------------------


def store_kv_to_cache(key, value, k_cache, v_cache, slot_mapping, *, skip_negative=False):
    """Scatter new K/V rows into the flat paged cache.

    key, value : [T, KVH, D] fp32 (values to be cast) or uint16 (bf16 bits).
    k_cache, v_cache : [num_slots, KVH, D] uint16 bf16 bit patterns; NOT
        modified -- updated copies are returned, like the functional original.
    slot_mapping : [T] int32.

    ``skip_negative=False`` reproduces the code as written
    (layers/attention.py:64-75): a negative slot is replaced by slot 0 and the
    row IS written there; only indices >= num_slots are dropped
    (``mode='drop'``).  ``skip_negative=True`` is the behaviour the docstring
    promises (layers/attention.py:57-58, "-1 indicates skip"), which the CUDA
    kernel implements.  The two agree whenever no slot is negative, which is
    all the model runner ever produces (engine/model_runner.py:300-309,361).
    """
    slot_mapping = np.asarray(slot_mapping, dtype=np.int64)
    kb = key if key.dtype == np.uint16 else f32_to_bf16_bits(key)  # :70
    vb = value if value.dtype == np.uint16 else f32_to_bf16_bits(value)  # :71
    k_out = np.array(k_cache, dtype=np.uint16, copy=True)
    v_out = np.array(v_cache, dtype=np.uint16, copy=True)
    num_slots = k_out.shape[0]
    valid = slot_mapping >= 0  # :64
    safe = np.where(valid, slot_mapping, 0)  # :67
    keep = safe < num_slots  # mode='drop' :74-75
    if skip_negative:
        keep &= valid
    idx = np.nonzero(keep)[0]
    # Sequential assignment: with unique slots (guaranteed by the block
    # manager) order is irrelevant; with duplicates the last writer wins here,
    # whereas XLA leaves the winner unspecified.
    k_out[safe[idx]] = kb[idx]
    v_out[safe[idx]] = vb[idx]
    return k_out, v_out


# --------------------------------------------------------------------------
# K2: paged decode attention   (layers/pallas_attention.py:146-238)
# --------------------------------------------------------------------------


def paged_decode_attention_vectorized(q, k_cache, v_cache, block_tables, context_lens, scale, block_size):
    """Line-by-line fp32 restatement; materialises [B, MB*blk, H, D] like the original.

    q : [B, H, D] fp32.  k_cache, v_cache : [NB, blk, KVH, D] fp32.
    block_tables : [B, MB] int32 (-1 padded).  context_lens : [B] int32.
    Returns fp32 [B, H, D] BEFORE the final cast to q.dtype (:238); apply
    ``round_to_bf16`` to obtain what a bf16 caller would see.
    Only for small cases: memory is B*MB*blk*H*D*4 bytes several times over.
    """
    q = np.asarray(q, dtype=np.float32)
    k_cache = np.asarray(k_cache, dtype=np.float32)
    v_cache = np.asarray(v_cache, dtype=np.float32)
    block_tables = np.asarray(block_tables, dtype=np.int64)
    context_lens = np.asarray(context_lens, dtype=np.int64)
    batch, num_heads, head_dim = q.shape  # :176
    nb, blk, num_kv_heads, _ = k_cache.shape  # :177
    assert blk == block_size
    max_blocks = block_tables.shape[1]
    max_ctx = max_blocks * block_size  # :179
    g = num_heads // num_kv_heads  # :182
    safe = np.clip(block_tables, 0, nb - 1)  # :185
    k_flat = k_cache[safe].reshape(batch, max_ctx, num_kv_heads, head_dim)  # :188-192
    v_flat = v_cache[safe].reshape(batch, max_ctx, num_kv_heads, head_dim)
    k_exp = np.repeat(k_flat, g, axis=2)  # :197
    v_exp = np.repeat(v_flat, g, axis=2)  # :198
    k_t = np.transpose(k_exp, (0, 2, 1, 3))  # [B,H,S,D] :209
    scores = np.matmul(q[:, :, None, :], np.transpose(k_t, (0, 1, 3, 2))) * np.float32(scale)  # :212
    scores = scores[:, :, 0, :]  # :213
    positions = np.arange(max_ctx)[None, None, :]  # :216
    mask = positions < context_lens[:, None, None]  # :217
    scores = np.where(mask, scores, np.float32(-1e9))  # :220
    smax = scores.max(axis=-1, keepdims=True)  # :223
    e = np.exp(scores - smax)  # :224
    e = np.where(mask, e, np.float32(0.0))  # :225
    ssum = e.sum(axis=-1, keepdims=True, dtype=np.float32)  # :226
    w = e / (ssum + np.float32(1e-9))  # :227
    v_t = np.transpose(v_exp, (0, 2, 1, 3))  # :232
    out = (w[:, :, :, None] * v_t).sum(axis=2, dtype=np.float32)  # :236
    return out.astype(np.float32)


def paged_decode_attention_streamed(q, k_cache, v_cache, block_tables, context_lens, scale, block_size, *, kv_dtype_bits=False):
    """Same arithmetic as ``paged_decode_attention_vectorized`` one sequence at a time.

    Gathers only the ``ceil(ctx/blk)`` live pages of each sequence (masked
    positions contribute exactly 0 to every sum in the original, so dropping
    them changes nothing), never builds the GQA-repeated tensors, and accepts
    the caches as bf16 bit patterns (``kv_dtype_bits=True``) so multi-GB caches
    need not be widened at once.  Used for the large workloads.
    """
    q = np.asarray(q, dtype=np.float32)
    block_tables = np.asarray(block_tables, dtype=np.int64)
    context_lens = np.asarray(context_lens, dtype=np.int64)
    batch, num_heads, head_dim = q.shape
    nb, blk, num_kv_heads, _ = k_cache.shape
    assert blk == block_size
    g = num_heads // num_kv_heads
    max_ctx = block_tables.shape[1] * block_size
    out = np.zeros((batch, num_heads, head_dim), dtype=np.float32)
    for b in range(batch):
        ctx = int(min(max(int(context_lens[b]), 0), max_ctx))
        if ctx == 0:
            continue  # all masked: 0 / (0 + 1e-9) = 0   (:225-227)
        nblk = -(-ctx // block_size)
        ids = np.clip(block_tables[b, :nblk], 0, nb - 1)
        kb = k_cache[ids].reshape(nblk * block_size, num_kv_heads, head_dim)[:ctx]
        vb = v_cache[ids].reshape(nblk * block_size, num_kv_heads, head_dim)[:ctx]
        if kv_dtype_bits:
            kb = bf16_bits_to_f32(kb)
            vb = bf16_bits_to_f32(vb)
        else:
            kb = kb.astype(np.float32, copy=False)
            vb = vb.astype(np.float32, copy=False)
        qb = q[b].reshape(num_kv_heads, g, head_dim)
        # scores[kvh, g, s] = q . k * scale
        s = np.einsum("hgd,shd->hgs", qb, kb, optimize=True).astype(np.float32) * np.float32(scale)
        smax = s.max(axis=-1, keepdims=True)
        e = np.exp(s - smax)
        ssum = e.sum(axis=-1, keepdims=True, dtype=np.float32)
        w = e / (ssum + np.float32(1e-9))
        o = np.einsum("hgs,shd->hgd", w, vb, optimize=True)
        out[b] = o.reshape(num_heads, head_dim)
    return out


# --------------------------------------------------------------------------
# K9: varlen causal prefill   (layers/attention.py:135-279)
# --------------------------------------------------------------------------


def variable_length_attention_prefill(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                      num_heads, num_kv_heads, scale, batch_size):
    """fp32 restatement computed per sequence instead of on the padded batch.

    q : [T, H, D], k, v : [Tk, KVH, D] fp32; returns fp32 [T, H, D] before the
    cast back to q.dtype.

    Semantics kept from the padded original:
    * causal mask on positions RELATIVE to each sequence, q_pos >= k_pos
      (:232-236), so with len_k > len_q the extra keys are simply never
      attended by early queries -- the original is only meaningful for
      cu_seqlens_q == cu_seqlens_k, which is what every test uses;
    * rows at positions >= max_seqlen_q (the pow-2 bucket capped at 8192,
      utils/context.py:18-32) are never gathered (:203-228) and come back as
      zeros (:272-277); keys at positions >= max_seqlen_k are never seen;
    * GQA: query head n reads kv head n // (H/KVH) (jax.nn.dot_product_attention
      grouping);
    * the single-sequence fast path (:172-191) is the same arithmetic without
      truncation.
    """
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    cu_q = np.asarray(cu_seqlens_q, dtype=np.int64)
    cu_k = np.asarray(cu_seqlens_k, dtype=np.int64)
    total, h, d = q.shape
    assert h == num_heads and k.shape[1] == num_kv_heads
    g = num_heads // num_kv_heads
    out = np.zeros_like(q)
    for b in range(batch_size):
        q0, q1 = int(cu_q[b]), int(cu_q[b + 1])
        k0, k1 = int(cu_k[b]), int(cu_k[b + 1])
        lq, lk = q1 - q0, k1 - k0
        if batch_size > 1:
            lq = min(lq, max_seqlen_q)
            lk = min(lk, max_seqlen_k)
        if lq <= 0:
            continue
        qb = q[q0:q0 + lq].reshape(lq, num_kv_heads, g, d)
        kb = k[k0:k0 + lk]
        vb = v[k0:k0 + lk]
        causal = np.arange(lq)[:, None] >= np.arange(lk)[None, :]
        for kh in range(num_kv_heads):
            s = np.einsum("qgd,sd->gqs", qb[:, kh], kb[:, kh], optimize=True).astype(np.float32) * np.float32(scale)
            s = np.where(causal[None], s, np.float32(-np.inf))
            smax = s.max(axis=-1, keepdims=True)
            e = np.exp(s - smax)
            w = e / e.sum(axis=-1, keepdims=True, dtype=np.float32)
            o = np.einsum("gqs,sd->qgd", w, vb[:, kh], optimize=True)
            out[q0:q0 + lq, kh * g:(kh + 1) * g] = o
    return out


# --------------------------------------------------------------------------
# Pre-attention step: per-head RMSNorm of q and k, rotary embedding
# (models/qwen3.py:157-163, layers/layernorm.py:31-48, layers/rotary_embedding.py:13-37,97-104)
# --------------------------------------------------------------------------


def rope_cos_sin_cache(head_dim, max_position, base):
    """The reference's table (layers/rotary_embedding.py:57-75): [max_pos, head_dim] fp32, cos(half) | sin(half)."""
    inv_freq = (np.float32(1.0) / (np.float32(base) ** (np.arange(0, head_dim, 2, dtype=np.float32) / np.float32(head_dim))))
    t = np.arange(max_position, dtype=np.float32)
    freqs = (t[:, None] * inv_freq[None, :]).astype(np.float32)
    return np.concatenate([np.cos(freqs), np.sin(freqs)], axis=-1).astype(np.float32)


def _sum_of_squares_fixed_order(x):
    """fp32 sum of squares over the last axis (128 elements) in ONE stated order: eight consecutive elements left to
    right, then a butterfly over the sixteen groups (partner distance 8, 4, 2, 1).  The reference leaves the order to
    XLA's reduction (jnp.mean, layers/layernorm.py:43); fixing one makes the bf16 results reproducible bit for bit."""
    sq = (x * x).astype(np.float32).reshape(*x.shape[:-1], 16, 8)
    part = sq[..., 0]
    for i in range(1, 8):
        part = (part + sq[..., i]).astype(np.float32)
    idx = np.arange(16)
    for o in (8, 4, 2, 1):
        part = (part + part[..., idx ^ o]).astype(np.float32)
    return part[..., 0]


def rms_norm_heads(x_bits, weight, eps):
    """RMSNorm over head_dim of bf16 rows (layers/layernorm.py:41-48): fp32 math, (x * rsqrt(mean(x^2) + eps)) * weight,
    cast back to bf16.  Returns bf16 bit patterns."""
    x = bf16_bits_to_f32(x_bits)
    var = (_sum_of_squares_fixed_order(x) * np.float32(1.0 / x.shape[-1])).astype(np.float32)  # :43
    inv = (np.float32(1.0) / np.sqrt((var + np.float32(eps)).astype(np.float32))).astype(np.float32)  # :44
    y = ((x * inv[..., None]).astype(np.float32) * np.asarray(weight, np.float32)).astype(np.float32)  # :44, :47
    return f32_to_bf16_bits(y)


def apply_rotary_emb(x_bits, cos, sin):
    """layers/rotary_embedding.py:31-37 on bf16 rows with the fp32 table: halves split at head_dim / 2, products and
    sums in fp32 (bf16 * fp32 promotes), result cast to bf16 where it is consumed (the cache dtype,
    layers/attention.py:70-71; q at :386-387).  x_bits [T, heads, D]; cos, sin [T, D/2]."""
    x = bf16_bits_to_f32(x_bits)
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :].astype(np.float32), sin[:, None, :].astype(np.float32)
    y1 = ((x1 * c).astype(np.float32) - (x2 * s).astype(np.float32)).astype(np.float32)
    y2 = ((x2 * c).astype(np.float32) + (x1 * s).astype(np.float32)).astype(np.float32)
    return f32_to_bf16_bits(np.concatenate([y1, y2], axis=-1))


def qk_norm_rope(q_bits, k_bits, q_weight, k_weight, cos_sin_cache, positions, eps):
    """models/qwen3.py:157-163: q_norm, k_norm, then rotary_emb(positions, q, k).  Returns (q, k) bf16 bit patterns."""
    pos = np.clip(np.asarray(positions, np.int64), 0, cos_sin_cache.shape[0] - 1)
    half = cos_sin_cache.shape[1] // 2
    cos, sin = cos_sin_cache[pos, :half], cos_sin_cache[pos, half:]  # layers/rotary_embedding.py:98-101
    qn = rms_norm_heads(q_bits, q_weight, eps)
    kn = rms_norm_heads(k_bits, k_weight, eps)
    return apply_rotary_emb(qn, cos, sin), apply_rotary_emb(kn, cos, sin)


# --------------------------------------------------------------------------
# Prefix-cached prefill: the definition the reference's metadata implies
# --------------------------------------------------------------------------


def prefix_cached_prefill_attention(q, k_cache, v_cache, block_tables, cu_seqlens_q, cu_seqlens_k, scale, block_size):
    """Causal attention of new query tokens over a sequence whose first tokens are already cached.

    The reference has NO correct function to restate for this case: on a prefix-cache hit its model runner emits
    cu_seqlens_k > cu_seqlens_q and attaches block tables (engine/model_runner.py:286-292, 311-314), but
    Attention._prefill_attention ignores the tables (layers/attention.py:351-364) and masks with positions relative to
    the new tokens (:232-236), which attends the wrong keys.  This function is therefore derived, not restated:
      * the keys/values of sequence b are the first len_k = cu_k[b+1]-cu_k[b] tokens of the pages block_tables[b, :]
        (the layout the model runner builds, engine/model_runner.py:300-314; the step's new K/V rows have been
        stored first, as Attention.__call__ does at layers/attention.py:465-467);
      * its len_q = cu_q[b+1]-cu_q[b] queries are the LAST len_q of those positions: query i sits at absolute
        position prefix + i with prefix = len_k - len_q (engine/model_runner.py:286-292: the uncached suffix);
      * query at position p attends keys 0..p, fp32 softmax, same GQA grouping as the decode path
        (layers/pallas_attention.py:197-198).
    With prefix = 0 it equals variable_length_attention_prefill on the same keys.

    q : [T, H, D] fp32; k_cache, v_cache : [NB, blk, KVH, D] fp32; returns fp32 [T, H, D].
    """
    q = np.asarray(q, dtype=np.float32)
    cu_q = np.asarray(cu_seqlens_q, dtype=np.int64)
    cu_k = np.asarray(cu_seqlens_k, dtype=np.int64)
    total, h, d = q.shape
    kvh = k_cache.shape[2]
    g = h // kvh
    out = np.zeros_like(q)
    for b in range(len(cu_q) - 1):
        q0, lq = int(cu_q[b]), int(cu_q[b + 1] - cu_q[b])
        lk = int(cu_k[b + 1] - cu_k[b])
        if lq <= 0:
            continue
        assert lk >= lq, "a sequence cannot have fewer keys than queries"
        prefix = lk - lq
        nblk = -(-lk // block_size)
        pages = np.asarray(block_tables[b][:nblk], dtype=np.int64)
        kb = np.asarray(k_cache[pages], dtype=np.float32).reshape(nblk * block_size, kvh, d)[:lk]
        vb = np.asarray(v_cache[pages], dtype=np.float32).reshape(nblk * block_size, kvh, d)[:lk]
        qb = q[q0:q0 + lq].reshape(lq, kvh, g, d)
        causal = (prefix + np.arange(lq))[:, None] >= np.arange(lk)[None, :]
        for kh in range(kvh):
            s = np.einsum("qgd,sd->gqs", qb[:, kh], kb[:, kh], optimize=True).astype(np.float32) * np.float32(scale)
            s = np.where(causal[None], s, np.float32(-np.inf))
            smax = s.max(axis=-1, keepdims=True)
            e = np.exp(s - smax)
            w = e / e.sum(axis=-1, keepdims=True, dtype=np.float32)
            out[q0:q0 + lq, kh * g:(kh + 1) * g] = np.einsum("gqs,sd->qgd", w, vb[:, kh], optimize=True)
    return out


# --------------------------------------------------------------------------
# Metadata exactly as the model runner builds it
# --------------------------------------------------------------------------


def pad_block_tables(block_lists):
    """engine/model_runner.py:225-246 -- ragged block lists -> [B, MB] int32, -1 padded."""
    mb = max(len(b) for b in block_lists)
    out = np.full((len(block_lists), mb), -1, dtype=np.int32)
    for i, bl in enumerate(block_lists):
        out[i, : len(bl)] = bl
    return out


def decode_slot_mapping(block_lists, context_lens, block_size):
    """engine/model_runner.py:357-361 -- slot of the newest token of each sequence."""
    slots = np.empty(len(block_lists), dtype=np.int32)
    for i, (bl, n) in enumerate(zip(block_lists, context_lens)):
        last_block_tokens = n - (len(bl) - 1) * block_size
        slots[i] = bl[-1] * block_size + last_block_tokens - 1
    return slots


def prefill_slot_mapping(block_lists, seq_lens, block_size):
    """engine/model_runner.py:300-309 -- slots of every prompt token, sequence after sequence."""
    parts = []
    for bl, n in zip(block_lists, seq_lens):
        nblk = -(-n // block_size)
        for i in range(nblk):
            start = bl[i] * block_size
            ln = block_size if i != nblk - 1 else n - (nblk - 1) * block_size
            parts.append(np.arange(start, start + ln, dtype=np.int32))
    return np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32)
