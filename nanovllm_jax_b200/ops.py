"""Operators over torch CUDA tensors -> C ABI.  torch is used for device memory and streams only.

Every function validates dtype / device / contiguity, then hands raw device pointers to
libnvllm_b200_attn.so on torch's current stream.  Nothing here computes on the host and nothing
falls back: a missing library or an unsupported shape raises.
"""
from __future__ import annotations

import torch

from . import _lib

_workspaces: dict = {}


def _need(t: torch.Tensor, name: str, dtype, ndim: int | None = None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name} must have {ndim} dims, got shape {tuple(t.shape)}")


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def workspace(device, nbytes: int) -> torch.Tensor:
    """A cached scratch buffer of at least ``nbytes`` on ``device`` (grown on demand, never shrunk).

    One buffer per (device, stream): calls on one stream are ordered, so they may share it.
    """
    key = (torch.device(device).index, _stream_ptr(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor) -> None:
    """In place: ``k_cache.view(-1, KVH, D)[slot_mapping[t]] = key[t]`` (same for value).

    key/value: [T, KVH, D] bf16 or fp32.  Caches: bf16, any leading shape whose flattening is
    [num_slots, KVH, D] (e.g. [NB, block, KVH, D]).  slot_mapping: [T] int32; negative = skip.
    """
    if key.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"key must be bf16 or fp32, got {key.dtype}")
    _need(key, "key", key.dtype, 3)
    _need(value, "value", key.dtype, 3)
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    t, kvh, d = key.shape
    if value.shape != key.shape:
        raise ValueError("key and value shapes differ")
    if slot_mapping.shape[0] != t:
        raise ValueError(f"slot_mapping has {slot_mapping.shape[0]} entries for {t} tokens")
    if k_cache.shape != v_cache.shape or tuple(k_cache.shape[-2:]) != (kvh, d):
        raise ValueError(f"cache shape {tuple(k_cache.shape)} does not end in ({kvh}, {d})")
    num_slots = k_cache.numel() // (kvh * d)
    with torch.cuda.device(key.device):
        _lib.check(_lib.load().nvllm_b200_store_kvcache(
            key.data_ptr(), value.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), slot_mapping.data_ptr(),
            t, kvh, d, num_slots, _lib.DTYPE_BF16 if key.dtype == torch.bfloat16 else _lib.DTYPE_F32,
            _stream_ptr(key.device)))


def paged_decode_workspace_bytes(batch: int, num_heads: int, num_kv_heads: int, head_dim: int, max_blocks: int,
                                 block_size: int, device=None) -> int:
    with torch.cuda.device(device):
        return int(_lib.load().nvllm_b200_paged_decode_workspace_bytes(batch, num_heads, num_kv_heads, head_dim,
                                                                       max_blocks, block_size))


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                 context_lens: torch.Tensor, scale: float, block_size: int, out: torch.Tensor | None = None,
                 scratch: torch.Tensor | None = None) -> torch.Tensor:
    """Decode attention over the paged cache; returns [B, H, D] bf16."""
    _need(q, "q", torch.bfloat16, 3)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    _need(block_tables, "block_tables", torch.int32, 2)
    _need(context_lens, "context_lens", torch.int32, 1)
    b, h, d = q.shape
    nb, blk, kvh, d2 = k_cache.shape
    if v_cache.shape != k_cache.shape or d2 != d or blk != block_size:
        raise ValueError(f"cache shape {tuple(k_cache.shape)} inconsistent with q {tuple(q.shape)} / block {block_size}")
    if block_tables.shape[0] != b or context_lens.shape[0] != b:
        raise ValueError("block_tables / context_lens batch mismatch")
    mb = block_tables.shape[1]
    if out is None:
        out = torch.empty_like(q)
    else:
        _need(out, "out", torch.bfloat16, 3)
        if out.shape != q.shape:
            raise ValueError("out shape mismatch")
    with torch.cuda.device(q.device):
        lib = _lib.load()
        need = int(lib.nvllm_b200_paged_decode_workspace_bytes(b, h, kvh, d, mb, block_size))
        if scratch is None:
            scratch = workspace(q.device, need)
        _lib.check(lib.nvllm_b200_paged_decode(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(), context_lens.data_ptr(),
            out.data_ptr(), scratch.data_ptr(), scratch.numel() * scratch.element_size(),
            b, h, kvh, d, nb, block_size, mb, float(scale), _stream_ptr(q.device)))
    return out


def decode_step(q: torch.Tensor, key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                slot_mapping: torch.Tensor, block_tables: torch.Tensor, context_lens: torch.Tensor, scale: float,
                block_size: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """One decode step of one layer in one C call: scatter key/value [B, KVH, D] into the cache by slot, then
    attend (same result as ``store_kvcache`` followed by ``paged_decode``).  Caches are [NB, block, KVH, D]."""
    if key.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"key must be bf16 or fp32, got {key.dtype}")
    _need(q, "q", torch.bfloat16, 3)
    _need(key, "key", key.dtype, 3)
    _need(value, "value", key.dtype, 3)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    _need(block_tables, "block_tables", torch.int32, 2)
    _need(context_lens, "context_lens", torch.int32, 1)
    b, h, d = q.shape
    nb, blk, kvh, d2 = k_cache.shape
    if v_cache.shape != k_cache.shape or d2 != d or blk != block_size:
        raise ValueError(f"cache shape {tuple(k_cache.shape)} inconsistent with q {tuple(q.shape)} / block {block_size}")
    if tuple(key.shape) != (b, kvh, d) or value.shape != key.shape:
        raise ValueError(f"key/value must be [{b}, {kvh}, {d}], got {tuple(key.shape)} / {tuple(value.shape)}")
    if block_tables.shape[0] != b or context_lens.shape[0] != b or slot_mapping.shape[0] != b:
        raise ValueError("block_tables / context_lens / slot_mapping batch mismatch")
    mb = block_tables.shape[1]
    if out is None:
        out = torch.empty_like(q)
    else:
        _need(out, "out", torch.bfloat16, 3)
        if out.shape != q.shape:
            raise ValueError("out shape mismatch")
    with torch.cuda.device(q.device):
        lib = _lib.load()
        need = int(lib.nvllm_b200_paged_decode_workspace_bytes(b, h, kvh, d, mb, block_size))
        scratch = workspace(q.device, need)
        _lib.check(lib.nvllm_b200_decode_step(
            q.data_ptr(), key.data_ptr(), value.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            slot_mapping.data_ptr(), block_tables.data_ptr(), context_lens.data_ptr(), out.data_ptr(),
            scratch.data_ptr(), scratch.numel(), b, h, kvh, d, nb, block_size, mb, float(scale),
            _lib.DTYPE_BF16 if key.dtype == torch.bfloat16 else _lib.DTYPE_F32, _stream_ptr(q.device)))
    return out


def varlen_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                   scale: float, out: torch.Tensor | None = None, cu_seqlens_host=None,
                   cu_seqlens_k: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention over packed sequences; returns [T, H, D] bf16.

    ``cu_seqlens_host`` (a CPU int32 tensor / numpy array equal to ``cu_seqlens``) lets the library size its
    grid exactly without a device read; without it the grid is sized from ``max_seqlen``.
    """
    _need(q, "q", torch.bfloat16, 3)
    _need(k, "k", torch.bfloat16, 3)
    _need(v, "v", torch.bfloat16, 3)
    _need(cu_seqlens, "cu_seqlens", torch.int32, 1)
    if cu_seqlens_k is None:
        cu_seqlens_k = cu_seqlens
    _need(cu_seqlens_k, "cu_seqlens_k", torch.int32, 1)
    t, h, d = q.shape
    if k.shape != v.shape or k.shape[0] != t or k.shape[2] != d:
        raise ValueError(f"k/v shape {tuple(k.shape)} inconsistent with q {tuple(q.shape)}")
    kvh = k.shape[1]
    b = cu_seqlens.shape[0] - 1
    if out is None:
        out = torch.empty_like(q)
    host_ptr, keep = None, None
    if cu_seqlens_host is not None:
        keep = torch.as_tensor(cu_seqlens_host, dtype=torch.int32, device="cpu").contiguous()
        if keep.shape[0] != b + 1:
            raise ValueError("cu_seqlens_host length mismatch")
        host_ptr = keep.data_ptr()
        covered = int(keep[-1])
        if 0 <= covered < t:
            out[covered:].zero_()  # rows that belong to no sequence: the reference returns zeros there (:272-277)
    with torch.cuda.device(q.device):
        lib = _lib.load()
        need = int(lib.nvllm_b200_varlen_prefill_workspace_bytes(t, b, h, kvh, d))
        scratch = workspace(q.device, max(need, 256))
        _lib.check(lib.nvllm_b200_varlen_prefill(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), cu_seqlens.data_ptr(), cu_seqlens_k.data_ptr(), host_ptr,
            out.data_ptr(), scratch.data_ptr(), scratch.numel(), t, b, int(max_seqlen), h, kvh, d, float(scale),
            _stream_ptr(q.device)))
    del keep
    return out


def paged_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                  cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_q: int, scale: float,
                  block_size: int, out: torch.Tensor | None = None, cu_seqlens_host=None) -> torch.Tensor:
    """Causal attention of packed new tokens over their whole sequences (cached prefix included), keys/values read from
    the paged cache [NB, block, KVH, D] through ``block_tables``; returns [T, H, D] bf16.  The new tokens' K/V rows
    must already be in the cache."""
    _need(q, "q", torch.bfloat16, 3)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    _need(block_tables, "block_tables", torch.int32, 2)
    _need(cu_seqlens_q, "cu_seqlens_q", torch.int32, 1)
    _need(cu_seqlens_k, "cu_seqlens_k", torch.int32, 1)
    t, h, d = q.shape
    nb, blk, kvh, d2 = k_cache.shape
    if v_cache.shape != k_cache.shape or d2 != d or blk != block_size:
        raise ValueError(f"cache shape {tuple(k_cache.shape)} inconsistent with q {tuple(q.shape)} / block {block_size}")
    b = cu_seqlens_q.shape[0] - 1
    if cu_seqlens_k.shape[0] != b + 1 or block_tables.shape[0] != b:
        raise ValueError("cu_seqlens_k / block_tables batch mismatch")
    if out is None:
        out = torch.empty_like(q)
    host_ptr, keep = None, None
    if cu_seqlens_host is not None:
        keep = torch.as_tensor(cu_seqlens_host, dtype=torch.int32, device="cpu").contiguous()
        if keep.shape[0] != b + 1:
            raise ValueError("cu_seqlens_host length mismatch")
        host_ptr = keep.data_ptr()
        covered = int(keep[-1])
        if 0 <= covered < t:
            out[covered:].zero_()
    with torch.cuda.device(q.device):
        lib = _lib.load()
        need = int(lib.nvllm_b200_varlen_prefill_workspace_bytes(t, b, h, kvh, d))
        scratch = workspace(q.device, max(need, 256))
        _lib.check(lib.nvllm_b200_paged_prefill(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(),
            block_tables.data_ptr(), host_ptr, out.data_ptr(), scratch.data_ptr(), scratch.numel(), t, b,
            int(max_seqlen_q), h, kvh, d, nb, block_size, block_tables.shape[1], float(scale), _stream_ptr(q.device)))
    del keep
    return out


def _check_pre_attention(q, key, value, q_weight, k_weight, cos_sin_cache, positions, slot_mapping):
    _need(q, "q", torch.bfloat16, 3)
    _need(key, "key", torch.bfloat16, 3)
    _need(value, "value", torch.bfloat16, 3)
    _need(q_weight, "q_weight", torch.float32, 1)
    _need(k_weight, "k_weight", torch.float32, 1)
    _need(cos_sin_cache, "cos_sin_cache", torch.float32, 2)
    _need(positions, "positions", torch.int32, 1)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    t, h, d = q.shape
    if key.shape != value.shape or key.shape[0] != t or key.shape[2] != d:
        raise ValueError(f"key/value shape {tuple(key.shape)} inconsistent with q {tuple(q.shape)}")
    if q_weight.shape[0] != d or k_weight.shape[0] != d or cos_sin_cache.shape[1] != d:
        raise ValueError("q_weight / k_weight / cos_sin_cache must have head_dim entries per row")
    if positions.shape[0] != t or slot_mapping.shape[0] != t:
        raise ValueError("positions / slot_mapping must have one entry per token")
    return t, h, key.shape[1], d


def qk_norm_rope_store(q: torch.Tensor, key: torch.Tensor, value: torch.Tensor, q_weight: torch.Tensor,
                       k_weight: torch.Tensor, cos_sin_cache: torch.Tensor, positions: torch.Tensor,
                       k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor, eps: float = 1e-6) -> None:
    """In place, one pass: per-head RMSNorm of q and key, rotary embedding of both, scatter of the rotated key rows and
    the value rows into the cache by slot.  Caches: any leading shape whose flattening is [num_slots, KVH, D]."""
    t, h, kvh, d = _check_pre_attention(q, key, value, q_weight, k_weight, cos_sin_cache, positions, slot_mapping)
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16)
    if k_cache.shape != v_cache.shape or tuple(k_cache.shape[-2:]) != (kvh, d):
        raise ValueError(f"cache shape {tuple(k_cache.shape)} does not end in ({kvh}, {d})")
    num_slots = k_cache.numel() // (kvh * d)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().nvllm_b200_qk_norm_rope_store(
            q.data_ptr(), key.data_ptr(), value.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr(),
            cos_sin_cache.data_ptr(), positions.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            slot_mapping.data_ptr(), t, h, kvh, d, num_slots, cos_sin_cache.shape[0], float(eps), _stream_ptr(q.device)))


def fused_decode_step(q: torch.Tensor, key: torch.Tensor, value: torch.Tensor, q_weight: torch.Tensor,
                      k_weight: torch.Tensor, cos_sin_cache: torch.Tensor, positions: torch.Tensor,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor,
                      block_tables: torch.Tensor, context_lens: torch.Tensor, scale: float, block_size: int,
                      eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """``qk_norm_rope_store`` (q and key updated in place) followed by ``paged_decode``, as one C call and two kernel
    launches; returns the attention output [B, H, D]."""
    b, h, kvh, d = _check_pre_attention(q, key, value, q_weight, k_weight, cos_sin_cache, positions, slot_mapping)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    _need(block_tables, "block_tables", torch.int32, 2)
    _need(context_lens, "context_lens", torch.int32, 1)
    nb, blk, kvh2, d2 = k_cache.shape
    if v_cache.shape != k_cache.shape or (kvh2, d2) != (kvh, d) or blk != block_size:
        raise ValueError(f"cache shape {tuple(k_cache.shape)} inconsistent with key {tuple(key.shape)} / block {block_size}")
    if block_tables.shape[0] != b or context_lens.shape[0] != b:
        raise ValueError("block_tables / context_lens batch mismatch")
    if out is None:
        out = torch.empty_like(q)
    with torch.cuda.device(q.device):
        lib = _lib.load()
        mb = block_tables.shape[1]
        need = int(lib.nvllm_b200_paged_decode_workspace_bytes(b, h, kvh, d, mb, block_size))
        scratch = workspace(q.device, need)
        _lib.check(lib.nvllm_b200_fused_decode_step(
            q.data_ptr(), key.data_ptr(), value.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr(),
            cos_sin_cache.data_ptr(), positions.data_ptr(), cos_sin_cache.shape[0], float(eps), k_cache.data_ptr(),
            v_cache.data_ptr(), slot_mapping.data_ptr(), block_tables.data_ptr(), context_lens.data_ptr(),
            out.data_ptr(), scratch.data_ptr(), scratch.numel(), b, h, kvh, d, nb, block_size, mb, float(scale),
            _stream_ptr(q.device)))
    return out
