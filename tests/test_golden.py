"""Committed fixtures (tests/golden/*.npz, made by tests/golden/make_golden.py).

CPU: the oracle of today reproduces the frozen answers.  GPU: the CUDA kernels, through the C ABI, match them --
cache contents bit for bit, attention within max-abs 2e-2 / mean-abs 2e-3.
"""
import os

import numpy as np
import pytest

from conftest import assert_attention_close, bits_to_torch, torch_to_bits, torch_to_f32
from oracle import reference_attention as ref

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return dict(np.load(os.path.join(GOLD, name)))


def test_oracle_store_matches_fixture():
    g = _load("store_kvcache.npz")
    k, v = ref.store_kv_to_cache(g["k"], g["v"], g["k_cache"], g["v_cache"], g["slot_mapping"], skip_negative=True)
    assert np.array_equal(k, g["k_cache_documented"]) and np.array_equal(v, g["v_cache_documented"])
    k, v = ref.store_kv_to_cache(g["k"], g["v"], g["k_cache"], g["v_cache"], g["slot_mapping"])
    assert np.array_equal(k, g["k_cache_as_written"]) and np.array_equal(v, g["v_cache_as_written"])
    # the two behaviours differ only in slot 0 (target of the -1 token in the code as written)
    differ = np.nonzero((g["k_cache_documented"] != g["k_cache_as_written"]).any(axis=(1, 2)))[0]
    assert differ.tolist() == [] or differ.tolist() == [0]


def test_oracle_decode_matches_fixture():
    g = _load("paged_decode.npz")
    args = (ref.bf16_bits_to_f32(g["q"]), ref.bf16_bits_to_f32(g["k_cache"]), ref.bf16_bits_to_f32(g["v_cache"]),
            g["block_tables"], g["context_lens"], float(g["scale"]), int(g["block_size"]))
    assert np.allclose(ref.paged_decode_attention_vectorized(*args), g["out_f32"], atol=2e-6, rtol=1e-5)
    assert np.allclose(ref.paged_decode_attention_streamed(*args), g["out_f32"], atol=2e-6, rtol=1e-5)
    assert np.all(g["out_f32"][2] == 0)


def test_oracle_prefill_matches_fixture():
    g = _load("varlen_prefill.npz")
    out = ref.variable_length_attention_prefill(ref.bf16_bits_to_f32(g["q"]), ref.bf16_bits_to_f32(g["k"]),
                                                ref.bf16_bits_to_f32(g["v"]), g["cu_seqlens"], g["cu_seqlens"], 256, 256,
                                                2, 1, float(g["scale"]), 2)
    assert np.allclose(out, g["out_f32"], atol=2e-6, rtol=1e-5)


@pytest.mark.gpu
def test_cuda_store_matches_fixture():
    import torch
    from nanovllm_jax_b200 import ops
    g = _load("store_kvcache.npz")
    kc, vc = bits_to_torch(g["k_cache"]), bits_to_torch(g["v_cache"])
    ops.store_kvcache(bits_to_torch(g["k"]), bits_to_torch(g["v"]), kc, vc, torch.from_numpy(g["slot_mapping"]).cuda())
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(kc), g["k_cache_documented"])
    assert np.array_equal(torch_to_bits(vc), g["v_cache_documented"])


@pytest.mark.gpu
def test_cuda_decode_matches_fixture():
    import torch
    from nanovllm_jax_b200 import ops
    g = _load("paged_decode.npz")
    out = ops.paged_decode(bits_to_torch(g["q"]), bits_to_torch(g["k_cache"]), bits_to_torch(g["v_cache"]),
                           torch.from_numpy(g["block_tables"]).cuda(), torch.from_numpy(g["context_lens"]).cuda(),
                           float(g["scale"]), int(g["block_size"]))
    torch.cuda.synchronize()
    assert_attention_close(torch_to_f32(out), g["out_f32"], "golden decode")


@pytest.mark.gpu
def test_cuda_prefill_matches_fixture():
    import torch
    from nanovllm_jax_b200 import ops
    g = _load("varlen_prefill.npz")
    out = ops.varlen_prefill(bits_to_torch(g["q"]), bits_to_torch(g["k"]), bits_to_torch(g["v"]),
                             torch.from_numpy(g["cu_seqlens"]).cuda(), 150, float(g["scale"]),
                             cu_seqlens_host=g["cu_seqlens"])
    torch.cuda.synchronize()
    assert_attention_close(torch_to_f32(out), g["out_f32"], "golden prefill")
