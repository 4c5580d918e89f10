"""store_kvcache through the C ABI vs the oracle: cache contents must match bit for bit."""
import numpy as np
import pytest

from conftest import bits_to_torch, torch_to_bits

pytestmark = pytest.mark.gpu


def _run(kb, vb, kcb, vcb, slots, src_f32=None):
    import torch
    from nanovllm_jax_b200 import ops
    kc, vc = bits_to_torch(kcb), bits_to_torch(vcb)
    if src_f32 is None:
        k, v = bits_to_torch(kb), bits_to_torch(vb)
    else:
        k, v = torch.from_numpy(src_f32[0]).cuda(), torch.from_numpy(src_f32[1]).cuda()
    ops.store_kvcache(k, v, kc, vc, torch.from_numpy(slots).cuda())
    torch.cuda.synchronize()
    return torch_to_bits(kc), torch_to_bits(vc)


def test_config1_decode_step_bit_exact():
    from nanovllm_jax_b200 import workloads
    from oracle import reference_attention as ref
    w = workloads.config1()
    t = workloads.decode_tensors_numpy(w)
    flat = (w.num_blocks * w.block_size, w.num_kv_heads, w.head_dim)
    want_k, want_v = ref.store_kv_to_cache(t["k_new_bits"], t["v_new_bits"], t["k_cache_bits"].reshape(flat),
                                           t["v_cache_bits"].reshape(flat), w.slot_mapping)
    got_k, got_v = _run(t["k_new_bits"], t["v_new_bits"], t["k_cache_bits"], t["v_cache_bits"], w.slot_mapping)
    assert np.array_equal(got_k.reshape(flat), want_k)
    assert np.array_equal(got_v.reshape(flat), want_v)
    # and something was actually written
    assert not np.array_equal(got_k, t["k_cache_bits"])


@pytest.mark.parametrize("kvh", [1, 2, 4, 8])
def test_prefill_slot_map_bit_exact(kvh):
    """Ragged prompt lengths scattered over a permuted pool (engine/model_runner.py:300-309 slot formula)."""
    from nanovllm_jax_b200 import workloads
    from oracle import reference_attention as ref
    w = workloads.make_prefill_workload("store-ragged", seed=4100 + kvh, batch=5, num_heads=4 * kvh, num_kv_heads=kvh,
                                        len_lo=1, len_hi=700)
    rng = np.random.Generator(np.random.PCG64(7))
    t = w.total_tokens
    _, kb = workloads.normal_bf16_numpy(rng, (t, kvh, 128))
    _, vb = workloads.normal_bf16_numpy(rng, (t, kvh, 128))
    _, kcb = workloads.normal_bf16_numpy(rng, (w.num_blocks * 256, kvh, 128))
    _, vcb = workloads.normal_bf16_numpy(rng, (w.num_blocks * 256, kvh, 128))
    assert np.array_equal(w.slot_mapping, ref.prefill_slot_mapping(w.block_lists, w.seq_lens, 256))
    want_k, want_v = ref.store_kv_to_cache(kb, vb, kcb, vcb, w.slot_mapping)
    got_k, got_v = _run(kb, vb, kcb, vcb, w.slot_mapping)
    assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)


def test_fp32_source_is_rounded_to_nearest_even():
    """The reference casts k/v to the cache dtype (layers/attention.py:70-71); include exact ties and specials."""
    from oracle import reference_attention as ref
    rng = np.random.Generator(np.random.PCG64(11))
    t, kvh = 37, 2
    k = rng.standard_normal((t, kvh, 128), dtype=np.float32) * 3
    v = rng.standard_normal((t, kvh, 128), dtype=np.float32) * 1e-3
    ties = np.array([0x3F808000, 0x3F818000, 0xBF808000, 0x3F80FFFF, 0x7F7FFFFF, 0x00000001, 0x80000000, 0x7F800000],
                    dtype=np.uint32).view(np.float32)
    k.reshape(-1)[: ties.size] = ties
    v.reshape(-1)[: ties.size] = ties[::-1]
    slots = rng.permutation(64).astype(np.int32)[:t]
    kcb = np.zeros((64, kvh, 128), np.uint16)
    vcb = np.full((64, kvh, 128), 0x1234, np.uint16)
    want_k, want_v = ref.store_kv_to_cache(k, v, kcb, vcb, slots)
    got_k, got_v = _run(None, None, kcb, vcb, slots, src_f32=(k, v))
    assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)


def test_negative_slot_skipped_and_out_of_range_dropped():
    """Documented behaviour (layers/attention.py:57-58): -1 = skip.  Out-of-range is dropped (:74-75)."""
    from oracle import reference_attention as ref
    rng = np.random.Generator(np.random.PCG64(13))
    from nanovllm_jax_b200 import workloads
    _, kb = workloads.normal_bf16_numpy(rng, (6, 8, 128))
    _, vb = workloads.normal_bf16_numpy(rng, (6, 8, 128))
    _, kcb = workloads.normal_bf16_numpy(rng, (32, 8, 128))
    _, vcb = workloads.normal_bf16_numpy(rng, (32, 8, 128))
    slots = np.array([5, -1, 31, 32, 1000, 0], dtype=np.int32)
    want_k, want_v = ref.store_kv_to_cache(kb, vb, kcb, vcb, slots, skip_negative=True)
    got_k, got_v = _run(kb, vb, kcb, vcb, slots)
    assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)
    assert np.array_equal(got_k[0], kb[5]) and np.array_equal(got_k[1], kcb[1])


def test_empty_and_bad_arguments():
    import torch
    from nanovllm_jax_b200 import _lib, ops
    kc = torch.zeros(16, 8, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    e = torch.zeros(0, 8, 128, dtype=torch.bfloat16, device="cuda")
    ops.store_kvcache(e, e, kc, vc, torch.zeros(0, dtype=torch.int32, device="cuda"))  # T = 0 is a no-op
    lib = _lib.load()
    assert lib.nvllm_b200_store_kvcache(None, None, None, None, None, 4, 8, 128, 16, 0, None) == _lib.EINVAL
    assert b"null" in lib.nvllm_b200_last_error_string()
    assert lib.nvllm_b200_store_kvcache(kc.data_ptr(), kc.data_ptr(), kc.data_ptr(), vc.data_ptr(), kc.data_ptr(),
                                        4, 8, 128, 16, 7, None) == _lib.EUNSUPPORTED
