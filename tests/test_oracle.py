"""CPU checks of the oracle itself: the restatement against independent formulations.

The reference holds no golden vectors for this path and JAX cannot be imported here, so these
cross-checks (plus the committed fixtures under tests/golden/) are what pins the oracle.
"""
import math

import numpy as np
import pytest

from oracle import reference_attention as ref


def test_bf16_rounding_known_answers():
    # (fp32 bit pattern, expected bf16 bits) -- ties go to even, carries propagate into the exponent.
    cases = [(0x3F800000, 0x3F80), (0x3F808000, 0x3F80), (0x3F818000, 0x3F82), (0x3F808001, 0x3F81),
             (0x3F80FFFF, 0x3F81), (0xBF808000, 0xBF80), (0x7F7FFFFF, 0x7F80), (0x00000001, 0x0000),
             (0x80000000, 0x8000), (0x7F800000, 0x7F80), (0x7FC00000, 0x7FC0), (0x477FE000, 0x4780)]
    x = np.array([c[0] for c in cases], dtype=np.uint32).view(np.float32)
    assert ref.f32_to_bf16_bits(x).tolist() == [c[1] for c in cases]
    # widening is exact and round trip is the identity on bf16 values
    bits = np.arange(0, 0x7F80, 7, dtype=np.uint16)
    assert np.array_equal(ref.f32_to_bf16_bits(ref.bf16_bits_to_f32(bits)), bits)


def test_bf16_rounding_matches_torch():
    import torch
    rng = np.random.Generator(np.random.PCG64(1))
    x = (rng.standard_normal(100_000, dtype=np.float32) * np.float32(10) ** rng.integers(-20, 20, 100_000)).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ref.f32_to_bf16_bits(x), want)


def test_store_semantics_as_written_vs_documented():
    kc = np.zeros((8, 1, 8), np.uint16)
    vc = np.zeros((8, 1, 8), np.uint16)
    k = np.arange(1, 4, dtype=np.float32)[:, None, None] * np.ones((3, 1, 8), np.float32)
    slots = np.array([5, -1, 99], np.int32)
    as_written, _ = ref.store_kv_to_cache(k, k, kc, vc, slots)                       # layers/attention.py:64-75
    documented, _ = ref.store_kv_to_cache(k, k, kc, vc, slots, skip_negative=True)   # layers/attention.py:57-58
    assert as_written[5, 0, 0] == 0x3F80 and documented[5, 0, 0] == 0x3F80
    assert as_written[0, 0, 0] == 0x4000, "-1 lands in slot 0 in the code as written"
    assert documented[0, 0, 0] == 0
    assert np.count_nonzero(as_written) == 16 and np.count_nonzero(documented) == 8  # slot 99 dropped
    assert np.count_nonzero(kc) == 0, "inputs are not modified"


def _decode_case(seed, b=5, h=8, kvh=2, d=32, blk=16, nb=40, mb=6):
    rng = np.random.Generator(np.random.PCG64(seed))
    q = rng.standard_normal((b, h, d), dtype=np.float32)
    kc = rng.standard_normal((nb, blk, kvh, d), dtype=np.float32)
    vc = rng.standard_normal((nb, blk, kvh, d), dtype=np.float32)
    ctx = rng.integers(0, mb * blk + 1, size=b).astype(np.int32)
    ctx[0] = 0
    tables = np.full((b, mb), -1, np.int32)
    perm = rng.permutation(nb)
    pos = 0
    for i in range(b):
        n = -(-int(ctx[i]) // blk)
        tables[i, :n] = perm[pos:pos + n]
        pos += n
    return q, kc, vc, tables, ctx, 1 / math.sqrt(d), blk


def test_decode_against_float64_direct_evaluation():
    q, kc, vc, tables, ctx, scale, blk = _decode_case(3)
    got = ref.paged_decode_attention_vectorized(q, kc, vc, tables, ctx, scale, blk)
    b, h, d = q.shape
    g = h // kc.shape[2]
    for i in range(b):
        n = int(ctx[i])
        if n == 0:
            assert np.all(got[i] == 0)
            continue
        ks = np.concatenate([kc[t] for t in tables[i, : -(-n // blk)]])[:n].astype(np.float64)
        vs = np.concatenate([vc[t] for t in tables[i, : -(-n // blk)]])[:n].astype(np.float64)
        for hh in range(h):
            s = ks[:, hh // g] @ q[i, hh].astype(np.float64) * scale
            p = np.exp(s - s.max())
            want = (p / p.sum()) @ vs[:, hh // g]
            assert np.allclose(got[i, hh], want, atol=2e-6, rtol=1e-5)


def test_streamed_equals_vectorized_and_torch_variant():
    import torch
    from oracle import reference_attention_torch as reft
    q, kc, vc, tables, ctx, scale, blk = _decode_case(4, b=7, h=16, kvh=4, d=64, blk=32, nb=60, mb=8)
    a = ref.paged_decode_attention_vectorized(q, kc, vc, tables, ctx, scale, blk)
    s = ref.paged_decode_attention_streamed(q, kc, vc, tables, ctx, scale, blk)
    t = reft.paged_decode_attention_vectorized(torch.from_numpy(q), torch.from_numpy(kc), torch.from_numpy(vc),
                                               torch.from_numpy(tables), torch.from_numpy(ctx), scale, blk).numpy()
    assert np.allclose(a, s, atol=3e-6, rtol=1e-5)
    assert np.allclose(a, t, atol=3e-6, rtol=1e-5)
    bits_k, bits_v = ref.f32_to_bf16_bits(kc), ref.f32_to_bf16_bits(vc)
    sb = ref.paged_decode_attention_streamed(q, bits_k, bits_v, tables, ctx, scale, blk, kv_dtype_bits=True)
    ab = ref.paged_decode_attention_vectorized(q, ref.bf16_bits_to_f32(bits_k), ref.bf16_bits_to_f32(bits_v), tables,
                                               ctx, scale, blk)
    assert np.allclose(ab, sb, atol=3e-6, rtol=1e-5)


def test_decode_against_torch_sdpa():
    """Independent formulation: torch's scaled_dot_product_attention on the gathered, unpadded keys."""
    import torch
    q, kc, vc, tables, ctx, scale, blk = _decode_case(5)
    got = ref.paged_decode_attention_vectorized(q, kc, vc, tables, ctx, scale, blk)
    g = q.shape[1] // kc.shape[2]
    for i in range(q.shape[0]):
        n = int(ctx[i])
        if n == 0:
            continue
        nb = -(-n // blk)
        ks = torch.from_numpy(np.concatenate([kc[t] for t in tables[i, :nb]])[:n])
        vs = torch.from_numpy(np.concatenate([vc[t] for t in tables[i, :nb]])[:n])
        qq = torch.from_numpy(q[i])[:, None, :]                                  # [H, 1, d]
        kk = ks.permute(1, 0, 2).repeat_interleave(g, dim=0)                      # [H, n, d]
        vv = vs.permute(1, 0, 2).repeat_interleave(g, dim=0)
        want = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, scale=scale)[:, 0].numpy()
        assert np.allclose(got[i], want, atol=3e-6, rtol=1e-5)


def test_decode_ignores_pages_past_context_and_clips_ids():
    q, kc, vc, tables, ctx, scale, blk = _decode_case(6)
    base = ref.paged_decode_attention_vectorized(q, kc, vc, tables, ctx, scale, blk)
    t2 = tables.copy()
    t2[t2 < 0] = 10_000  # clipped to the last block (:185); masked anyway
    assert np.array_equal(base, ref.paged_decode_attention_vectorized(q, kc, vc, t2, ctx, scale, blk))


@pytest.mark.parametrize("lens", [[7], [1, 5, 16, 33], [64, 3]])
def test_prefill_against_torch_sdpa_causal(lens):
    import torch
    from oracle import reference_attention_torch as reft
    rng = np.random.Generator(np.random.PCG64(sum(lens)))
    h, kvh, d = 8, 2, 32
    t = sum(lens)
    q = rng.standard_normal((t, h, d), dtype=np.float32)
    k = rng.standard_normal((t, kvh, d), dtype=np.float32)
    v = rng.standard_normal((t, kvh, d), dtype=np.float32)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    scale = 1 / math.sqrt(d)
    got = ref.variable_length_attention_prefill(q, k, v, cu, cu, 64, 64, h, kvh, scale, len(lens))
    got_t = reft.variable_length_attention_prefill(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v), cu,
                                                   h, kvh, scale).numpy()
    assert np.allclose(got, got_t, atol=3e-6, rtol=1e-5)
    for b in range(len(lens)):
        s0, s1 = cu[b], cu[b + 1]
        qq = torch.from_numpy(q[s0:s1]).permute(1, 0, 2)
        kk = torch.from_numpy(k[s0:s1]).permute(1, 0, 2).repeat_interleave(h // kvh, dim=0)
        vv = torch.from_numpy(v[s0:s1]).permute(1, 0, 2).repeat_interleave(h // kvh, dim=0)
        want = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=scale)
        assert np.allclose(got[s0:s1], want.permute(1, 0, 2).numpy(), atol=3e-6, rtol=1e-5)


def test_prefill_bucket_truncation_quirk():
    """Rows past max_seqlen_q are never gathered and come back zero (layers/attention.py:203-228, 272-277)."""
    rng = np.random.Generator(np.random.PCG64(9))
    lens = [20, 5]
    q = rng.standard_normal((25, 4, 16), dtype=np.float32)
    k = rng.standard_normal((25, 2, 16), dtype=np.float32)
    cu = np.array([0, 20, 25], np.int32)
    out = ref.variable_length_attention_prefill(q, k, k, cu, cu, 16, 16, 4, 2, 0.25, 2)
    assert np.all(out[16:20] == 0) and np.any(out[15] != 0) and np.any(out[20:] != 0)


def test_metadata_matches_model_runner_formulas():
    lists = [[7, 2], [5], [1, 3, 9]]
    lens = [300, 256, 513]
    assert ref.decode_slot_mapping(lists, lens, 256).tolist() == [2 * 256 + 43, 5 * 256 + 255, 9 * 256 + 0]
    t = ref.pad_block_tables(lists)
    assert t.tolist() == [[7, 2, -1], [5, -1, -1], [1, 3, 9]]
    sm = ref.prefill_slot_mapping(lists, lens, 256)
    assert sm.shape[0] == sum(lens) and sm[0] == 7 * 256 and sm[256] == 2 * 256 and sm[299] == 2 * 256 + 43
    assert sm[300] == 5 * 256 and sm[-1] == 9 * 256
    assert len(set(sm.tolist())) == sm.shape[0]


def test_workload_generators_are_seeded_and_consistent():
    from nanovllm_jax_b200 import workloads
    a, b = workloads.config1(), workloads.config1()
    assert np.array_equal(a.context_lens, b.context_lens) and np.array_equal(a.block_tables, b.block_tables)
    assert a.block_tables.shape == (8, 4) and a.context_lens.min() >= 64 and a.context_lens.max() <= 1024
    assert np.array_equal(a.slot_mapping, ref.decode_slot_mapping(a.block_lists, a.context_lens, 256))
    assert np.array_equal(a.block_tables, ref.pad_block_tables(a.block_lists))
    used = [x for bl in a.block_lists for x in bl]
    assert len(used) == len(set(used))
    w2 = workloads.config2()
    assert w2.block_tables.shape == (64, 32) and 512 <= w2.context_lens.min() and w2.context_lens.max() <= 8192
    w3 = workloads.config3()
    assert w3.block_tables.shape == (256, 128) and w3.context_lens.min() >= 16 and w3.context_lens.max() <= 32768
    w4 = workloads.config4()
    assert w4.batch == 16 and w4.cu_seqlens[-1] == w4.seq_lens.sum() == w4.slot_mapping.shape[0]
    assert np.array_equal(w4.slot_mapping, ref.prefill_slot_mapping(w4.block_lists, w4.seq_lens, 256))


def test_prefix_cached_prefill_is_the_tail_of_a_full_causal_prefill():
    """The derived definition (oracle.prefix_cached_prefill_attention): the new tokens' rows must equal the LAST rows
    of a plain causal prefill over the whole sequence (restated reference function, cu_q == cu_k), whatever the
    split between cached and new tokens; with no prefix it is that function."""
    rng = np.random.Generator(np.random.PCG64(77))
    h, kvh, blk = 4, 2, 16
    lens_k, prefixes = [40, 17, 64, 5], [0, 16, 33, 4]
    nb = sum(-(-n // blk) for n in lens_k) + 2
    kc = rng.standard_normal((nb, blk, kvh, 8), dtype=np.float32)
    vc = rng.standard_normal((nb, blk, kvh, 8), dtype=np.float32)
    pool = rng.permutation(nb)
    tables = np.full((4, 5), -1, np.int32)
    pos = 0
    for b, n in enumerate(lens_k):
        m = -(-n // blk)
        tables[b, :m] = pool[pos:pos + m]
        pos += m
    # the whole sequences, packed, and their full causal prefill
    k_full = np.concatenate([kc[tables[b, :-(-n // blk)]].reshape(-1, kvh, 8)[:n] for b, n in enumerate(lens_k)])
    v_full = np.concatenate([vc[tables[b, :-(-n // blk)]].reshape(-1, kvh, 8)[:n] for b, n in enumerate(lens_k)])
    q_full = rng.standard_normal((sum(lens_k), h, 8), dtype=np.float32)
    cu_k = np.concatenate([[0], np.cumsum(lens_k)]).astype(np.int32)
    full = ref.variable_length_attention_prefill(q_full, k_full, v_full, cu_k, cu_k, 1 << 30, 1 << 30, h, kvh, 0.3, 4)
    new_lens = [n - p for n, p in zip(lens_k, prefixes)]
    cu_q = np.concatenate([[0], np.cumsum(new_lens)]).astype(np.int32)
    q_new = np.concatenate([q_full[cu_k[b] + prefixes[b]: cu_k[b + 1]] for b in range(4)])
    got = ref.prefix_cached_prefill_attention(q_new, kc, vc, tables, cu_q, cu_k, 0.3, blk)
    want = np.concatenate([full[cu_k[b] + prefixes[b]: cu_k[b + 1]] for b in range(4)])
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
