"""nvllm_b200_qk_norm_rope_store and nvllm_b200_fused_decode_step through the C ABI vs the oracle's restatement of
q_norm / k_norm / rotary_emb / store_kv_to_cache (models/qwen3.py:157-166).  q, k and the cache must match the
restated fp32 math BIT FOR BIT after rounding to bf16; the attention output is held to the attention tolerance."""
import math

import numpy as np
import pytest

from conftest import assert_attention_close, bits_to_torch, torch_to_bits, torch_to_f32

pytestmark = pytest.mark.gpu


def _inputs(t, h, kvh, seed, max_pos=4096, nb=8, block=256, scale_in=1.0):
    from nanovllm_jax_b200 import workloads
    from oracle import reference_attention as ref
    rng = np.random.Generator(np.random.PCG64(seed))
    _, qb = workloads.normal_bf16_numpy(rng, (t, h, 128))
    _, kb = workloads.normal_bf16_numpy(rng, (t, kvh, 128))
    _, vb = workloads.normal_bf16_numpy(rng, (t, kvh, 128))
    if scale_in != 1.0:
        qb = ref.f32_to_bf16_bits(ref.bf16_bits_to_f32(qb) * np.float32(scale_in))
    wq = (1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    wk = (1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    cs = ref.rope_cos_sin_cache(128, max_pos, 1e6)
    pos = rng.integers(0, max_pos, size=t).astype(np.int32)
    _, kcb = workloads.normal_bf16_numpy(rng, (nb, block, kvh, 128))
    _, vcb = workloads.normal_bf16_numpy(rng, (nb, block, kvh, 128))
    slots = rng.permutation(nb * block)[:t].astype(np.int32)
    return qb, kb, vb, wq, wk, cs, pos, kcb, vcb, slots


@pytest.mark.parametrize("t,h,kvh", [(1, 8, 2), (7, 32, 8), (64, 16, 8), (300, 4, 4), (33, 8, 1)])
def test_qk_norm_rope_store_is_bit_exact(t, h, kvh):
    import torch
    from nanovllm_jax_b200 import ops
    from oracle import reference_attention as ref
    qb, kb, vb, wq, wk, cs, pos, kcb, vcb, slots = _inputs(t, h, kvh, 700 + t, scale_in=3.0 if t == 7 else 1.0)
    slots[t // 2] = -1  # a padded row: normalised and rotated, but not stored
    want_q, want_k = ref.qk_norm_rope(qb, kb, wq, wk, cs, pos, 1e-6)
    flat = (kcb.shape[0] * kcb.shape[1], kvh, 128)
    want_kc, want_vc = ref.store_kv_to_cache(want_k, vb, kcb.reshape(flat), vcb.reshape(flat), slots, skip_negative=True)
    q, k, v = bits_to_torch(qb), bits_to_torch(kb), bits_to_torch(vb)
    kc, vc = bits_to_torch(kcb), bits_to_torch(vcb)
    ops.qk_norm_rope_store(q, k, v, torch.from_numpy(wq).cuda(), torch.from_numpy(wk).cuda(), torch.from_numpy(cs).cuda(),
                           torch.from_numpy(pos).cuda(), kc, vc, torch.from_numpy(slots).cuda(), eps=1e-6)
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(q), want_q), "q after norm + rope"
    assert np.array_equal(torch_to_bits(k), want_k), "k after norm + rope"
    assert np.array_equal(torch_to_bits(v), vb), "v must pass through untouched"
    assert np.array_equal(torch_to_bits(kc).reshape(flat), want_kc), "k cache (untouched slots included)"
    assert np.array_equal(torch_to_bits(vc).reshape(flat), want_vc), "v cache (untouched slots included)"


def test_positions_are_clamped_to_the_table():
    import torch
    from nanovllm_jax_b200 import ops
    from oracle import reference_attention as ref
    qb, kb, vb, wq, wk, cs, pos, kcb, vcb, slots = _inputs(5, 4, 2, 720, max_pos=64)
    pos[:] = [-3, 0, 63, 64, 10_000]
    want_q, want_k = ref.qk_norm_rope(qb, kb, wq, wk, cs, pos, 1e-5)
    q, k, v = bits_to_torch(qb), bits_to_torch(kb), bits_to_torch(vb)
    ops.qk_norm_rope_store(q, k, v, torch.from_numpy(wq).cuda(), torch.from_numpy(wk).cuda(), torch.from_numpy(cs).cuda(),
                           torch.from_numpy(pos).cuda(), bits_to_torch(kcb), bits_to_torch(vcb),
                           torch.from_numpy(slots).cuda(), eps=1e-5)
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(q), want_q) and np.array_equal(torch_to_bits(k), want_k)


def test_fused_decode_step_equals_the_separate_calls_and_the_oracle():
    """One C call (norm + rope + store + ticket clear | decode) against qk_norm_rope_store + paged_decode bit for bit,
    and against the oracle chain: restated norm/rope -> restated store -> restated decode."""
    import torch
    from nanovllm_jax_b200 import ops, workloads, _lib
    from oracle import reference_attention as ref
    w = workloads.make_decode_workload("fused", seed=93, batch=21, num_heads=32, num_kv_heads=8, num_blocks=120,
                                       ctx_lo=1, ctx_hi=1400, max_blocks=6)
    t = workloads.decode_tensors_numpy(w)
    rng = np.random.Generator(np.random.PCG64(94))
    wq = (1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    wk = (1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    cs = ref.rope_cos_sin_cache(128, 2048, 1e6)
    pos = (w.context_lens - 1).astype(np.int32)  # the new token's position (engine/model_runner.py:357-361)
    want_q, want_k = ref.qk_norm_rope(t["q_bits"], t["k_new_bits"], wq, wk, cs, pos, 1e-6)
    flat = (w.num_blocks * w.block_size, 8, 128)
    kcb, vcb = ref.store_kv_to_cache(want_k, t["v_new_bits"], t["k_cache_bits"].reshape(flat),
                                     t["v_cache_bits"].reshape(flat), w.slot_mapping, skip_negative=True)
    shape4 = t["k_cache_bits"].shape
    want = ref.paged_decode_attention_streamed(ref.bf16_bits_to_f32(want_q), kcb.reshape(shape4), vcb.reshape(shape4),
                                               w.block_tables, w.context_lens, w.scale, w.block_size, kv_dtype_bits=True)
    dev = lambda a: torch.from_numpy(a).cuda()
    args = (dev(wq), dev(wk), dev(cs), dev(pos))
    sl, bt, cl = dev(w.slot_mapping), dev(w.block_tables), dev(w.context_lens)
    q1, k1, v1 = bits_to_torch(t["q_bits"]), bits_to_torch(t["k_new_bits"]), bits_to_torch(t["v_new_bits"])
    kc1, vc1 = bits_to_torch(t["k_cache_bits"]), bits_to_torch(t["v_cache_bits"])
    ops.qk_norm_rope_store(q1, k1, v1, *args, kc1, vc1, sl)
    two = ops.paged_decode(q1, kc1, vc1, bt, cl, w.scale, w.block_size)
    q2, k2, v2 = bits_to_torch(t["q_bits"]), bits_to_torch(t["k_new_bits"]), bits_to_torch(t["v_new_bits"])
    kc2, vc2 = bits_to_torch(t["k_cache_bits"]), bits_to_torch(t["v_cache_bits"])
    one = ops.fused_decode_step(q2, k2, v2, *args, kc2, vc2, sl, bt, cl, w.scale, w.block_size)
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(q2), want_q) and np.array_equal(torch_to_bits(k2), want_k)
    assert np.array_equal(torch_to_bits(kc2).reshape(flat), kcb) and np.array_equal(torch_to_bits(vc2).reshape(flat), vcb)
    assert np.array_equal(torch_to_bits(one), torch_to_bits(two))
    assert_attention_close(torch_to_f32(one), want, "fused decode step")
    assert _lib.device_status() == 0
