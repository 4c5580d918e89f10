"""nvllm_b200_paged_prefill (prefill over a cached prefix, keys/values read through block tables) vs the fp32 oracle
(tolerance: max-abs 2e-2, mean-abs 2e-3), through the C ABI and through the Attention layer."""
import math

import numpy as np
import pytest

from conftest import assert_attention_close, bits_to_torch, torch_to_bits, torch_to_f32

pytestmark = pytest.mark.gpu


def _case(prefixes, new_lens, h, kvh, block_size, seed, poison=False):
    """Sequences with `prefixes[b]` cached tokens and `new_lens[b]` new ones; pages dealt from a shuffled pool."""
    from nanovllm_jax_b200 import workloads
    rng = np.random.Generator(np.random.PCG64(seed))
    lens_k = [p + n for p, n in zip(prefixes, new_lens)]
    need = [-(-lk // block_size) for lk in lens_k]
    nb = sum(need) + 3
    pool = rng.permutation(nb).astype(np.int32)
    mb = max(need) + 1
    tables = np.full((len(lens_k), mb), -1, np.int32)
    pos = 0
    for b, n in enumerate(need):
        tables[b, :n] = pool[pos:pos + n]
        pos += n
    t = int(sum(new_lens))
    q, qb = workloads.normal_bf16_numpy(rng, (t, h, 128))
    kc, kcb = workloads.normal_bf16_numpy(rng, (nb, block_size, kvh, 128))
    vc, vcb = workloads.normal_bf16_numpy(rng, (nb, block_size, kvh, 128))
    if poison:  # rows past each sequence's last key, and every page no sequence owns, hold NaN / Inf bit patterns
        kcp, vcp = np.full_like(kcb, 0x7FC0), np.full_like(vcb, 0x7F80)
        for b, lk in enumerate(lens_k):
            for j in range(need[b]):
                n = min(block_size, lk - j * block_size)
                kcp[tables[b, j], :n] = kcb[tables[b, j], :n]
                vcp[tables[b, j], :n] = vcb[tables[b, j], :n]
        kcb, vcb = kcp, vcp
    cu_q = np.concatenate([[0], np.cumsum(new_lens)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(lens_k)]).astype(np.int32)
    return dict(q=q, q_bits=qb, k_cache=kc, k_bits=kcb, v_cache=vc, v_bits=vcb, tables=tables, cu_q=cu_q, cu_k=cu_k,
                block_size=block_size, scale=1.0 / math.sqrt(128), h=h, kvh=kvh, max_q=int(max(new_lens)))


def _run(c, host_cu=True):
    import torch
    from nanovllm_jax_b200 import ops
    out = ops.paged_prefill(bits_to_torch(c["q_bits"]), bits_to_torch(c["k_bits"]), bits_to_torch(c["v_bits"]),
                            torch.from_numpy(c["tables"]).cuda(), torch.from_numpy(c["cu_q"]).cuda(),
                            torch.from_numpy(c["cu_k"]).cuda(), c["max_q"], c["scale"], c["block_size"],
                            cu_seqlens_host=c["cu_q"] if host_cu else None)
    torch.cuda.synchronize()
    return out


def _want(c):
    from oracle import reference_attention as ref
    return ref.prefix_cached_prefill_attention(c["q"], c["k_cache"], c["v_cache"], c["tables"], c["cu_q"], c["cu_k"],
                                               c["scale"], c["block_size"])


def _status_clean():
    from nanovllm_jax_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("h,kvh", [(8, 2), (3, 1)])
@pytest.mark.parametrize("prefix", [0, 1, 255, 256, 257, 3 * 256 + 17])
def test_prefix_lengths_with_ragged_new_lengths(prefix, h, kvh):
    """Every sequence of the batch has the same cached prefix; the new lengths straddle the 128 / 256 row tiles.
    (8, 2): an item is 128 rows of two heads; (3, 1): the group size is odd, an item is 256 rows of one head."""
    new_lens = [1, 5, 127, 128, 129, 255, 256, 257, 300, 700]
    c = _case([prefix] * len(new_lens), new_lens, h=h, kvh=kvh, block_size=256, seed=600 + prefix + h)
    assert_attention_close(torch_to_f32(_run(c)), _want(c), f"prefix {prefix} H={h} KVH={kvh}")
    _status_clean()


def test_mixed_prefixes_block_128_and_grid_from_max_seqlen():
    prefixes = [0, 130, 1, 512, 77, 1000, 384]
    new_lens = [300, 1, 513, 64, 256, 90, 129]
    c = _case(prefixes, new_lens, h=16, kvh=4, block_size=128, seed=611)
    want = _want(c)
    assert_attention_close(torch_to_f32(_run(c)), want, "mixed, block 128")
    assert_attention_close(torch_to_f32(_run(c, host_cu=False)), want, "mixed, grid sized from max_seqlen_q")
    _status_clean()


@pytest.mark.parametrize("h,kvh", [(4, 4), (8, 1), (32, 8), (6, 2)])
def test_head_ratios(h, kvh):
    c = _case([200, 0, 333], [260, 140, 31], h=h, kvh=kvh, block_size=256, seed=620 + h)
    assert_attention_close(torch_to_f32(_run(c)), _want(c), f"H={h} KVH={kvh}")
    _status_clean()


def test_cache_rows_past_the_sequence_are_never_used():
    """Recycled or never-written cache rows may hold NaN / Inf bit patterns: the output must not see them."""
    prefixes, new_lens = [0, 100, 256, 300], [50, 129, 1, 212]
    clean = _case(prefixes, new_lens, h=8, kvh=2, block_size=256, seed=630)
    dirty = _case(prefixes, new_lens, h=8, kvh=2, block_size=256, seed=630, poison=True)
    a, b = _run(clean), _run(dirty)
    assert np.isfinite(torch_to_f32(b)).all()
    assert np.array_equal(torch_to_bits(a), torch_to_bits(b))
    _status_clean()


def test_no_prefix_equals_the_packed_entry_point():
    """With cu_seqlens_k == cu_seqlens_q the paged entry computes what nvllm_b200_varlen_prefill does (same tiles in
    the same order: bit for bit)."""
    import torch
    from nanovllm_jax_b200 import ops
    from oracle import reference_attention as ref
    new_lens = [300, 17, 256, 1000]
    c = _case([0] * 4, new_lens, h=8, kvh=2, block_size=256, seed=640)
    paged = _run(c)
    # gather the same keys into packed [T, KVH, D] tensors
    t = sum(new_lens)
    kp = np.zeros((t, 2, 128), np.uint16)
    vp = np.zeros_like(kp)
    for b, n in enumerate(new_lens):
        for j in range(-(-n // 256)):
            m = min(256, n - j * 256)
            kp[c["cu_q"][b] + j * 256: c["cu_q"][b] + j * 256 + m] = c["k_bits"][c["tables"][b, j], :m]
            vp[c["cu_q"][b] + j * 256: c["cu_q"][b] + j * 256 + m] = c["v_bits"][c["tables"][b, j], :m]
    packed = ops.varlen_prefill(bits_to_torch(c["q_bits"]), bits_to_torch(kp), bits_to_torch(vp),
                                torch.from_numpy(c["cu_q"]).cuda(), max(new_lens), c["scale"], cu_seqlens_host=c["cu_q"])
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(paged), torch_to_bits(packed))
    want = ref.variable_length_attention_prefill(c["q"], ref.bf16_bits_to_f32(kp), ref.bf16_bits_to_f32(vp), c["cu_q"],
                                                 c["cu_q"], 1 << 30, 1 << 30, 8, 2, c["scale"], 4)
    assert_attention_close(torch_to_f32(paged), want, "no prefix")


def test_attention_layer_takes_the_paged_path_on_a_prefix_hit():
    """Attention.__call__ with a prefill context that carries block_tables (engine/model_runner.py:311-314): the new
    tokens' K/V are stored first, then the whole sequence is attended through the pages."""
    import torch
    from nanovllm_jax_b200.layers.attention import Attention
    from nanovllm_jax_b200.utils.context import create_prefill_context
    from oracle import reference_attention as ref
    prefixes, new_lens = [256, 0, 512 + 40], [130, 300, 77]
    c = _case(prefixes, new_lens, h=8, kvh=2, block_size=256, seed=650)
    rng = np.random.Generator(np.random.PCG64(651))
    t = sum(new_lens)
    k_new = ref.round_to_bf16(rng.standard_normal((t, 2, 128), dtype=np.float32))
    v_new = ref.round_to_bf16(rng.standard_normal((t, 2, 128), dtype=np.float32))
    # slots of the new tokens: positions prefix .. prefix + n - 1 of each sequence (engine/model_runner.py:300-309)
    slots = np.concatenate([[c["tables"][b, p // 256] * 256 + p % 256 for p in range(pre, pre + n)]
                            for b, (pre, n) in enumerate(zip(prefixes, new_lens))]).astype(np.int32)
    nbk = c["k_bits"].shape[0]
    flat = (nbk * 256, 2, 128)
    kcb, vcb = ref.store_kv_to_cache(k_new, v_new, c["k_bits"].reshape(flat), c["v_bits"].reshape(flat), slots)
    want = ref.prefix_cached_prefill_attention(c["q"], ref.bf16_bits_to_f32(kcb).reshape(c["k_bits"].shape),
                                               ref.bf16_bits_to_f32(vcb).reshape(c["k_bits"].shape), c["tables"],
                                               c["cu_q"], c["cu_k"], c["scale"], 256)
    attn = Attention(8, 128, c["scale"], 2, 256)
    kc, vc = bits_to_torch(c["k_bits"]), bits_to_torch(c["v_bits"])
    attn.set_kv_cache(kc, vc)
    ctx = create_prefill_context(torch.from_numpy(c["cu_q"]).cuda(), torch.from_numpy(c["cu_k"]).cuda(),
                                 max(new_lens), max(p + n for p, n in zip(prefixes, new_lens)),
                                 torch.from_numpy(slots).cuda(), block_tables=torch.from_numpy(c["tables"]).cuda())
    out = attn(bits_to_torch(c["q_bits"]), torch.from_numpy(k_new).cuda().bfloat16(),
               torch.from_numpy(v_new).cuda().bfloat16(), ctx)
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(kc).reshape(flat), kcb), "cache rows of the new tokens"
    assert_attention_close(torch_to_f32(out), want, "Attention.__call__ on a prefix hit")
    _status_clean()


def test_inconsistent_lengths_raise_the_status_bit_and_compute_nothing():
    """Packed keys with cu_seqlens_k != cu_seqlens_q (a cached prefix the packed entry cannot serve), and a sequence
    with fewer keys than queries: bit 5 of the device status, output untouched."""
    import torch
    from nanovllm_jax_b200 import _lib, ops
    c = _case([0, 0], [100, 60], h=4, kvh=2, block_size=256, seed=660)
    q = bits_to_torch(c["q_bits"])
    k = torch.zeros((160, 2, 128), dtype=torch.bfloat16, device="cuda")
    cu_q = torch.from_numpy(c["cu_q"]).cuda()
    cu_k_longer = torch.tensor([0, 356, 416], dtype=torch.int32, device="cuda")
    out = torch.full_like(q, 7.0)
    try:
        ops.varlen_prefill(q, k, k, cu_q, 100, c["scale"], out=out, cu_seqlens_k=cu_k_longer)
        torch.cuda.synchronize()
        assert _lib.device_status() & 32
        assert bool((out == 7.0).all())
        _lib.device_status_reset()
        assert _lib.device_status() == 0
        cu_k_shorter = torch.tensor([0, 50, 110], dtype=torch.int32, device="cuda")
        ops.paged_prefill(q, bits_to_torch(c["k_bits"]), bits_to_torch(c["v_bits"]), torch.from_numpy(c["tables"]).cuda(),
                          cu_q, cu_k_shorter, 100, c["scale"], 256, out=out)
        torch.cuda.synchronize()
        assert _lib.device_status() & 32
        assert bool((out == 7.0).all())
    finally:
        _lib.device_status_reset()
    assert _lib.device_status() == 0
