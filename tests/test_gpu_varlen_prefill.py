"""varlen_prefill through the C ABI vs the fp32 oracle (tolerance: max-abs 2e-2, mean-abs 2e-3)."""
import math

import numpy as np
import pytest

from conftest import assert_attention_close, bits_to_torch, torch_to_bits, torch_to_f32

pytestmark = pytest.mark.gpu


def _status_clean():
    from nanovllm_jax_b200 import _lib
    assert _lib.device_status() == 0


def _run_case(lens, h, kvh, seed, host_cu=True, k_gain=None, max_seqlen=None):
    import torch
    from nanovllm_jax_b200 import ops, workloads
    from oracle import reference_attention as ref
    rng = np.random.Generator(np.random.PCG64(seed))
    t = int(sum(lens))
    q, qb = workloads.normal_bf16_numpy(rng, (t, h, 128))
    k, kb = workloads.normal_bf16_numpy(rng, (t, kvh, 128))
    v, vb = workloads.normal_bf16_numpy(rng, (t, kvh, 128))
    if k_gain is not None:  # make later keys dominate so the running max keeps growing
        k = ref.round_to_bf16(k * k_gain[:, None, None].astype(np.float32))
        kb = ref.f32_to_bf16_bits(k)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    scale = 1.0 / math.sqrt(128)
    want = ref.variable_length_attention_prefill(q, k, v, cu, cu, 1 << 30, 1 << 30, h, kvh, scale, len(lens))
    out = ops.varlen_prefill(bits_to_torch(qb), bits_to_torch(kb), bits_to_torch(vb), torch.from_numpy(cu).cuda(),
                             max_seqlen if max_seqlen is not None else int(max(lens)), scale,
                             cu_seqlens_host=cu if host_cu else None)
    torch.cuda.synchronize()
    return torch_to_f32(out), want, cu


@pytest.mark.parametrize("lens", [[1], [5], [127], [128], [129], [255], [256], [257], [300], [511, 1, 130],
                                  [64, 700, 3, 256, 385]])
def test_ragged_lengths_around_tile_edges(lens):
    got, want, _ = _run_case(lens, h=8, kvh=2, seed=1 + sum(lens))
    assert_attention_close(got, want, f"lens={lens}")
    _status_clean()


@pytest.mark.parametrize("h,kvh", [(2, 2), (6, 2)])
@pytest.mark.parametrize("lens", [[1], [128], [129], [256], [257], [511, 1, 130], [64, 700, 3, 256, 385]])
def test_ragged_lengths_with_odd_group_sizes(lens, h, kvh):
    """An odd GQA group size makes a work item 256 rows of one head instead of 128 rows of two heads."""
    got, want, _ = _run_case(lens, h=h, kvh=kvh, seed=7 + sum(lens) + h)
    assert_attention_close(got, want, f"lens={lens} H={h} KVH={kvh}")
    _status_clean()


@pytest.mark.parametrize("h,kvh", [(4, 4), (8, 4), (16, 4), (32, 8), (8, 1), (4, 1)])
def test_gqa_ratios_and_head_shards(h, kvh):
    got, want, _ = _run_case([200, 513, 40], h=h, kvh=kvh, seed=50 + h + kvh)
    assert_attention_close(got, want, f"H={h} KVH={kvh}")


def test_reference_smoke_shapes():
    """test_mosaic_kernels.py:105-125: four sequences 512/768/1024/1536, 32 q heads over 8 kv heads."""
    got, want, _ = _run_case([512, 768, 1024, 1536], h=32, kvh=8, seed=42)
    assert_attention_close(got, want, "reference smoke shapes")
    _status_clean()


def test_grid_from_max_seqlen_only():
    """Without a host copy of cu_seqlens the grid is sized from the (bucketed) max_seqlen; extra CTAs must idle."""
    got, want, _ = _run_case([100, 900, 257], h=8, kvh=2, seed=7, host_cu=False, max_seqlen=1024)
    assert_attention_close(got, want, "max_seqlen grid")
    _status_clean()


def test_running_max_growth_forces_accumulator_rescale():
    """Keys grow 4x every 128 positions: each new KV tile raises the row max by far more than 2^8, so the
    accumulator in tensor memory has to be rescaled tile after tile."""
    n = 1100
    gain = (1.0 + 0.35 * (np.arange(n) // 64)).astype(np.float32) ** 2
    got, want, _ = _run_case([n], h=4, kvh=2, seed=9, k_gain=gain)
    assert_attention_close(got, want, "rescale")
    _status_clean()


def test_bitwise_deterministic():
    a, _, _ = _run_case([700, 333], h=8, kvh=2, seed=11)
    b, _, _ = _run_case([700, 333], h=8, kvh=2, seed=11)
    assert np.array_equal(a, b)


def test_config4_full_size_with_cache_scatter():
    """Qwen3-8B prefill: 16 packed sequences U[128, 4096], 32/8 heads; K/V are also scattered into the paged cache.
    Attention is checked on all 16 sequences; the cache bit for bit."""
    import torch
    from nanovllm_jax_b200 import workloads
    from nanovllm_jax_b200.layers.attention import Attention
    from nanovllm_jax_b200.utils.context import create_prefill_context
    from oracle import reference_attention as ref
    w = workloads.config4()
    t = workloads.prefill_tensors_numpy(w)
    attn = Attention(w.num_heads, w.head_dim, w.scale, w.num_kv_heads, w.block_size)
    kc = torch.zeros((w.num_blocks, w.block_size, w.num_kv_heads, w.head_dim), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    attn.set_kv_cache(kc, vc)
    cu = torch.from_numpy(w.cu_seqlens).cuda()
    ctx = create_prefill_context(cu, cu, int(w.seq_lens.max()), int(w.seq_lens.max()),
                                 torch.from_numpy(w.slot_mapping).cuda(), cu_seqlens_host=w.cu_seqlens)
    out = attn(bits_to_torch(t["q_bits"]), bits_to_torch(t["k_bits"]), bits_to_torch(t["v_bits"]), ctx)
    torch.cuda.synchronize()
    got = torch_to_f32(out)
    assert np.isfinite(got).all()
    for b in range(w.batch):
        s0, s1 = int(w.cu_seqlens[b]), int(w.cu_seqlens[b + 1])
        cu1 = np.array([0, s1 - s0], np.int32)
        want = ref.variable_length_attention_prefill(t["q"][s0:s1], t["k"][s0:s1], t["v"][s0:s1], cu1, cu1, 1 << 30,
                                                     1 << 30, w.num_heads, w.num_kv_heads, w.scale, 1)
        assert_attention_close(got[s0:s1], want, f"cfg4 seq {b} len {s1 - s0}")
    flat = (w.num_blocks * w.block_size, w.num_kv_heads, w.head_dim)
    zero = np.zeros(flat, np.uint16)
    want_k, want_v = ref.store_kv_to_cache(t["k_bits"], t["v_bits"], zero, zero, w.slot_mapping)
    assert np.array_equal(torch_to_bits(kc).reshape(flat), want_k)
    assert np.array_equal(torch_to_bits(vc).reshape(flat), want_v)
    _status_clean()


def test_padding_rows_after_the_last_sequence_are_never_used():
    """T larger than cu_seqlens[B] (a bucketed token count): the trailing rows of q / k / v belong to no sequence and
    may hold NaN bit patterns; the last sequence's final KV tile reaches into them."""
    import torch
    from nanovllm_jax_b200 import ops, workloads
    from oracle import reference_attention as ref
    lens, pad = [300, 70], 90
    rng = np.random.Generator(np.random.PCG64(21))
    t = sum(lens)
    q, qb = workloads.normal_bf16_numpy(rng, (t, 8, 128))
    k, kb = workloads.normal_bf16_numpy(rng, (t, 2, 128))
    v, vb = workloads.normal_bf16_numpy(rng, (t, 2, 128))
    cu = np.array([0, 300, 370], np.int32)
    want = ref.variable_length_attention_prefill(q, k, v, cu, cu, 1 << 30, 1 << 30, 8, 2, 1 / math.sqrt(128), 2)
    nan_rows = lambda heads: np.full((pad, heads, 128), 0x7FC0, np.uint16)
    out = ops.varlen_prefill(bits_to_torch(np.concatenate([qb, nan_rows(8)])), bits_to_torch(np.concatenate([kb, nan_rows(2)])),
                             bits_to_torch(np.concatenate([vb, nan_rows(2)])), torch.from_numpy(cu).cuda(), 300,
                             1 / math.sqrt(128), cu_seqlens_host=cu)
    torch.cuda.synchronize()
    got = torch_to_f32(out)
    assert_attention_close(got[:t], want, "rows of real sequences")
    assert np.all(got[t:] == 0), "rows that belong to no sequence come back as zeros"
    _status_clean()


def test_bad_arguments():
    import torch
    from nanovllm_jax_b200 import _lib, ops
    q = torch.zeros(10, 4, 64, dtype=torch.bfloat16, device="cuda")
    cu = torch.tensor([0, 10], dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.NvllmError) as e:
        ops.varlen_prefill(q, q, q, cu, 10, 0.1)
    assert e.value.code == _lib.EUNSUPPORTED
    q = torch.zeros(10, 4, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.NvllmError):
        ops.varlen_prefill(q, q, q, cu, 10, 0.1, cu_seqlens_host=np.array([0, 11], np.int32))
