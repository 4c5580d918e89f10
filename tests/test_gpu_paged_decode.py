"""paged_decode through the C ABI vs the fp32 oracle (tolerance: max-abs 2e-2, mean-abs 2e-3)."""
import math

import numpy as np
import pytest

from conftest import assert_attention_close, bits_to_torch, torch_to_bits, torch_to_f32

pytestmark = pytest.mark.gpu


def _gpu_decode(t, w, kvh_slice=None):
    import torch
    from nanovllm_jax_b200 import ops
    q = bits_to_torch(t["q_bits"])
    kc, vc = bits_to_torch(t["k_cache_bits"]), bits_to_torch(t["v_cache_bits"])
    bt = torch.from_numpy(w.block_tables).cuda()
    cl = torch.from_numpy(w.context_lens).cuda()
    out = ops.paged_decode(q, kc, vc, bt, cl, w.scale, w.block_size)
    torch.cuda.synchronize()
    return out


def _status_clean():
    from nanovllm_jax_b200 import _lib
    assert _lib.device_status() == 0


def test_config1_store_then_decode():
    """Qwen3-0.6B shapes; the step first stores the 8 new tokens, then attends (layers/attention.py:465-480)."""
    import torch
    from nanovllm_jax_b200 import ops, workloads
    from oracle import reference_attention as ref
    w = workloads.config1()
    t = workloads.decode_tensors_numpy(w)
    flat = (w.num_blocks * w.block_size, w.num_kv_heads, w.head_dim)
    kcb, vcb = ref.store_kv_to_cache(t["k_new_bits"], t["v_new_bits"], t["k_cache_bits"].reshape(flat),
                                     t["v_cache_bits"].reshape(flat), w.slot_mapping)
    shape4 = t["k_cache_bits"].shape
    want = ref.paged_decode_attention_vectorized(t["q"], ref.bf16_bits_to_f32(kcb).reshape(shape4),
                                                 ref.bf16_bits_to_f32(vcb).reshape(shape4), w.block_tables,
                                                 w.context_lens, w.scale, w.block_size)
    q = bits_to_torch(t["q_bits"])
    kc, vc = bits_to_torch(t["k_cache_bits"]), bits_to_torch(t["v_cache_bits"])
    ops.store_kvcache(bits_to_torch(t["k_new_bits"]), bits_to_torch(t["v_new_bits"]), kc, vc,
                      torch.from_numpy(w.slot_mapping).cuda())
    out = ops.paged_decode(q, kc, vc, torch.from_numpy(w.block_tables).cuda(), torch.from_numpy(w.context_lens).cuda(),
                           w.scale, w.block_size)
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(kc).reshape(flat), kcb)
    assert_attention_close(torch_to_f32(out), want, "cfg1")
    _status_clean()


def _random_case(seed, batch, h, kvh, block_size, nb, mb, ctx_list=None, ctx_hi=None):
    from nanovllm_jax_b200 import workloads
    rng = np.random.Generator(np.random.PCG64(seed))
    if ctx_list is None:
        ctx = rng.integers(1, ctx_hi + 1, size=batch).astype(np.int32)
    else:
        ctx = np.asarray(ctx_list, dtype=np.int32)
        batch = len(ctx)
    tables = np.full((batch, mb), -1, dtype=np.int32)
    pool = rng.permutation(nb)
    pos = 0
    for b in range(batch):
        need = min(mb, -(-int(ctx[b]) // block_size))
        tables[b, :need] = pool[pos:pos + need]
        pos += need
    assert pos <= nb
    q, qb = workloads.normal_bf16_numpy(rng, (batch, h, 128))
    k, kb = workloads.normal_bf16_numpy(rng, (nb, block_size, kvh, 128))
    v, vb = workloads.normal_bf16_numpy(rng, (nb, block_size, kvh, 128))
    return dict(q=q, q_bits=qb, k=k, k_bits=kb, v=v, v_bits=vb, tables=tables, ctx=ctx, block_size=block_size,
                scale=1.0 / math.sqrt(128))


def _check_case(c, what, streamed=False):
    import torch
    from nanovllm_jax_b200 import ops
    from oracle import reference_attention as ref
    fn = ref.paged_decode_attention_streamed if streamed else ref.paged_decode_attention_vectorized
    want = fn(c["q"], c["k"], c["v"], c["tables"], c["ctx"], c["scale"], c["block_size"])
    out = ops.paged_decode(bits_to_torch(c["q_bits"]), bits_to_torch(c["k_bits"]), bits_to_torch(c["v_bits"]),
                           torch.from_numpy(c["tables"]).cuda(), torch.from_numpy(c["ctx"]).cuda(), c["scale"],
                           c["block_size"])
    torch.cuda.synchronize()
    got = torch_to_f32(out)
    assert_attention_close(got, want, what)
    return out, want


@pytest.mark.parametrize("h,kvh", [(8, 8), (16, 8), (32, 8), (64, 8), (4, 1), (8, 1), (8, 2), (16, 4), (2, 2)])
def test_gqa_ratios_and_head_shards(h, kvh):
    """G = 1, 2, 4, 8 and the per-rank kv-head counts of tensor parallel 1/2/4/8 (8/tp kv heads)."""
    c = _random_case(100 + h * 10 + kvh, batch=6, h=h, kvh=kvh, block_size=256, nb=24, mb=4, ctx_hi=1024)
    _check_case(c, f"H={h} KVH={kvh}")
    _status_clean()


@pytest.mark.parametrize("block_size", [64, 128, 256])
def test_context_edges(block_size):
    """Lengths around tile (64) and page boundaries, a single token, an empty sequence; -1 padded tables."""
    ctx = [0, 1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, 257, 511, 512, 513, 0, 1000]
    mb = -(-1000 // block_size)
    c = _random_case(200 + block_size, batch=len(ctx), h=16, kvh=4, block_size=block_size, nb=len(ctx) * mb, mb=mb,
                     ctx_list=ctx)
    out, want = _check_case(c, f"edges blk={block_size}")
    got = torch_to_f32(out)
    assert np.all(got[0] == 0) and np.all(got[18] == 0), "ctx == 0 must give zero rows (0 / (0 + 1e-9))"
    _status_clean()


def test_reference_selftest_layout():
    """The tables and lengths of the reference's own self-test (layers/pallas_attention.py:622-649),
    at head_dim 128 (the reference draws head_dim 64 there, which this library does not support)."""
    from nanovllm_jax_b200 import workloads
    rng = np.random.Generator(np.random.PCG64(42))
    q, qb = workloads.normal_bf16_numpy(rng, (4, 8, 128))
    k, kb = workloads.normal_bf16_numpy(rng, (32, 256, 2, 128))
    v, vb = workloads.normal_bf16_numpy(rng, (32, 256, 2, 128))
    c = dict(q=q, q_bits=qb, k=k, k_bits=kb, v=v, v_bits=vb, tables=np.arange(16, dtype=np.int32).reshape(4, 4),
             ctx=np.array([200, 512, 300, 100], np.int32), block_size=256, scale=1 / math.sqrt(128))
    _check_case(c, "reference self-test layout")


def test_reference_smoke_shapes():
    """test_mosaic_kernels.py:30-54: B=64, H=32, KVH=8, 128 blocks shared modulo the pool, ctx 200 + 50 i."""
    from nanovllm_jax_b200 import workloads
    rng = np.random.Generator(np.random.PCG64(43))
    q, qb = workloads.normal_bf16_numpy(rng, (64, 32, 128))
    k, kb = workloads.normal_bf16_numpy(rng, (128, 256, 8, 128))
    v, vb = workloads.normal_bf16_numpy(rng, (128, 256, 8, 128))
    tables = (np.arange(64 * 8, dtype=np.int32).reshape(64, 8) % 128).astype(np.int32)
    ctx = np.minimum(np.array([200 + 50 * i for i in range(64)], np.int32), 8 * 256).astype(np.int32)
    c = dict(q=q, q_bits=qb, k=k, k_bits=kb, v=v, v_bits=vb, tables=tables, ctx=ctx, block_size=256,
             scale=1 / math.sqrt(128))
    _check_case(c, "reference smoke shapes", streamed=True)
    _status_clean()


def test_context_longer_than_table_is_clamped_and_ids_are_clipped():
    """positions >= MB*block never exist in the reference (:179,:216-217); ids are clipped to the pool (:185)."""
    c = _random_case(300, batch=3, h=8, kvh=2, block_size=256, nb=8, mb=2, ctx_list=[512, 300, 100])
    c2 = dict(c)
    c2["ctx"] = np.array([5000, 300, 100], np.int32)         # beyond 2 pages -> behaves like 512
    c2["tables"] = c["tables"].copy()
    c2["tables"][1, 1] = 10_000                                # clipped to block 7
    c2["tables"][2, 1] = -1
    _check_case(c2, "clamp/clip")


def test_rows_past_context_are_never_used():
    """Cache rows at positions >= ctx may hold NaN/Inf bit patterns (recycled pages): output must not see them."""
    import torch
    from nanovllm_jax_b200 import ops
    c = _random_case(400, batch=4, h=16, kvh=4, block_size=256, nb=8, mb=2, ctx_list=[1, 70, 200, 259])
    kb, vb = c["k_bits"].copy(), c["v_bits"].copy()
    for b, n in enumerate(c["ctx"]):
        for j, blk in enumerate(c["tables"][b]):
            if blk < 0:
                continue
            lo = max(0, min(256, int(n) - j * 256))
            kb[blk, lo:] = 0x7FC0  # NaN
            vb[blk, lo:] = 0x7F80 if b % 2 else 0x7FC0  # +Inf / NaN
    clean, want = _check_case(c, "clean")
    out = ops.paged_decode(bits_to_torch(c["q_bits"]), bits_to_torch(kb), bits_to_torch(vb),
                           torch.from_numpy(c["tables"]).cuda(), torch.from_numpy(c["ctx"]).cuda(), c["scale"], 256)
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(out), torch_to_bits(clean))


def test_bitwise_deterministic_and_workspace_reuse():
    import torch
    from nanovllm_jax_b200 import ops, workloads
    w = workloads.make_decode_workload("det", seed=77, batch=40, num_heads=32, num_kv_heads=8, num_blocks=400,
                                       ctx_lo=1, ctx_hi=2300, max_blocks=9)
    t = workloads.decode_tensors_numpy(w)
    a = _gpu_decode(t, w)
    b = _gpu_decode(t, w)
    assert np.array_equal(torch_to_bits(a), torch_to_bits(b))
    _status_clean()


def _sampled_check(w, n_sample, seed, what):
    """Full-size workload on the GPU (tensors drawn on the device); the oracle re-computes a sample of sequences
    from the pages those sequences own, copied back to the host."""
    import torch
    from nanovllm_jax_b200 import ops
    from oracle import reference_attention as ref
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    q = torch.randn(w.batch, w.num_heads, 128, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    shape = (w.num_blocks, w.block_size, w.num_kv_heads, 128)
    kc = torch.empty(shape, device="cuda", dtype=torch.bfloat16)
    vc = torch.empty(shape, device="cuda", dtype=torch.bfloat16)
    for buf in (kc, vc):  # chunked draw keeps the fp32 temporary small
        flat = buf.view(-1)
        step = 1 << 27
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = torch.randn(n, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    bt = torch.from_numpy(w.block_tables).cuda()
    cl = torch.from_numpy(w.context_lens).cuda()
    out = ops.paged_decode(q, kc, vc, bt, cl, w.scale, w.block_size)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    rng = np.random.Generator(np.random.PCG64(seed))
    order = np.argsort(w.context_lens)
    pick = set(order[:4].tolist() + order[-4:].tolist()
               + rng.choice(w.batch, min(n_sample, w.batch), replace=False).tolist())
    worst = 0.0
    for b in sorted(pick):
        ids = [i for i in w.block_lists[b]]
        idx = torch.tensor(ids, device="cuda", dtype=torch.long)
        kb = torch_to_bits(kc[idx])
        vb = torch_to_bits(vc[idx])
        tables = np.arange(len(ids), dtype=np.int32)[None, :]
        want = ref.paged_decode_attention_streamed(torch_to_f32(q[b:b + 1]), kb, vb, tables, w.context_lens[b:b + 1],
                                                   w.scale, w.block_size, kv_dtype_bits=True)
        mx, _ = assert_attention_close(torch_to_f32(out[b:b + 1]), want, f"{what} seq {b} ctx {w.context_lens[b]}")
        worst = max(worst, mx)
    _status_clean()
    return worst


def test_config2_full_size_every_sequence():
    """Qwen3-8B, batch 64, ctx U[512, 8192], 4096-block pool (4.3 GB of cache): all 64 sequences vs the oracle."""
    from nanovllm_jax_b200 import workloads
    w = workloads.config2()
    _sampled_check(w, w.batch, 2000, "cfg2")


def test_config3_skewed_long_context_sampled():
    """Qwen3-32B shapes, batch 256, log-uniform ctx in [16, 32768], G = 8: the 4 shortest, the 4 longest and 28
    random sequences."""
    from nanovllm_jax_b200 import workloads
    _sampled_check(workloads.config3(), 28, 3000, "cfg3")


@pytest.mark.parametrize("src", ["bf16", "f32"])
def test_decode_step_equals_store_then_decode(src):
    """nvllm_b200_decode_step (one C call) against nvllm_b200_store_kvcache + nvllm_b200_paged_decode: caches and
    outputs bit for bit, and the output against the oracle run on the oracle's own updated cache."""
    import torch
    from nanovllm_jax_b200 import ops, workloads
    from oracle import reference_attention as ref
    w = workloads.make_decode_workload("step", seed=91, batch=33, num_heads=32, num_kv_heads=8, num_blocks=200,
                                       ctx_lo=1, ctx_hi=1500, max_blocks=6)
    t = workloads.decode_tensors_numpy(w)
    w.slot_mapping[5] = -1  # a padded row of a fixed-shape batch: nothing is stored for it
    rng = np.random.Generator(np.random.PCG64(5))
    k_new = rng.standard_normal((w.batch, 8, 128), dtype=np.float32)
    v_new = rng.standard_normal((w.batch, 8, 128), dtype=np.float32)
    if src == "bf16":
        k_new, v_new = ref.round_to_bf16(k_new), ref.round_to_bf16(v_new)
    flat = (w.num_blocks * w.block_size, 8, 128)
    kcb, vcb = ref.store_kv_to_cache(k_new, v_new, t["k_cache_bits"].reshape(flat), t["v_cache_bits"].reshape(flat),
                                     w.slot_mapping, skip_negative=True)
    shape4 = t["k_cache_bits"].shape
    want = ref.paged_decode_attention_streamed(t["q"], kcb.reshape(shape4), vcb.reshape(shape4), w.block_tables,
                                               w.context_lens, w.scale, w.block_size, kv_dtype_bits=True)
    dt = torch.bfloat16 if src == "bf16" else torch.float32
    k_dev, v_dev = torch.from_numpy(k_new).cuda().to(dt), torch.from_numpy(v_new).cuda().to(dt)
    q = bits_to_torch(t["q_bits"])
    sl = torch.from_numpy(w.slot_mapping).cuda()
    bt = torch.from_numpy(w.block_tables).cuda()
    cl = torch.from_numpy(w.context_lens).cuda()
    kc1, vc1 = bits_to_torch(t["k_cache_bits"]), bits_to_torch(t["v_cache_bits"])
    kc2, vc2 = kc1.clone(), vc1.clone()
    ops.store_kvcache(k_dev, v_dev, kc1.view(flat), vc1.view(flat), sl)
    two = ops.paged_decode(q, kc1, vc1, bt, cl, w.scale, w.block_size)
    one = ops.decode_step(q, k_dev, v_dev, kc2, vc2, sl, bt, cl, w.scale, w.block_size)
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_bits(kc2).reshape(flat), kcb) and np.array_equal(torch_to_bits(vc2).reshape(flat), vcb)
    assert np.array_equal(torch_to_bits(kc1), torch_to_bits(kc2))
    assert np.array_equal(torch_to_bits(one), torch_to_bits(two))
    assert_attention_close(torch_to_f32(one), want, "decode_step")
    _status_clean()


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_kv_head_shards_reassemble_to_unsharded(tp):
    """Head-parallel split (layers/linear.py:339-381): rank r owns kv heads [r*KVH/tp, ...) and the matching
    q heads; concatenating the ranks' outputs must reproduce the tp=1 result.  (Not bit for bit: the number
    of kv heads changes where the tile stream is cut, hence the fp32 summation order -- differences stay
    within one bf16 rounding step.)"""
    import torch
    from nanovllm_jax_b200 import ops, workloads
    w = workloads.make_decode_workload("tp", seed=88, batch=12, num_heads=32, num_kv_heads=8, num_blocks=64,
                                       ctx_lo=1, ctx_hi=1200, max_blocks=5)
    t = workloads.decode_tensors_numpy(w)
    full = _gpu_decode(t, w)
    q = bits_to_torch(t["q_bits"])
    kc, vc = bits_to_torch(t["k_cache_bits"]), bits_to_torch(t["v_cache_bits"])
    bt = torch.from_numpy(w.block_tables).cuda()
    cl = torch.from_numpy(w.context_lens).cuda()
    hs, ks = 32 // tp, 8 // tp
    parts = []
    for r in range(tp):
        parts.append(ops.paged_decode(q[:, r * hs:(r + 1) * hs].contiguous(), kc[:, :, r * ks:(r + 1) * ks].contiguous(),
                                      vc[:, :, r * ks:(r + 1) * ks].contiguous(), bt, cl, w.scale, w.block_size))
    torch.cuda.synchronize()
    got, want = torch_to_f32(torch.cat(parts, dim=1)), torch_to_f32(full)
    diff = np.abs(got - want)
    assert diff.max() <= 2.0 ** -7 * max(1.0, float(np.abs(want).max())) and diff.mean() <= 1e-4, (diff.max(), diff.mean())
    from oracle import reference_attention as ref
    shape4 = t["k_cache_bits"].shape
    oracle = ref.paged_decode_attention_streamed(t["q"], t["k_cache"], t["v_cache"], w.block_tables, w.context_lens,
                                                 w.scale, w.block_size)
    assert_attention_close(got, oracle, f"tp={tp} vs tp=1 oracle")


def test_unsupported_shapes_fail_loudly():
    import torch
    from nanovllm_jax_b200 import _lib, ops
    q = torch.zeros(2, 8, 64, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(4, 256, 2, 64, dtype=torch.bfloat16, device="cuda")
    bt = torch.zeros(2, 2, dtype=torch.int32, device="cuda")
    cl = torch.ones(2, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.NvllmError) as e:
        ops.paged_decode(q, kc, kc, bt, cl, 0.125, 256)  # head_dim 64
    assert e.value.code == _lib.EUNSUPPORTED
    q = torch.zeros(2, 32, 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(4, 256, 2, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.NvllmError):
        ops.paged_decode(q, kc, kc, bt, cl, 0.1, 256)  # G = 16
    lib = _lib.load()
    rc = lib.nvllm_b200_paged_decode(q.data_ptr(), kc.data_ptr(), kc.data_ptr(), bt.data_ptr(), cl.data_ptr(),
                                     q.data_ptr(), None, 0, 2, 8, 2, 128, 4, 256, 2, 0.1, None)
    assert rc == _lib.EWORKSPACE
