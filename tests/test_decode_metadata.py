"""Fixed-shape decode metadata (nanovllm_jax_b200/utils/decode_metadata.py): bucketing rules, padding values, pointer
stability -- on CPU -- and, on the GPU, one CUDA graph of the decode step replayed over batches of different sizes."""
import math

import numpy as np
import pytest

from nanovllm_jax_b200.utils.decode_metadata import DecodeMetadata, bucket_batch, bucket_blocks, compiled_batch_sizes


def test_batch_buckets_follow_the_reference_list():
    # engine/model_runner.py:209-210: [1, 2, 4, 8] + range(16, max_bs + 1, 16), max_bs = min(max_num_seqs, 512)
    assert compiled_batch_sizes(128) == [1, 2, 4, 8, 16, 32, 48, 64, 80, 96, 112, 128]
    assert compiled_batch_sizes(4) == [1, 2, 4]
    assert compiled_batch_sizes(10_000)[-1] == 512
    assert [bucket_batch(n, 128) for n in (1, 3, 8, 9, 16, 17, 100, 128)] == [1, 4, 8, 16, 16, 32, 112, 128]
    assert bucket_batch(600, 512) == 600
    assert [bucket_blocks(n) for n in (0, 1, 2, 3, 4, 5, 31, 32, 33)] == [1, 1, 2, 4, 4, 8, 32, 32, 64]


def test_padding_values_and_pointer_stability():
    md = DecodeMetadata(max_batch=32, max_blocks=6, device="cpu")
    assert md.max_blocks == 8
    ptrs = [t.data_ptr() for t in (md.input_ids, md.positions, md.slot_mapping, md.context_lens, md.block_tables)]
    nb, w = md.update([7, 8, 9], [10, 300, 5], [266, 1324, 517], [11, 301, 6], [[1], [5, 4], [2]], max_num_seqs=32)
    assert (nb, w) == (4, 2)
    ctx = md.context()
    assert ctx.context_lens.tolist() == [11, 301, 6, 0] and ctx.slot_mapping.tolist() == [266, 1324, 517, -1]
    assert ctx.block_tables.shape == (4, 8) and ctx.block_tables.is_contiguous()
    assert ctx.block_tables[1].tolist() == [5, 4] + [-1] * 6 and ctx.block_tables[3].tolist() == [-1] * 8
    ids, pos = md.inputs()
    assert ids.tolist() == [7, 8, 9, 0] and pos.tolist() == [10, 300, 5, 0]
    # a larger batch, then a smaller one: rows that were live go back to padding; the storage never moves
    md.update(list(range(20)), [1] * 20, list(range(100, 120)), [2] * 20, [[3, 4, 5]] * 20, max_num_seqs=32)
    assert md.padded_batch == 32 and md.width == 4
    nb, w = md.update([1], [0], [40], [1], [[9]], max_num_seqs=32)
    assert (nb, w) == (1, 1)
    assert md.context_lens[:32].tolist() == [1] + [0] * 31 and md.slot_mapping[:32].tolist() == [40] + [-1] * 31
    assert bool((md.block_tables[1:] == -1).all()) and md.block_tables[0].tolist() == [9] + [-1] * 7
    assert ptrs == [t.data_ptr() for t in (md.input_ids, md.positions, md.slot_mapping, md.context_lens, md.block_tables)]
    with pytest.raises(ValueError):
        md.update([0] * 33, [0] * 33, [0] * 33, [1] * 33, [[0]] * 33)
    with pytest.raises(ValueError):
        md.update([0], [0], [0], [1], [list(range(9))])


@pytest.mark.gpu
def test_one_captured_decode_step_serves_batches_of_different_sizes():
    """Capture Attention.__call__ (decode) once on the fixed buffers at the 16-row bucket, then replay it for batches of
    9, 16 and 12 sequences with different lengths and pages; every replay must match the oracle on the live rows,
    return zeros on the padded rows, and store exactly the live rows' K/V."""
    import torch
    from conftest import assert_attention_close, bits_to_torch, torch_to_bits, torch_to_f32
    from nanovllm_jax_b200 import workloads
    from nanovllm_jax_b200.layers.attention import Attention
    from oracle import reference_attention as ref
    h, kvh, blk, nb_pool = 16, 4, 256, 64
    rng = np.random.Generator(np.random.PCG64(4242))
    _, kcb = workloads.normal_bf16_numpy(rng, (nb_pool, blk, kvh, 128))
    _, vcb = workloads.normal_bf16_numpy(rng, (nb_pool, blk, kvh, 128))
    kc, vc = bits_to_torch(kcb), bits_to_torch(vcb)
    attn = Attention(h, 128, 1 / math.sqrt(128), kvh, blk)
    attn.set_kv_cache(kc, vc)
    md = DecodeMetadata(max_batch=16, max_blocks=4, device="cuda")
    q = torch.zeros((16, h, 128), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((16, kvh, 128), dtype=torch.bfloat16, device="cuda")
    v = torch.zeros_like(k)
    md.update([0], [0], [0], [1], [[0]], max_num_seqs=16)
    ctx = md.context(16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        attn(q, k, v, ctx)  # warm-up outside the capture: workspace allocation, kernel attributes
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    kc.copy_(bits_to_torch(kcb))
    vc.copy_(bits_to_torch(vcb))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = attn(q, k, v, ctx)
    kc_ref, vc_ref = kcb.copy(), vcb.copy()
    flat = (nb_pool * blk, kvh, 128)
    for step, n in enumerate((9, 16, 12)):
        lens = rng.integers(1, 4 * blk + 1, size=n)
        pool = rng.permutation(nb_pool)
        tables, pos = [], 0
        for c in lens:
            need = -(-int(c) // blk)
            tables.append(pool[pos:pos + need].tolist())
            pos += need
        slots = [t[-1] * blk + (int(c) - 1) % blk for t, c in zip(tables, lens)]
        qf, qb = workloads.normal_bf16_numpy(rng, (n, h, 128))
        _, kb = workloads.normal_bf16_numpy(rng, (n, kvh, 128))
        _, vb = workloads.normal_bf16_numpy(rng, (n, kvh, 128))
        q.zero_(); k.zero_(); v.zero_()
        q[:n] = bits_to_torch(qb); k[:n] = bits_to_torch(kb); v[:n] = bits_to_torch(vb)
        assert md.update([0] * n, (lens - 1).tolist(), slots, lens.tolist(), tables, max_num_seqs=16) == (16, 4)
        graph.replay()
        torch.cuda.synchronize()
        k_new, v_new = ref.store_kv_to_cache(kb, vb, kc_ref.reshape(flat), vc_ref.reshape(flat), np.array(slots, np.int32))
        kc_ref, vc_ref = k_new.reshape(kcb.shape), v_new.reshape(vcb.shape)
        assert np.array_equal(torch_to_bits(kc), kc_ref) and np.array_equal(torch_to_bits(vc), vc_ref), f"step {step}"
        padded = np.full((n, 4), -1, np.int32)
        for i, t in enumerate(tables):
            padded[i, :len(t)] = t
        want = ref.paged_decode_attention_streamed(qf, kc_ref, vc_ref, padded, lens.astype(np.int32), 1 / math.sqrt(128),
                                                   blk, kv_dtype_bits=True)
        got = torch_to_f32(out)
        assert_attention_close(got[:n], want, f"replay {step} with {n} live rows")
        assert np.all(got[n:] == 0), "padded rows attend to nothing"
