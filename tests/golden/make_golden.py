"""Generates the committed fixtures in this directory from the CPU oracle.

    python tests/golden/make_golden.py

The reference project holds no golden vectors for the attention path and JAX cannot be imported in the
build image, so these files are NOT outputs of the reference: they freeze the oracle's answers on small,
fully specified inputs (inputs are stored too, as bf16 bit patterns), so that (i) any later change to the
oracle shows up as a diff against them and (ii) the CUDA kernels are checked against numbers that do not
depend on the oracle code of the day.
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import reference_attention as ref  # noqa: E402


def bf16(rng, shape):
    x = rng.standard_normal(size=shape, dtype=np.float32)
    bits = ref.f32_to_bf16_bits(x)
    return ref.bf16_bits_to_f32(bits), bits


def main():
    # ---- store_kvcache: 7 tokens into a 48-slot cache, one negative and one out-of-range slot ----
    rng = np.random.Generator(np.random.PCG64(20260001))
    _, k = bf16(rng, (7, 2, 128))
    _, v = bf16(rng, (7, 2, 128))
    _, kc = bf16(rng, (48, 2, 128))
    _, vc = bf16(rng, (48, 2, 128))
    slots = np.array([5, 47, -1, 0, 48, 17, 30], dtype=np.int32)
    k_doc, v_doc = ref.store_kv_to_cache(k, v, kc, vc, slots, skip_negative=True)
    k_asw, v_asw = ref.store_kv_to_cache(k, v, kc, vc, slots, skip_negative=False)
    np.savez_compressed(os.path.join(HERE, "store_kvcache.npz"), k=k, v=v, k_cache=kc, v_cache=vc, slot_mapping=slots,
                        k_cache_documented=k_doc, v_cache_documented=v_doc, k_cache_as_written=k_asw,
                        v_cache_as_written=v_asw)

    # ---- paged decode: 4 sequences (one empty), G = 4, block 64, permuted pages, -1 padding ----
    rng = np.random.Generator(np.random.PCG64(20260002))
    q, qb = bf16(rng, (4, 4, 128))
    kcf, kcb = bf16(rng, (9, 64, 1, 128))
    vcf, vcb = bf16(rng, (9, 64, 1, 128))
    ctx = np.array([1, 100, 0, 200], dtype=np.int32)
    tables = np.array([[3, -1, -1, -1], [7, 0, -1, -1], [-1, -1, -1, -1], [5, 8, 2, 6]], dtype=np.int32)
    scale = 1.0 / math.sqrt(128)
    out = ref.paged_decode_attention_vectorized(q, kcf, vcf, tables, ctx, scale, 64)
    np.savez_compressed(os.path.join(HERE, "paged_decode.npz"), q=qb, k_cache=kcb, v_cache=vcb, block_tables=tables,
                        context_lens=ctx, scale=np.float32(scale), block_size=np.int32(64), out_f32=out)

    # ---- varlen prefill: two packed sequences (40 and 150 tokens), G = 2 ----
    rng = np.random.Generator(np.random.PCG64(20260003))
    lens = [40, 150]
    t = sum(lens)
    q, qb = bf16(rng, (t, 2, 128))
    k, kb = bf16(rng, (t, 1, 128))
    v, vb = bf16(rng, (t, 1, 128))
    cu = np.array([0, 40, 190], dtype=np.int32)
    out = ref.variable_length_attention_prefill(q, k, v, cu, cu, 256, 256, 2, 1, scale, 2)
    np.savez_compressed(os.path.join(HERE, "varlen_prefill.npz"), q=qb, k=kb, v=vb, cu_seqlens=cu,
                        scale=np.float32(scale), out_f32=out)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
