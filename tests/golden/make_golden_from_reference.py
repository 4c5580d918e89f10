"""Pins the CPU oracle to the REAL reference: run this where JAX is installed.

    python tests/golden/make_golden_from_reference.py /path/to/nanovllm_jax [--write]

CANNOT RUN IN THE IMAGE THIS LIBRARY WAS BUILT IN (jax, jaxlib and flax are absent and there is no network);
it is committed so that a maintainer with JAX can turn the oracle's "parity unpinned" into a pinned one.

What it does.  It imports the reference's own functions for the attention hot path,

    store_kv_to_cache                         layers/attention.py:42-77
    paged_decode_attention_vectorized         layers/pallas_attention.py:146-238
    variable_length_attention_prefill         layers/attention.py:135-279
    RMSNorm._rms_forward + apply_rotary_emb   layers/layernorm.py:31-48, layers/rotary_embedding.py:13-37

runs them on the CPU backend (``JAX_PLATFORMS=cpu``) on the inputs stored in the committed fixtures
(``store_kvcache.npz``, ``paged_decode.npz``, ``varlen_prefill.npz``: inputs are bf16 bit patterns drawn from
fixed PCG64 seeds by ``make_golden.py``) plus one seeded pre-attention case, and

  * prints, per function, how far the reference's output is from the oracle's frozen answer
    (cache contents: number of differing bf16 words, must be 0; attention: max-abs / mean-abs in fp32);
  * with ``--write`` stores the reference's outputs next to the fixtures as ``reference_outputs.npz``; once that
    file exists, ``tests/test_golden.py::test_oracle_matches_reference_outputs`` checks the oracle against it on
    every CPU run, which is what "pinned" means.

The reference package imports JAX in its ``__init__`` and Flax in its layers, so both must be importable.  The
package is loaded from the given directory under the name ``nanovllm_jax``.
"""
from __future__ import annotations

import argparse
import importlib.util
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def load_reference(path: str):
    """Import the reference checkout at `path` as the package ``nanovllm_jax``."""
    os.environ.setdefault("JAX_PLATFORMS", "cpu")
    spec = importlib.util.spec_from_file_location("nanovllm_jax", os.path.join(path, "__init__.py"),
                                                  submodule_search_locations=[path])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["nanovllm_jax"] = mod
    spec.loader.exec_module(mod)
    return mod


def bits_to_jnp(bits):
    import jax.numpy as jnp
    return jnp.asarray(np.ascontiguousarray(bits).view(np.uint16)).view(jnp.bfloat16)


def jnp_to_bits(x):
    import jax.numpy as jnp
    return np.asarray(x.astype(jnp.bfloat16).view(jnp.uint16))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("reference", help="directory of the nanovllm_jax checkout")
    ap.add_argument("--write", action="store_true", help="store the reference's outputs as reference_outputs.npz")
    args = ap.parse_args()
    try:
        import jax  # noqa: F401
        import jax.numpy as jnp
    except ImportError:
        raise SystemExit("JAX is not installed here: this script has to run where the reference itself can run")
    load_reference(os.path.abspath(args.reference))
    from nanovllm_jax.layers import attention as ref_attn
    from nanovllm_jax.layers import pallas_attention as ref_paged
    from nanovllm_jax.layers.layernorm import RMSNorm
    from nanovllm_jax.layers.rotary_embedding import apply_rotary_emb
    from oracle import reference_attention as oracle

    out = {}
    report = []

    # ---- store_kv_to_cache (bit-exact gate) ----
    g = dict(np.load(os.path.join(HERE, "store_kvcache.npz")))
    kc, vc = ref_attn.store_kv_to_cache(bits_to_jnp(g["k"]), bits_to_jnp(g["v"]), bits_to_jnp(g["k_cache"]),
                                        bits_to_jnp(g["v_cache"]), jnp.asarray(g["slot_mapping"]))
    out["store_k_cache"], out["store_v_cache"] = jnp_to_bits(kc), jnp_to_bits(vc)
    report.append(("store_kv_to_cache vs oracle (code as written)",
                   int((out["store_k_cache"] != g["k_cache_as_written"]).sum()
                       + (out["store_v_cache"] != g["v_cache_as_written"]).sum()), "differing bf16 words (must be 0)"))

    # ---- paged decode ----
    g = dict(np.load(os.path.join(HERE, "paged_decode.npz")))
    o = ref_paged.paged_decode_attention_vectorized(
        bits_to_jnp(g["q"]).astype(jnp.float32), bits_to_jnp(g["k_cache"]).astype(jnp.float32),
        bits_to_jnp(g["v_cache"]).astype(jnp.float32), jnp.asarray(g["block_tables"]), jnp.asarray(g["context_lens"]),
        float(g["scale"]), int(g["block_size"]))
    out["decode_out_f32"] = np.asarray(o, dtype=np.float32)
    d = np.abs(out["decode_out_f32"] - g["out_f32"])
    report.append(("paged_decode_attention_vectorized vs oracle", float(d.max()), f"max-abs (mean {d.mean():.3e})"))

    # ---- varlen prefill ----
    g = dict(np.load(os.path.join(HERE, "varlen_prefill.npz")))
    cu = jnp.asarray(g["cu_seqlens"])
    o = ref_attn.variable_length_attention_prefill(
        bits_to_jnp(g["q"]).astype(jnp.float32), bits_to_jnp(g["k"]).astype(jnp.float32),
        bits_to_jnp(g["v"]).astype(jnp.float32), cu, cu, 256, 256, 2, 1, float(g["scale"]), 2)
    out["prefill_out_f32"] = np.asarray(o, dtype=np.float32)
    d = np.abs(out["prefill_out_f32"] - g["out_f32"])
    report.append(("variable_length_attention_prefill vs oracle", float(d.max()), f"max-abs (mean {d.mean():.3e})"))

    # ---- q_norm / k_norm / rotary_emb (models/qwen3.py:157-163) ----
    rng = np.random.Generator(np.random.PCG64(20260004))
    qb = oracle.f32_to_bf16_bits(rng.standard_normal((9, 4, 128), dtype=np.float32))
    kb = oracle.f32_to_bf16_bits(rng.standard_normal((9, 2, 128), dtype=np.float32))
    wq = (1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    wk = (1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    pos = rng.integers(0, 512, size=9).astype(np.int32)
    cs = oracle.rope_cos_sin_cache(128, 512, 1e6)
    norm_q, norm_k = RMSNorm(128, eps=1e-6), RMSNorm(128, eps=1e-6)
    norm_q.weight.value, norm_k.weight.value = jnp.asarray(wq), jnp.asarray(wk)
    cos, sin = jnp.asarray(cs[pos, None, :64]), jnp.asarray(cs[pos, None, 64:])
    q_ref = apply_rotary_emb(norm_q(bits_to_jnp(qb)), cos, sin)
    k_ref = apply_rotary_emb(norm_k(bits_to_jnp(kb)), cos, sin)
    out["rope_q_bits"], out["rope_k_bits"] = jnp_to_bits(q_ref), jnp_to_bits(k_ref)
    want_q, want_k = oracle.qk_norm_rope(qb, kb, wq, wk, cs, pos, 1e-6)
    report.append(("q_norm + rotary_emb vs oracle", int((out["rope_q_bits"] != want_q).sum()),
                   f"differing bf16 words of {want_q.size} (XLA's reduction order may differ from the oracle's)"))
    report.append(("k_norm + rotary_emb vs oracle", int((out["rope_k_bits"] != want_k).sum()),
                   f"differing bf16 words of {want_k.size}"))

    for name, value, what in report:
        print(f"{name:55s} {value!s:>12s}  {what}")
    if args.write:
        path = os.path.join(HERE, "reference_outputs.npz")
        np.savez_compressed(path, **out)
        print("wrote", path)


if __name__ == "__main__":
    main()
