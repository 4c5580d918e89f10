"""The Python surface of this package against the reference's source text (parsed with `ast`, never imported -- it
needs JAX): same function and method names, same parameter names in the same order, same AttentionContext fields.
Skipped where the reference checkout is not mounted."""
import ast
import dataclasses
import inspect
import os

import pytest

# the reference checkout: NANOVLLM_JAX_REFERENCE, else a directory named "reference" beside this repository
REF = os.environ.get("NANOVLLM_JAX_REFERENCE") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "layers", "attention.py")),
                                reason="reference checkout not available")


def _tree(rel):
    with open(os.path.join(REF, rel)) as f:
        return ast.parse(f.read())


def _func_args(node):
    return [a.arg for a in node.args.args]


def _find(tree, name, cls=None):
    for node in ast.walk(tree):
        if cls is None and isinstance(node, ast.FunctionDef) and node.name == name:
            return node
        if cls is not None and isinstance(node, ast.ClassDef) and node.name == cls:
            for sub in node.body:
                if isinstance(sub, ast.FunctionDef) and sub.name == name:
                    return sub
    raise AssertionError(f"{cls or ''}.{name} not found in the reference")


def _mine(fn):
    return [p for p in inspect.signature(fn).parameters]


def test_attention_layer_signatures():
    from nanovllm_jax_b200.layers import attention as mine
    ref = _tree("layers/attention.py")
    assert _mine(mine.Attention.__init__) == _func_args(_find(ref, "__init__", "Attention"))
    assert _mine(mine.Attention.set_kv_cache) == _func_args(_find(ref, "set_kv_cache", "Attention"))
    assert _mine(mine.Attention.__call__) == _func_args(_find(ref, "__call__", "Attention"))
    assert _mine(mine.Attention._prefill_attention) == _func_args(_find(ref, "_prefill_attention", "Attention"))
    assert _mine(mine.Attention._decode_attention) == _func_args(_find(ref, "_decode_attention", "Attention"))
    assert _mine(mine.store_kv_to_cache) == _func_args(_find(ref, "store_kv_to_cache"))
    want = _func_args(_find(ref, "variable_length_attention_prefill"))
    got = _mine(mine.variable_length_attention_prefill)
    assert got[: len(want)] == want and got[len(want):] == ["cu_seqlens_host"]  # one optional extra, at the end
    assert mine.KVCache._fields == ("k_cache", "v_cache")
    init = _find(ref, "__init__", "Attention")
    assert ast.literal_eval(init.args.defaults[-1]) == 256 == inspect.signature(mine.Attention.__init__).parameters[
        "block_size"].default


def test_paged_module_signatures():
    from nanovllm_jax_b200.layers import attention as mine
    ref = _tree("layers/pallas_attention.py")
    assert _mine(mine.paged_attention) == _func_args(_find(ref, "paged_attention"))
    assert _mine(mine.paged_prefill_attention) == _func_args(_find(ref, "paged_prefill_attention"))
    assert mine.PALLAS_AVAILABLE is True


def test_attention_context_fields_and_builders():
    from nanovllm_jax_b200.utils import context as mine
    ref = _tree("utils/context.py")
    cls = next(n for n in ast.walk(ref) if isinstance(n, ast.ClassDef) and n.name == "AttentionContext")
    ref_fields = [s.target.id for s in cls.body if isinstance(s, ast.AnnAssign)]
    my_fields = [f.name for f in dataclasses.fields(mine.AttentionContext)]
    assert my_fields[: len(ref_fields)] == ref_fields and my_fields[len(ref_fields):] == ["cu_seqlens_host"]
    want = _func_args(_find(ref, "create_prefill_context"))
    got = _mine(mine.create_prefill_context)
    assert got[: len(want)] == want and got[len(want):] == ["cu_seqlens_host"]
    assert _mine(mine.create_decode_context) == _func_args(_find(ref, "create_decode_context"))
    assert _mine(mine._bucket_to_power_of_2) == _func_args(_find(ref, "_bucket_to_power_of_2"))
    for v in (1, 16, 17, 100, 129, 1000, 4096, 4097, 8192, 9000, 100000):
        p = 1
        while p < v:
            p *= 2
        assert mine._bucket_to_power_of_2(v) == (16 if v <= 16 else 8192 if v >= 8192 else min(p, 8192))


def test_context_builders_on_cpu_tensors():
    import torch
    from nanovllm_jax_b200.utils.context import create_decode_context, create_prefill_context
    cu = torch.tensor([0, 5, 12], dtype=torch.int32)
    c = create_prefill_context(cu, cu, 7, 7, torch.arange(12, dtype=torch.int32))
    assert c.is_prefill and c.max_seqlen_q == 16 and c.last_token_indices.tolist() == [4, 11] and c.block_tables is None
    d = create_decode_context(torch.tensor([3, 9]), torch.tensor([2, 8]), torch.zeros(2, 1, dtype=torch.int32))
    assert not d.is_prefill and d.last_token_indices is None and d.cu_seqlens_q is None
