"""jax.ffi binding of the C ABI: the module that replaces the reference's ``layers/pallas_attention.py``.

Same public names and signatures as the module it replaces (reference layers/pallas_attention.py:465-474,
557-564) plus ``store_kv_to_cache`` (layers/attention.py:42-77), all as ``jax.ffi.ffi_call`` custom calls into
``libnvllm_b200_attn.so`` through the small XLA FFI adapter in ``csrc/xla_ffi/nvllm_b200_ffi.cc``.

UNVERIFIED: JAX, jaxlib and Flax are not installed in the image this library was built in, so nothing in this module
has been executed against a real JAX.  It imports without JAX; every function raises ImportError when JAX is missing.
The same kernels are exercised through ``ctypes`` by the test-suite (``nanovllm_jax_b200.ops``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

from . import _lib

_HERE = os.path.dirname(os.path.abspath(__file__))
ADAPTER_SOURCE = os.path.join(_HERE, "csrc", "xla_ffi", "nvllm_b200_ffi.cc")
ADAPTER_LIB = os.path.join(_HERE, "libnvllm_b200_ffi.so")
TARGETS = ("NvllmStore", "NvllmDecode", "NvllmPrefill", "NvllmPagedPrefill", "NvllmStoreInPlace", "NvllmDecodeStepInPlace")

PALLAS_AVAILABLE = True  # flag tested by the reference at layers/attention.py:384
_registered = False


def _jax():
    try:
        import jax  # noqa: F401
        import jax.numpy as jnp  # noqa: F401
    except ImportError as exc:  # pragma: no cover - depends on the environment
        raise ImportError("nanovllm_jax_b200.jax_ffi needs JAX (jax, jaxlib) installed; the kernels themselves are "
                          "reachable without it through nanovllm_jax_b200.ops") from exc
    return jax, jnp


def build_ffi_adapter(cxx: str = "g++") -> str:
    """Compile the XLA FFI adapter against the headers jaxlib ships and link it to the CUDA library."""
    jax, _ = _jax()
    include = jax.ffi.include_dir()
    root = os.path.dirname(_HERE)
    cmd = [cxx, "-std=c++17", "-O2", "-shared", "-fPIC", f"-I{include}", f"-I{os.path.join(root, 'include')}",
           "-I/usr/local/cuda/include", ADAPTER_SOURCE, f"-L{_HERE}", "-lnvllm_b200_attn", f"-Wl,-rpath,{_HERE}",
           "-o", ADAPTER_LIB]
    subprocess.run(cmd, check=True)
    return ADAPTER_LIB


def register() -> None:
    """Load both shared libraries and register the three custom-call targets for the CUDA platform (idempotent)."""
    global _registered
    if _registered:
        return
    jax, _ = _jax()
    _lib.load()
    if not os.path.exists(ADAPTER_LIB):
        build_ffi_adapter()
    adapter = ctypes.CDLL(ADAPTER_LIB)
    for name in TARGETS:
        jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(adapter, name)), platform="CUDA")
    _registered = True


def store_kv_to_cache(key, value, k_cache, v_cache, slot_mapping):
    """Reference layers/attention.py:42-77; the caches are aliased to the results like donate_argnums=(2, 3)."""
    jax, jnp = _jax()
    register()
    call = jax.ffi.ffi_call("NvllmStore", (jax.ShapeDtypeStruct(k_cache.shape, k_cache.dtype),
                                           jax.ShapeDtypeStruct(v_cache.shape, v_cache.dtype)),
                            input_output_aliases={2: 0, 3: 1})
    return call(key, value, k_cache, v_cache, slot_mapping.astype(jnp.int32))


def paged_attention(q, k_cache, v_cache, block_tables, context_lens, scale: float, block_size: int):
    """Reference layers/pallas_attention.py:465-507."""
    import numpy as np
    jax, jnp = _jax()
    register()
    b, h, d = q.shape
    kvh, mb = k_cache.shape[2], block_tables.shape[1]
    nbytes = int(_lib.load().nvllm_b200_paged_decode_workspace_bytes(b, h, kvh, d, mb, block_size))
    out, _ = jax.ffi.ffi_call("NvllmDecode", (jax.ShapeDtypeStruct(q.shape, q.dtype),
                                              jax.ShapeDtypeStruct((nbytes,), jnp.uint8)))(
        q, k_cache, v_cache, block_tables.astype(jnp.int32), context_lens.astype(jnp.int32), scale=np.float32(scale))
    return out


def paged_prefill_attention(q, k, v, cu_seqlens, max_seqlen: int, scale: float):
    """Reference layers/pallas_attention.py:557-608 (cu_seqlens_q == cu_seqlens_k)."""
    import numpy as np
    jax, jnp = _jax()
    register()
    t, h, d = q.shape
    nbytes = max(256, int(_lib.load().nvllm_b200_varlen_prefill_workspace_bytes(t, cu_seqlens.shape[0] - 1, h,
                                                                               k.shape[1], d)))
    cu = cu_seqlens.astype(jnp.int32)
    out, _ = jax.ffi.ffi_call("NvllmPrefill", (jax.ShapeDtypeStruct(q.shape, q.dtype),
                                               jax.ShapeDtypeStruct((nbytes,), jnp.uint8)))(
        q, k, v, cu, cu, scale=np.float32(scale), max_seqlen=np.int32(max_seqlen))
    return out


def paged_prefill_from_cache(q, k_cache, v_cache, block_tables, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int,
                             scale: float, block_size: int):
    """Prefill over a cached prefix (``nvllm_b200_paged_prefill``): the branch Attention._prefill_attention takes when the
    context carries block_tables (engine/model_runner.py:311-314).  The new tokens' K/V rows must already be stored."""
    import numpy as np
    jax, jnp = _jax()
    register()
    t, h, d = q.shape
    nbytes = max(256, int(_lib.load().nvllm_b200_varlen_prefill_workspace_bytes(t, cu_seqlens_q.shape[0] - 1, h,
                                                                               k_cache.shape[2], d)))
    out, _ = jax.ffi.ffi_call("NvllmPagedPrefill", (jax.ShapeDtypeStruct(q.shape, q.dtype),
                                                    jax.ShapeDtypeStruct((nbytes,), jnp.uint8)))(
        q, k_cache, v_cache, cu_seqlens_q.astype(jnp.int32), cu_seqlens_k.astype(jnp.int32),
        block_tables.astype(jnp.int32), scale=np.float32(scale), max_seqlen=np.int32(max_seqlen_q))
    return out


# ---- mode B: caches held outside the traced state, written through a stable device pointer ------------------------
# The functional store above is always correct, but under the reference's outer, non-donating nnx.jit
# (engine/model_runner.py:217-223) XLA may copy each layer's cache every step before the aliased call.  In this mode
# the cache buffers are allocated once by the runner, stay out of the jitted function's operands, and the custom
# calls receive their ADDRESSES as 64-bit attributes and are marked side-effecting: nothing can be copied, nothing is
# rebound.  The buffers must outlive every executable that embeds the addresses; re-allocating the cache means
# re-tracing.  UNVERIFIED like the rest of this module (JAX absent in the build image).

def cache_address(array) -> int:
    """Device address of a committed, single-device jax.Array (its buffer must stay alive while the address is used)."""
    return int(array.unsafe_buffer_pointer())


def store_kv_to_cache_side_effect(key, value, k_cache_addr: int, v_cache_addr: int, num_slots: int, slot_mapping):
    """``store_kv_to_cache`` writing through fixed cache addresses; returns a token array the caller threads into the
    attention call so that XLA keeps the order store -> attend."""
    import numpy as np
    jax, jnp = _jax()
    register()
    call = jax.ffi.ffi_call("NvllmStoreInPlace", jax.ShapeDtypeStruct((1,), jnp.int32), has_side_effect=True)
    return call(key, value, slot_mapping.astype(jnp.int32), k_cache=np.int64(k_cache_addr), v_cache=np.int64(v_cache_addr),
                num_slots=np.int64(num_slots))


def decode_step_side_effect(q, key, value, k_cache_addr: int, v_cache_addr: int, num_blocks: int, num_kv_heads: int,
                            slot_mapping, block_tables, context_lens, scale: float, block_size: int):
    """Store + decode attention (``nvllm_b200_decode_step``) on caches addressed by pointer: one side-effecting call per
    layer and decode step."""
    import numpy as np
    jax, jnp = _jax()
    register()
    b, h, d = q.shape
    nbytes = int(_lib.load().nvllm_b200_paged_decode_workspace_bytes(b, h, num_kv_heads, d, block_tables.shape[1],
                                                                     block_size))
    out, _ = jax.ffi.ffi_call("NvllmDecodeStepInPlace", (jax.ShapeDtypeStruct(q.shape, q.dtype),
                                                         jax.ShapeDtypeStruct((nbytes,), jnp.uint8)),
                              has_side_effect=True)(
        q, key, value, slot_mapping.astype(jnp.int32), block_tables.astype(jnp.int32), context_lens.astype(jnp.int32),
        k_cache=np.int64(k_cache_addr), v_cache=np.int64(v_cache_addr), num_blocks=np.int32(num_blocks),
        block_size=np.int32(block_size), scale=np.float32(scale))
    return out
