"""ctypes binding of libnvllm_b200_attn.so (the C ABI declared in include/nvllm_b200_attn.h).

There is no fallback: if the shared library is missing, ``load()`` raises and so does every
operator of this package.  Build it with ``python -m nanovllm_jax_b200.csrc.build``.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
# NVLLM_B200_LIB points the package at another build of the same library (e.g. a candidate kernel under test).
LIB_PATH = os.environ.get("NVLLM_B200_LIB") or os.path.join(_HERE, "libnvllm_b200_attn.so")

OK, EINVAL, EUNSUPPORTED, EWORKSPACE, ECUDA, EDRIVER = 0, -1, -2, -3, -4, -5
DTYPE_BF16, DTYPE_F32 = 0, 1

_c = ctypes
_vp, _i32, _i64, _sz, _f32 = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_size_t, _c.c_float

# name -> (restype, argtypes); mirrors include/nvllm_b200_attn.h one to one.
SIGNATURES = {
    "nvllm_b200_version": (_i32, []),
    "nvllm_b200_last_error_string": (_c.c_char_p, []),
    "nvllm_b200_store_kvcache": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i64, _i32, _vp]),
    "nvllm_b200_paged_decode_workspace_bytes": (_sz, [_i32] * 6),
    "nvllm_b200_paged_decode": (_i32, [_vp] * 7 + [_sz] + [_i32] * 7 + [_f32, _vp]),
    "nvllm_b200_decode_step": (_i32, [_vp] * 10 + [_sz] + [_i32] * 7 + [_f32, _i32, _vp]),
    "nvllm_b200_paged_decode_static": (_i32, [_vp] * 6 + [_i32] * 7 + [_f32, _vp]),
    "nvllm_b200_device_status": (_i32, [_c.POINTER(_i32)]),
    "nvllm_b200_varlen_prefill_workspace_bytes": (_sz, [_i64, _i32, _i32, _i32, _i32]),
    "nvllm_b200_varlen_prefill": (_i32, [_vp] * 8 + [_sz, _i64, _i32, _i32, _i32, _i32, _i32, _f32, _vp]),
    "nvllm_b200_paged_prefill": (_i32, [_vp] * 9 + [_sz, _i64] + [_i32] * 8 + [_f32, _vp]),
    "nvllm_b200_device_status_reset": (_i32, []),
    "nvllm_b200_comm_buffer_bytes": (_sz, [_sz]),
    "nvllm_b200_comm_alloc": (_i32, [_sz, _c.POINTER(_vp), _vp]),
    "nvllm_b200_comm_open": (_i32, [_vp, _c.POINTER(_vp)]),
    "nvllm_b200_comm_close": (_i32, [_vp]),
    "nvllm_b200_comm_free": (_i32, [_vp]),
    "nvllm_b200_allreduce_sum": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i64, _sz, _c.c_uint, _i64, _vp]),
    "nvllm_b200_allreduce_sum_emulated": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, _sz, _c.c_uint, _i64, _vp]),
    "nvllm_b200_qk_norm_rope_store": (_i32, [_vp] * 10 + [_i64, _i32, _i32, _i32, _i64, _i64, _f32, _vp]),
    "nvllm_b200_fused_decode_step": (_i32, [_vp] * 7 + [_i64, _f32] + [_vp] * 7 + [_sz] + [_i32] * 7 + [_f32, _vp]),
}

_lock = threading.Lock()
_lib = None


class NvllmError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"nvllm_b200 error {code}: {text}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the shared library once and attach the C signatures.  Raises if it is absent."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise ImportError(
                    f"{LIB_PATH} not found: the CUDA library has not been built "
                    "(run `python -m nanovllm_jax_b200.csrc.build`); there is no fallback path")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise NvllmError(code, load().nvllm_b200_last_error_string().decode("utf-8", "replace"))


def device_status() -> int:
    flags = _i32(0)
    check(load().nvllm_b200_device_status(ctypes.byref(flags)))
    return int(flags.value)


def device_status_reset() -> None:
    check(load().nvllm_b200_device_status_reset())
