"""CPU checks of the drop-in boundary: the shared library loads and exports exactly what the header declares,
the ctypes signatures mirror the header, and argument validation answers without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nvllm_b200_attn.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvllm_b200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from nanovllm_jax_b200.csrc import build
    from nanovllm_jax_b200 import _lib
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    names = _declared()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_ctypes_table_matches_header(lib):
    from nanovllm_jax_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    for name, (_, args) in _lib.SIGNATURES.items():
        m = re.search(name + r"\s*\(([^)]*)\)", text)
        params = [p for p in m.group(1).split(",") if p.strip() not in ("", "void")]
        assert len(params) == len(args), f"{name}: header has {len(params)} parameters, ctypes table {len(args)}"


def test_header_cites_the_reference_for_every_entry_point():
    text = open(HEADER).read()
    for cite in ("layers/attention.py:42-77", "layers/pallas_attention.py:465-507", "layers/attention.py:135-279"):
        assert cite in text


def test_version_and_error_text(lib):
    assert lib.nvllm_b200_version() >= 100
    assert isinstance(lib.nvllm_b200_last_error_string(), bytes)


def test_argument_validation_needs_no_gpu(lib):
    from nanovllm_jax_b200 import _lib
    assert lib.nvllm_b200_store_kvcache(None, None, None, None, None, -1, 8, 128, 16, 0, None) == _lib.EINVAL
    assert lib.nvllm_b200_store_kvcache(None, None, None, None, None, 0, 8, 128, 16, 0, None) == _lib.OK
    assert lib.nvllm_b200_store_kvcache(None, None, None, None, None, 4, 8, 128, 16, 0, None) == _lib.EINVAL
    assert lib.nvllm_b200_paged_decode(None, None, None, None, None, None, None, 0, 4, 8, 2, 64, 4, 256, 2, 0.1,
                                       None) == _lib.EUNSUPPORTED
    assert b"head_dim" in lib.nvllm_b200_last_error_string()
    assert lib.nvllm_b200_paged_decode(None, None, None, None, None, None, None, 0, 4, 8, 2, 128, 4, 100, 2, 0.1,
                                       None) == _lib.EUNSUPPORTED
    assert lib.nvllm_b200_paged_decode(None, None, None, None, None, None, None, 0, 4, 64, 2, 128, 4, 256, 2, 0.1,
                                       None) == _lib.EUNSUPPORTED  # 32 q heads per kv head
    assert lib.nvllm_b200_paged_decode(None, None, None, None, None, None, None, 0, 0, 8, 2, 128, 4, 256, 2, 0.1,
                                       None) == _lib.OK            # empty batch
    assert lib.nvllm_b200_paged_decode(None, None, None, None, None, None, None, 0, 4, 8, 2, 128, 4, 256, 2, 0.1,
                                       None) == _lib.EINVAL        # null pointers
    assert lib.nvllm_b200_varlen_prefill(None, None, None, None, None, None, None, None, 0, 10, 1, 10, 4, 2, 64, 0.1,
                                         None) == _lib.EUNSUPPORTED
    assert lib.nvllm_b200_varlen_prefill(None, None, None, None, None, None, None, None, 0, 0, 0, 10, 4, 2, 128, 0.1,
                                         None) == _lib.OK
    assert lib.nvllm_b200_varlen_prefill(None, None, None, None, None, None, None, None, 0, 10, 1, 10, 4, 2, 128, 0.1,
                                         None) == _lib.EINVAL
    assert lib.nvllm_b200_varlen_prefill_workspace_bytes(33800, 16, 32, 8, 128) % 256 == 0
    assert lib.nvllm_b200_device_status(None) == _lib.EINVAL


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from nanovllm_jax_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError):
        _lib.load()


def test_operators_reject_host_tensors():
    import torch
    from nanovllm_jax_b200 import ops
    x = torch.zeros(2, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        ops.paged_decode(x, x, x, x, x, 0.1, 256)
    with pytest.raises(TypeError):
        ops.store_kvcache(x, x, x, x, torch.zeros(2, dtype=torch.int32))


def test_jax_glue_imports_without_jax_and_names_its_targets():
    """The jax.ffi module is shipped but cannot run here: it must import cleanly, say why it cannot be used, and the
    adapter source must define exactly the handlers it registers, each forwarding to a declared C-ABI entry point."""
    from nanovllm_jax_b200 import jax_ffi
    assert os.path.isfile(jax_ffi.ADAPTER_SOURCE)
    src = open(jax_ffi.ADAPTER_SOURCE).read()
    for name in jax_ffi.TARGETS:
        assert f"XLA_FFI_DEFINE_HANDLER_SYMBOL({name}," in src
    declared = set(_declared())
    for call in ("nvllm_b200_store_kvcache", "nvllm_b200_paged_decode", "nvllm_b200_varlen_prefill"):
        assert call in declared and call + "(" in src
    try:
        import jax  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="JAX"):
            jax_ffi.paged_attention(None, None, None, None, None, 0.1, 256)


def test_header_is_plain_c_and_links_from_a_c_program(lib, tmp_path):
    """The boundary is a C ABI: the header must compile as C99 with no C++ or torch types, and a C program linked
    against the shared library must be able to call it (argument validation only: no GPU needed)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    from nanovllm_jax_b200 import _lib
    src = tmp_path / "host.c"
    src.write_text(
        '#include <stdio.h>\n#include "nvllm_b200_attn.h"\n'
        "int main(void) {\n"
        "    if (nvllm_b200_version() <= 0) return 1;\n"
        "    /* head_dim 64 is outside the supported set: must answer with a code and a message, not crash */\n"
        "    int rc = nvllm_b200_store_kvcache(0, 0, 0, 0, 0, 4, 8, 64, 1024, 0, 0);\n"
        '    printf("%d %s\\n", rc, nvllm_b200_last_error_string());\n'
        "    return rc < 0 ? 0 : 2;\n"
        "}\n")
    exe = tmp_path / "host"
    libdir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(ROOT, "include"),
                    str(src), "-o", str(exe), "-L", libdir, "-l:libnvllm_b200_attn.so", f"-Wl,-rpath,{libdir}"],
                   check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stdout + out.stderr
    code, _, text = out.stdout.strip().partition(" ")
    assert int(code) < 0 and len(text) > 0
