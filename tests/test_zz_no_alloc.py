"""nvllm_b200_paged_decode_static -- the decode entry point for callers that cannot allocate.

Some hosts can pass this library only their inputs and outputs and have no way to get scratch memory at
call time (a framework custom-call handler inside a process whose memory pool already owns the GPU's
memory, or a loop that must never hit the device-wide synchronisation of cudaMalloc / cudaFree).  For
them the split-K scratch of the decode kernels is a fixed array inside the library.  This file checks,
through the C ABI, that the entry point gives the same answers as nvllm_b200_paged_decode with a caller
workspace -- on two calls in a row over different batches, so that whatever the first call left in the
shared array is there when the second one runs -- and that sizes beyond the array's capacity are refused.

Both entry points run the same kernels over the same partition of the work, so their outputs must agree bit
for bit; the first batch is also compared with the fp32 oracle directly.

It is named so that pytest collects it last.
"""
import numpy as np
import pytest

from conftest import assert_attention_close, bits_to_torch, torch_to_bits, torch_to_f32

pytestmark = pytest.mark.gpu


def _both_entry_points(w, t):
    import torch
    from nanovllm_jax_b200 import _lib
    lib = _lib.load()
    q = bits_to_torch(t["q_bits"])
    kc, vc = bits_to_torch(t["k_cache_bits"]), bits_to_torch(t["v_cache_bits"])
    bt = torch.from_numpy(w.block_tables).cuda()
    cl = torch.from_numpy(w.context_lens).cuda()
    want = torch.empty_like(q)
    got = torch.full_like(q, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    dims = (w.batch, w.num_heads, w.num_kv_heads, w.head_dim, w.num_blocks, w.block_size, w.max_blocks)
    need = lib.nvllm_b200_paged_decode_workspace_bytes(w.batch, w.num_heads, w.num_kv_heads, w.head_dim, w.max_blocks,
                                                       w.block_size)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    _lib.check(lib.nvllm_b200_paged_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), cl.data_ptr(),
                                           want.data_ptr(), ws.data_ptr(), need, *dims, w.scale, stream))
    _lib.check(lib.nvllm_b200_paged_decode_static(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(),
                                                  cl.data_ptr(), got.data_ptr(), *dims, w.scale, stream))
    torch.cuda.synchronize()
    return got, want


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    from nanovllm_jax_b200 import _lib, workloads
    # First a batch whose long sequences are cut across many CTAs (many partial results land in the array) ...
    w1 = workloads.make_decode_workload("static-1", seed=901, batch=24, num_heads=32, num_kv_heads=8, num_blocks=300,
                                        ctx_lo=1, ctx_hi=3000, max_blocks=12)
    # ... then a smaller one with another head grouping, which finds the first call's leftovers in place.
    w2 = workloads.make_decode_workload("static-2", seed=902, batch=7, num_heads=16, num_kv_heads=2, num_blocks=80,
                                        ctx_lo=1, ctx_hi=2000, max_blocks=8)
    from oracle import reference_attention as ref
    for w in (w1, w2):
        t = workloads.decode_tensors_numpy(w)
        got, want = _both_entry_points(w, t)
        assert np.isfinite(torch_to_f32(got)).all(), "the entry point left rows unwritten"
        assert np.array_equal(torch_to_bits(got), torch_to_bits(want)), w.name
        if w is w1:
            oracle = ref.paged_decode_attention_streamed(t["q"], t["k_cache"], t["v_cache"], w.block_tables,
                                                         w.context_lens, w.scale, w.block_size)
            assert_attention_close(torch_to_f32(got), oracle, w.name)
    assert _lib.device_status() == 0


def test_sizes_beyond_the_built_in_scratch_are_refused():
    import torch
    from nanovllm_jax_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    rc = lib.nvllm_b200_paged_decode_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                            x.data_ptr(), 4097, 8, 2, 128, 4, 256, 2, 0.1, None)
    assert rc == _lib.EWORKSPACE
    text = lib.nvllm_b200_last_error_string()
    assert b"4096" in text and b"nvllm_b200_paged_decode" in text
