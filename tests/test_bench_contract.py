"""bench.py on CPU: the reference arm runs without a GPU and prints one JSON line with the contract's keys; the
workload bookkeeping (bytes, page sets) is consistent."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.strip().splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_prints_the_contract_line():
    d = _run("--impl", "reference", "--workload", "cfg1", "--steps", "2", "--warmup", "3")
    assert d["impl"] == "reference" and d["metric"] == "paged_decode_attn_hbm_gbps" and d["unit"] == "GB/s"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["steps"] == 2 and d["warmup"] == 3 and d["vs_baseline"] is None and d["higher_is_better"] is True
    assert d["value"] > 0 and d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"] == d["e2e"]["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"] and "model" not in d["config"]


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "cfg1",
                          "--gpus", "2", "--steps", "1", "--warmup", "3"], capture_output=True, text=True, timeout=300,
                         cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_page_sets_are_disjoint_and_bytes_add_up():
    sys.path.insert(0, ROOT)
    import bench
    from nanovllm_jax_b200 import workloads
    w = workloads.config2()
    sets = bench.page_sets(w)
    assert len(sets) == 3
    used = [set(t[t >= 0].tolist()) for t, _ in sets]
    assert not (used[0] & used[1]) and not (used[1] & used[2]) and not (used[0] & used[2])
    for tables, slots in sets:
        assert np.array_equal((tables >= 0).sum(axis=1), [len(bl) for bl in w.block_lists])
        last = tables[np.arange(w.batch), (w.context_lens - 1) // 256]
        assert np.array_equal(slots, last * 256 + (w.context_lens - 1) % 256)
    ctx = int(w.context_lens.astype(np.int64).sum())
    assert w.kv_bytes() == ctx * 8 * 128 * 4 + 2 * 64 * 32 * 128 * 2 + 4 * (sum(len(b) for b in w.block_lists) + 64)
    assert w.kv_bytes(4) < w.kv_bytes() and workloads.config4().flops() > 9e11


def test_step_inputs_are_views_of_one_buffer_and_one_copy_moves_them_all():
    """The end-to-end step moves q, k, v and the index tensors with ONE host -> device copy: every device tensor must
    alias the device buffer, keep its dtype / shape / contiguity, and change when the flat buffer is overwritten."""
    import torch
    sys.path.insert(0, ROOT)
    import bench
    w = bench.pick_workload("cfg1", None)
    sets = bench.page_sets(w)
    host, devflat, devin = bench.make_step_inputs(w, sets, 16, 8, "cpu", pin=False)
    assert len(host) == len(devflat) == len(devin) == len(sets)
    for (tables, slots), hflat, dflat, views in zip(sets, host, devflat, devin):
        q, k, v, sl, cl, bt = views
        assert q.shape == (w.batch, 16, w.head_dim) and q.dtype == torch.bfloat16 and q.is_contiguous()
        assert k.shape == v.shape == (w.batch, 8, w.head_dim)
        assert sl.dtype == cl.dtype == bt.dtype == torch.int32
        assert np.array_equal(sl.numpy(), slots) and np.array_equal(bt.numpy(), tables)
        assert np.array_equal(cl.numpy(), w.context_lens.astype(np.int32))
        lo, hi = dflat.data_ptr(), dflat.data_ptr() + dflat.numel()
        for t in views:
            assert lo <= t.data_ptr() and t.data_ptr() + t.numel() * t.element_size() <= hi
            assert (t.data_ptr() - lo) % 256 == 0
        assert torch.equal(dflat, hflat)
        before = q.clone()
        hflat.zero_()
        dflat.copy_(hflat)  # the single copy of the end-to-end step
        assert not torch.equal(q, before) and int(sl.abs().sum()) == 0 and int(bt.abs().sum()) == 0
