#!/usr/bin/env python
"""Benchmark of the paged-attention decode step (store_kvcache + paged decode) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload cfg2|cfg3|cfg1|cfg4] [--scaling weak|strong]

One step = one decode-attention pass over one batch: the step's new K/V rows are scattered into the
paged cache by slot and every sequence attends over its pages -- what ``Attention.__call__`` does for
one layer in the decode phase.  The default workload is the Qwen3-8B batch-64 configuration
(32 q heads / 8 kv heads, head_dim 128, ctx U[512, 8192], block 256, pool of 4096 blocks) on synthetic
N(0,1) bf16 data.

Prints ONE JSON line (rank 0).  ``value`` is aggregate algorithmic GB/s with everything resident in
HBM; ``e2e`` is the same metric through the ``Attention`` layer with the step's inputs coming from
pinned host memory and the result copied back to the host inside the timed region (the KV cache is
device-resident state, not a step input, exactly as in the reference engine).  ``roofline`` times the
decode kernels alone with CUDA events inside the timed loop.  ``cpu_baseline`` is the reference's own
algorithm restated for the host cores (``oracle/``), timed on a bounded sample.

``--workload cfg4`` switches to the prefill step (store_kvcache of all prompt tokens + varlen causal attention,
16 packed Qwen3-8B sequences) and reports TFLOP/s against the bf16 tensor roofline.

``--impl reference`` times that CPU restatement alone, on rank 0, each step a bounded sample of the
same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "paged_decode_attn_hbm_gbps"
UNIT = "GB/s"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu captures
# summarised in profiles/paged_decode_cfg2_qwen3-8b_b64.md and profiles/varlen_prefill_cfg4_qwen3-8b_16seq.md
# (a property of the launch, independent of the page-pool size the capture used); None where no capture exists.
NCU_TRAFFIC_BYTES = {"cfg2": 1_021_617_440, "cfg4": 1_380_623_264}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML every `period` seconds."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period: float = 0.005):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v for v in visible.split(",") if v.strip() != ""]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None
        self.period = period

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# workload
# ----------------------------------------------------------------------------------------------
def pick_workload(name: str, pool_blocks: int | None = None):
    from nanovllm_jax_b200 import workloads
    if name == "cfg1":
        return workloads.config1()
    fn = {"cfg2": workloads.config2, "cfg3": workloads.config3}[name]
    return fn() if not pool_blocks else fn(num_blocks=pool_blocks)


def page_sets(w, max_sets: int = 3):
    """Disjoint physical page assignments for the same sequences, rotated between steps so that no step
    finds its pages in L2 from the previous one.  Returns a list of (block_tables, slot_mapping)."""
    need = [len(bl) for bl in w.block_lists]
    total = sum(need)
    sets = max(1, min(max_sets, w.num_blocks // max(total, 1)))
    rng = np.random.Generator(np.random.PCG64(w.seed + 77))
    perm = rng.permutation(w.num_blocks).astype(np.int32)
    out, pos = [], 0
    for _ in range(sets):
        tables = np.full_like(w.block_tables, -1)
        slots = np.empty(w.batch, dtype=np.int32)
        for b, n in enumerate(need):
            ids = perm[pos:pos + n]
            pos += n
            tables[b, :n] = ids
            ctx = int(w.context_lens[b])
            slots[b] = int(ids[-1]) * w.block_size + (ctx - (n - 1) * w.block_size) - 1
        out.append((tables, slots))
    return out


def fill_normal_bf16(t, gen):
    import torch
    flat = t.view(-1)
    step = 1 << 27
    for i in range(0, flat.numel(), step):
        n = min(step, flat.numel() - i)
        flat[i:i + n] = torch.randn(n, generator=gen, device=t.device, dtype=torch.float32).to(t.dtype)


# ----------------------------------------------------------------------------------------------
# CPU baseline (the oracle as the timed thing -- the only place bench.py runs it)
# ----------------------------------------------------------------------------------------------
class CpuReference:
    """Times the torch-CPU restatement of the reference's decode path on (sequence, kv head) samples."""

    def __init__(self, w, kvh_total: int):
        import torch
        self.torch = torch
        self.w = w
        self.kvh_total = kvh_total
        self.g = w.num_heads // w.num_kv_heads
        self.threads = torch.get_num_threads()
        gen = torch.Generator()
        gen.manual_seed(w.seed + 9)
        self.gen = gen
        self._cache = {}

    def _inputs(self, n_seqs: int, n_kvh: int):
        key = (n_seqs, n_kvh)
        if key not in self._cache:
            torch, w = self.torch, self.w
            self._cache.clear()
            # compact pool holding just the pages of the sampled sequences
            lists, pos = [], 0
            for b in range(n_seqs):
                n = len(w.block_lists[b])
                lists.append(list(range(pos, pos + n)))
                pos += n
            tables = np.full((n_seqs, w.max_blocks), -1, dtype=np.int32)
            for b, bl in enumerate(lists):
                tables[b, : len(bl)] = bl
            shape = (max(pos, 1), w.block_size, n_kvh, w.head_dim)
            kc = torch.randn(shape, generator=self.gen, dtype=torch.float32).bfloat16()
            vc = torch.randn(shape, generator=self.gen, dtype=torch.float32).bfloat16()
            q = torch.randn((n_seqs, n_kvh * self.g, w.head_dim), generator=self.gen).bfloat16()
            k_new = torch.randn((n_seqs, n_kvh, w.head_dim), generator=self.gen).bfloat16()
            slots = torch.tensor([bl[-1] * w.block_size + (int(w.context_lens[b]) - (len(bl) - 1) * w.block_size) - 1
                                  for b, bl in enumerate(lists)], dtype=torch.int32)
            ctx = torch.from_numpy(w.context_lens[:n_seqs].copy())
            self._cache[key] = (q, k_new, kc, vc, torch.from_numpy(tables), ctx, slots)
        return self._cache[key]

    def sample_bytes(self, n_seqs: int, n_kvh: int) -> int:
        w = self.w
        ctx = int(w.context_lens[:n_seqs].astype(np.int64).sum())
        return ctx * n_kvh * w.head_dim * 4 + 2 * n_seqs * n_kvh * self.g * w.head_dim * 2

    def step(self, n_seqs: int, n_kvh: int) -> float:
        from oracle import reference_attention_torch as reft
        q, k_new, kc, vc, tables, ctx, slots = self._inputs(n_seqs, n_kvh)
        w = self.w
        t0 = time.perf_counter()
        flat = (kc.shape[0] * w.block_size, n_kvh, w.head_dim)
        kc2, vc2 = reft.store_kv_to_cache(k_new, k_new, kc.view(flat), vc.view(flat), slots)
        reft.paged_decode_attention_vectorized(q, kc2.view(kc.shape), vc2.view(vc.shape), tables, ctx, w.scale,
                                               w.block_size)
        return time.perf_counter() - t0

    def plan(self, budget_s: float):
        """Pick (n_seqs, n_kvh) so one step costs about ``budget_s`` seconds."""
        t1 = min(self.step(1, 1), self.step(1, 1))
        n_kvh = int(max(1, min(self.kvh_total, budget_s / max(t1, 1e-6))))
        n_seqs = int(max(1, min(self.w.batch, 8, budget_s / max(t1 * n_kvh, 1e-6))))  # <= 8: bounds host RAM
        if n_kvh < self.kvh_total:
            n_seqs = 1
        return n_seqs, n_kvh


def cpu_baseline_leg(w, kvh_local: int, target_s: float = 12.0):
    """Times the CPU restatement on a bounded sample: as many passes over the sample as fit in about ``target_s``."""
    ref = CpuReference(w, kvh_local)
    n_seqs, n_kvh = ref.plan(target_s)
    first = ref.step(n_seqs, n_kvh)  # untimed: first touch of the sample's pages
    passes = int(max(1, min(40, target_s / max(first, 1e-3))))
    dt = sum(ref.step(n_seqs, n_kvh) for _ in range(passes)) / passes
    return {"value": ref.sample_bytes(n_seqs, n_kvh) / dt / 1e9, "unit": UNIT, "cores": ref.threads, "kind": "port",
            "sample": f"restated reference jnp path (torch CPU, fp32 math, padded gather + GQA repeat as "
                      f"layers/pallas_attention.py:185-238) on the first {n_seqs} of {w.batch} sequences x {n_kvh} of "
                      f"{kvh_local} kv heads, mean of {passes} timed passes of {dt:.2f} s; JAX itself is not installed"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = pick_workload(args.workload, args.pool_blocks)
    ref = CpuReference(w, w.num_kv_heads)
    total_steps = args.steps + args.warmup
    n_seqs, n_kvh = ref.plan(min(20.0, 150.0 / max(total_steps, 1)))
    for _ in range(args.warmup):
        ref.step(n_seqs, n_kvh)
    t = 0.0
    for _ in range(args.steps):
        t += ref.step(n_seqs, n_kvh)
    ms = t / max(args.steps, 1) * 1e3
    value = ref.sample_bytes(n_seqs, n_kvh) / (ms / 1e3) / 1e9
    sample = (f"restated reference jnp path (torch CPU) per step on the first {n_seqs} of {w.batch} sequences x "
              f"{n_kvh} of {w.num_kv_heads} kv heads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(w, args, 1, w.num_kv_heads, None),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": ref.threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(w, args, n_gpus, kvh_local, n_sets):
    return {"workload": f"{w.name}: paged decode attention, {w.num_heads} q heads / {w.num_kv_heads} kv heads, "
                        f"head_dim {w.head_dim}, batch {w.batch}, ctx {int(w.context_lens.min())}.."
                        f"{int(w.context_lens.max())} (mean {float(w.context_lens.mean()):.0f}), block {w.block_size}, "
                        f"pool {w.num_blocks} blocks, plus store_kvcache of {w.batch} new tokens",
            "kv_heads_per_gpu": kvh_local, "q_heads_per_gpu": kvh_local * (w.num_heads // w.num_kv_heads),
            "parallelism": f"kv-head shards x{n_gpus}, no collective in the path",
            "l2": (f"{n_sets} disjoint page sets rotated between steps; each step streams "
                   f"{w.kv_bytes(kvh_local) / 1e6:.0f} MB > 126 MB L2") if n_sets else None,
            "seed": w.seed}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def make_step_inputs(w, sets, h, kvh, dev, pin):
    """Per page set: the step's inputs (q, k, v, slot_mapping, context_lens, block_tables) laid out in ONE host buffer
    and ONE device buffer, so that the end-to-end step moves them with a single host -> device copy.
    Returns (host_flats, device_flats, device_views) with device_views[s] = (q, k, v, slots, ctx, tables)."""
    import torch
    from nanovllm_jax_b200.utils.staging import packed_like
    host, devflat, devin = [], [], []
    cl_np = w.context_lens.astype(np.int32)
    for tables, slots in sets:
        src = (torch.randn((w.batch, h, w.head_dim), dtype=torch.float32).bfloat16(),
               torch.randn((w.batch, kvh, w.head_dim), dtype=torch.float32).bfloat16(),
               torch.randn((w.batch, kvh, w.head_dim), dtype=torch.float32).bfloat16(),
               torch.from_numpy(np.ascontiguousarray(slots, dtype=np.int32)),
               torch.from_numpy(cl_np.copy()),
               torch.from_numpy(np.ascontiguousarray(tables, dtype=np.int32)))
        hflat, hviews = packed_like(src, "cpu", pin=pin)
        for dst, x in zip(hviews, src):
            dst.copy_(x)
        dflat, dviews = packed_like(src, dev)
        dflat.copy_(hflat)
        host.append(hflat)
        devflat.append(dflat)
        devin.append(tuple(dviews))
    return host, devflat, devin


def run_b200(args):
    import torch
    import torch.distributed as dist
    from nanovllm_jax_b200 import _lib, ops
    from nanovllm_jax_b200.layers.attention import Attention
    from nanovllm_jax_b200.utils.context import create_decode_context

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()  # fail loudly before anything is timed

    w = pick_workload(args.workload, args.pool_blocks)
    g = w.num_heads // w.num_kv_heads
    if args.scaling == "strong":
        if w.num_kv_heads % world:
            raise SystemExit("strong scaling needs kv heads divisible by the GPU count")
        kvh = w.num_kv_heads // world
    else:
        kvh = w.num_kv_heads  # weak: every GPU holds a full 8-kv-head shard
    h = kvh * g
    sets = page_sets(w)
    n_sets = len(sets)

    gen = torch.Generator(device=dev)
    gen.manual_seed(w.seed * 100 + rank)
    shape = (w.num_blocks, w.block_size, kvh, w.head_dim)
    kc = torch.empty(shape, dtype=torch.bfloat16, device=dev)
    vc = torch.empty(shape, dtype=torch.bfloat16, device=dev)
    fill_normal_bf16(kc, gen)
    fill_normal_bf16(vc, gen)
    attn = Attention(h, w.head_dim, w.scale, kvh, w.block_size)
    attn.set_kv_cache(kc, vc)

    host, devflat, devin = make_step_inputs(w, sets, h, kvh, dev, pin=True)
    ctxs = [create_decode_context(context_lens=d[4], slot_mapping=d[3], block_tables=d[5]) for d in devin]
    out = torch.empty((w.batch, h, w.head_dim), dtype=torch.bfloat16, device=dev)
    out_host = torch.empty((w.batch, h, w.head_dim), dtype=torch.bfloat16).pin_memory()

    step_bytes = w.kv_bytes(kvh) + w.batch * (kvh * w.head_dim * 2 * 2 * 2 + 4)
    decode_bytes = w.kv_bytes(kvh)

    def step(i):
        s = i % n_sets
        q, k, v, _, _, _ = devin[s]
        return attn(q, k, v, ctxs[s])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()

    # --- timed region: K steps, device-resident inputs -----------------------------------------
    # The decode kernels alone are timed on every 8th step only: an event between two kernels keeps the
    # second from overlapping its launch with the first, so the other steps run as a user's would.
    ev_every = 8
    n_ev = min((args.steps + ev_every - 1) // ev_every, 1024)
    ev_a = [torch.cuda.Event(enable_timing=True) for _ in range(n_ev)]
    ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(n_ev)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flat = (w.num_blocks * w.block_size, kvh, w.head_dim)
    kflat, vflat = kc.view(flat), vc.view(flat)
    with ClockSampler(local) as clocks:
        t_start.record()
        for i in range(args.steps):
            s = i % n_sets
            q, k, v, sl, cl, bt = devin[s]
            ops.store_kvcache(k, v, kflat, vflat, sl)
            timed = (i % ev_every == 0) and (i // ev_every < n_ev)
            if timed:
                ev_a[i // ev_every].record()
            ops.paged_decode(q, kc, vc, bt, cl, w.scale, w.block_size, out=out)
            if timed:
                ev_b[i // ev_every].record()
        t_end.record()
        torch.cuda.synchronize()
    elapsed_ms = t_start.elapsed_time(t_end)
    decode_samples = [a.elapsed_time(b) for a, b in zip(ev_a, ev_b)]
    decode_ms = float(np.mean(decode_samples)) if n_ev else float("nan")
    # spread of the kernel-only samples on this rank: [p10, median, p90] in microseconds
    decode_pct = [float(x) * 1e3 for x in np.percentile(decode_samples, [10, 50, 90])] if n_ev else None
    if world > 1:
        t = torch.tensor([elapsed_ms, decode_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, decode_ms = float(t[0]), float(t[1])
    barrier()
    status = _lib.device_status()

    # --- end to end: host inputs in, host result out, every step --------------------------------
    e2e_steps = max(1, min(args.steps, 300))
    h2d = host[0].numel()  # one packed copy: q, k, v, slot_mapping, context_lens, block_tables (256-byte aligned slices)
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step(i):
        s = i % n_sets
        devflat[s].copy_(host[s], non_blocking=True)
        o = attn(devin[s][0], devin[s][1], devin[s][2], ctxs[s])
        out_host.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0])
    barrier()

    if rank == 0:
        peak, peak_kind = load_peaks()
        ms_per_step = elapsed_ms / args.steps
        achieved = decode_bytes / (decode_ms / 1e3) / 1e9
        line = {
            "metric": METRIC, "value": world * step_bytes / (ms_per_step / 1e3) / 1e9, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(w, args, world, kvh, n_sets),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                         "kernel": "paged_decode_kernel + paged_decode_merge_kernel (one C-ABI call)",
                         "bytes_per_launch": decode_bytes, "us_per_launch": decode_ms * 1e3,
                         "us_per_launch_p10_p50_p90": decode_pct, "launches_timed": n_ev,
                         "peak_kind": f"{peak_kind} copy bandwidth", "frac_of_nominal_8tbs": achieved / 8000.0},
            "e2e": {"value": world * step_bytes / (e2e_ms / 1e3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "what": "Attention.__call__ with q/k/v/slot_mapping/context_lens/block_tables copied from pinned "
                            "host memory (one packed copy) and the output copied back, stream-synchronised every "
                            "step; the KV cache stays in HBM"},
            "clocks": clocks.summary(), "gpu_launches": 3 * args.steps, "device_status": status,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg(w, kvh)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------
# prefill workload (cfg4): metric = causal attention TFLOP/s, tensor-core roofline
# ----------------------------------------------------------------------------------------------
PREFILL_METRIC, PREFILL_UNIT = "varlen_prefill_tflops", "TFLOP/s"


def prefill_cpu_sample(w, budget_s: float):
    """Times the torch-CPU restatement of the reference prefill on the shortest sequences that fit the budget."""
    import torch
    from oracle import reference_attention_torch as reft
    order = np.argsort(w.seq_lens)
    gen = torch.Generator()
    gen.manual_seed(w.seed)
    used, flops, t_total = [], 0, 0.0
    for b in order:
        n = int(w.seq_lens[b])
        est = 4 * w.head_dim * w.num_heads * n * (n + 1) // 2
        q = torch.randn((n, w.num_heads, w.head_dim), generator=gen).bfloat16()
        k = torch.randn((n, w.num_kv_heads, w.head_dim), generator=gen).bfloat16()
        v = torch.randn((n, w.num_kv_heads, w.head_dim), generator=gen).bfloat16()
        t0 = time.perf_counter()
        reft.variable_length_attention_prefill(q, k, v, [0, n], w.num_heads, w.num_kv_heads, w.scale)
        dt = time.perf_counter() - t0
        used.append(n)
        flops += est
        t_total += dt
        if t_total > budget_s:
            break
    return flops / t_total / 1e12, used, t_total, torch.get_num_threads()


def prefill_config(w, world, h, kvh):
    return {"workload": f"{w.name}: varlen causal prefill attention, {w.num_heads} q heads / {w.num_kv_heads} kv heads, "
                        f"head_dim {w.head_dim}, {w.batch} packed sequences of {int(w.seq_lens.min())}.."
                        f"{int(w.seq_lens.max())} tokens (T = {w.total_tokens}), plus store_kvcache of all T tokens "
                        f"(block {w.block_size})",
            "kv_heads_per_gpu": kvh, "q_heads_per_gpu": h,
            "parallelism": f"kv-head shards x{world}, no collective in the path",
            "l2": f"q/k/v/out of one step are {(2 * h + 2 * kvh) * w.total_tokens * w.head_dim * 2 / 1e6:.0f} MB "
                  f"> 126 MB L2; K/V tile reuse inside a step is meant to hit L2",
            "seed": w.seed}


def run_prefill(args):
    import torch
    import torch.distributed as dist
    from nanovllm_jax_b200 import _lib, ops, workloads
    from nanovllm_jax_b200.layers.attention import Attention
    from nanovllm_jax_b200.utils.context import create_prefill_context

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    w = workloads.config4()
    if args.impl == "reference":
        if rank != 0:
            return
        budget = min(20.0, 150.0 / max(args.steps + args.warmup, 1))
        vals = [prefill_cpu_sample(w, budget) for _ in range(min(args.steps + args.warmup, 3))]
        tf, used, dt, threads = vals[-1]
        sample = f"restated reference prefill (torch CPU, fp32) on the {len(used)} shortest sequences ({used} tokens)"
        print(json.dumps({"impl": "reference", "metric": PREFILL_METRIC, "value": tf, "unit": PREFILL_UNIT,
                          "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
                          "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16",
                          "data": "synthetic", "config": prefill_config(w, 1, w.num_heads, w.num_kv_heads),
                          "cpu_baseline": {"value": tf, "unit": PREFILL_UNIT, "cores": threads, "kind": "port",
                                           "sample": sample},
                          "e2e": {"value": tf, "unit": PREFILL_UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                          "gpu_launches": 0}), flush=True)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    g = w.num_heads // w.num_kv_heads
    kvh = w.num_kv_heads // world if args.scaling == "strong" else w.num_kv_heads
    h = kvh * g
    t = w.total_tokens
    gen = torch.Generator(device=dev)
    gen.manual_seed(w.seed * 100 + rank)
    q = torch.empty((t, h, w.head_dim), dtype=torch.bfloat16, device=dev)
    k = torch.empty((t, kvh, w.head_dim), dtype=torch.bfloat16, device=dev)
    v = torch.empty_like(k)
    for x in (q, k, v):
        fill_normal_bf16(x, gen)
    kc = torch.zeros((w.num_blocks, w.block_size, kvh, w.head_dim), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    attn = Attention(h, w.head_dim, w.scale, kvh, w.block_size)
    attn.set_kv_cache(kc, vc)
    cu = torch.from_numpy(w.cu_seqlens).to(dev)
    slots = torch.from_numpy(w.slot_mapping).to(dev)
    ctx = create_prefill_context(cu, cu, int(w.seq_lens.max()), int(w.seq_lens.max()), slots,
                                 cu_seqlens_host=w.cu_seqlens)
    out = torch.empty_like(q)
    flat = (w.num_blocks * w.block_size, kvh, w.head_dim)
    flops = w.flops(h)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        attn(q, k, v, ctx)
    barrier()
    ev_every = 4
    n_ev = (args.steps + ev_every - 1) // ev_every
    ev_a = [torch.cuda.Event(enable_timing=True) for _ in range(n_ev)]
    ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(n_ev)]
    t0e, t1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        t0e.record()
        for i in range(args.steps):
            ops.store_kvcache(k, v, kc.view(flat), vc.view(flat), slots)
            if i % ev_every == 0:
                ev_a[i // ev_every].record()
            ops.varlen_prefill(q, k, v, cu, int(w.seq_lens.max()), w.scale, out=out, cu_seqlens_host=w.cu_seqlens)
            if i % ev_every == 0:
                ev_b[i // ev_every].record()
        t1e.record()
        torch.cuda.synchronize()
    elapsed_ms = t0e.elapsed_time(t1e)
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in zip(ev_a, ev_b)]))
    if world > 1:
        tt = torch.tensor([elapsed_ms, kern_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms, kern_ms = float(tt[0]), float(tt[1])
    barrier()
    status = _lib.device_status()

    hq, hk, hv = (x.cpu().pin_memory() for x in (q, k, v))
    hout = torch.empty_like(hq).pin_memory()
    e2e_steps = max(1, min(args.steps, 10))

    def e2e_step():
        q.copy_(hq, non_blocking=True)
        k.copy_(hk, non_blocking=True)
        v.copy_(hv, non_blocking=True)
        o = attn(q, k, v, ctx)
        hout.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()
    barrier()
    tw = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_ms = (time.perf_counter() - tw) / e2e_steps * 1e3
    if world > 1:
        tt = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt[0])
    barrier()
    if rank == 0:
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peak, kind = float(json.load(f)["bf16_tflops_sustained"]), "measured sustained cuBLAS bf16"
        except Exception:
            peak, kind = 1400.0, "fallback sustained"
        ms = elapsed_ms / args.steps
        achieved = flops / (kern_ms / 1e3) / 1e12
        line = {"metric": PREFILL_METRIC, "value": world * flops / (ms / 1e3) / 1e12, "unit": PREFILL_UNIT,
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": prefill_config(w, world, h, kvh),
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                             "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get("cfg4"),
                             "kernel": "prefill_plan_kernel + varlen_prefill_kernel (one C-ABI call)",
                             "flops_per_launch": flops, "us_per_launch": kern_ms * 1e3, "peak_kind": kind},
                "e2e": {"value": world * flops / (e2e_ms / 1e3) / 1e12, "unit": PREFILL_UNIT,
                        "h2d_bytes_per_step": sum(x.numel() * 2 for x in (hq, hk, hv)),
                        "d2h_bytes_per_step": hout.numel() * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                        "what": "Attention.__call__ (store_kvcache + varlen prefill) with q/k/v copied from pinned host "
                                "memory and the output copied back every step"},
                "clocks": clocks.summary(), "gpu_launches": 3 * args.steps, "device_status": status}
        if world == 1 and not args.no_cpu_baseline:
            tf, used, dt, threads = prefill_cpu_sample(w, 12.0)
            line["cpu_baseline"] = {"value": tf, "unit": PREFILL_UNIT, "cores": threads, "kind": "port",
                                    "sample": f"restated reference prefill (torch CPU, fp32) on the {len(used)} shortest "
                                              f"sequences ({used} tokens), {dt:.1f} s; JAX itself is not installed"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", choices=["cfg1", "cfg2", "cfg3", "cfg4"], default="cfg2")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--pool-blocks", type=int, default=0,
                    help="shrink the physical page pool (same sequences); for profiler captures only")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_prefill(args) if args.workload == "cfg4" else run_reference(args)
    if args.gpus > 1 and "RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__)] + sys.argv[1:]
        os.execv(sys.executable, cmd)
    if args.workload == "cfg4":
        if args.steps == 1000:
            args.steps = 100  # default sized for the decode step; a prefill step is ~10x longer
        return run_prefill(args)
    run_b200(args)


if __name__ == "__main__":
    main()
