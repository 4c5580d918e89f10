#!/usr/bin/env python
"""Benchmark of the paged-attention decode step (store_kvcache + paged decode) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload auto|cfg1|cfg2|cfg3|cfg4] [--scaling auto|weak|strong] [--shard-of TP]

One step = one decode-attention pass over one batch: the step's new K/V rows are scattered into the
paged cache by slot and every sequence attends over its pages -- what ``Attention.__call__`` does for
one layer in the decode phase.

Workloads.  With one GPU the step runs the Qwen3-8B batch-64 configuration (32 q heads / 8 kv heads,
head_dim 128, ctx U[512, 8192], block 256, pool of 4096 blocks).  With N > 1 GPUs it runs the Qwen3-32B
skewed batch-256 configuration (64 q heads / 8 kv heads, ctx log-U[16, 32768]) with its 8 kv heads cut
across the N ranks (``scaling: "strong"``, 8/N kv heads and 64/N q heads per GPU; no collective is in the
path), and every rank re-computes four sequences of its shard with the CPU oracle after the timed
region (``parity``).  ``--workload`` / ``--scaling`` override the choice; ``--shard-of TP`` runs rank 0's
shard of a TP-way split on one GPU (the shards share nothing, so this is what one GPU of TP does).

Prints ONE JSON line (rank 0):
  value        aggregate algorithmic GB/s of the step with everything resident in HBM.  The block of K
               steps the driver asked for is repeated until at least ``--min-seconds`` of GPU time have
               passed (a 20-step block lasts 3 ms: too short to time or to sample clocks over);
               ``ms_per_step`` is total time / total steps, max over ranks, ``blocks`` says how many ran.
  roofline     the decode C call alone (clear + main kernel), timed in its own pass of back-to-back
               launches after warm-up, page sets rotated: one event pair around the pass gives the mean
               the fraction is computed from, a second pass with an event pair per launch gives
               p10 / p50 / p90.
  e2e          the same step through ``Attention.__call__`` with the step's inputs copied from pinned host
               memory and the result copied back inside the timed region (the KV cache is device state).
  secondary    (one GPU only) the other workloads, each timed the same way: Qwen3-32B decode, the
               16-sequence Qwen3-8B prefill (TFLOP/s against the sustained and the burst bf16 peak) and
               store_kvcache at the prefill's size.
  cpu_baseline the reference's own algorithm restated for the host cores (``oracle/``) on a bounded sample.

``--workload cfg4`` makes the prefill step the headline instead (metric ``varlen_prefill_tflops``).
``--impl reference`` times the CPU restatement alone, on rank 0, with all host cores, each step a
bounded sample of the same workload and the same ``config``.
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
PREFILL_METRIC, PREFILL_UNIT = "varlen_prefill_tflops", "TFLOP/s"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (a property of the launch, independent of the page-pool size the capture used);
# None where no capture exists.
NCU_TRAFFIC_BYTES = {"cfg2": 1_021_858_480, "cfg4": 1_781_467_008}


def load_peaks():
    """(hbm GB/s, sustained bf16 TFLOP/s, burst bf16 TFLOP/s, kind)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1400.0, 1590.0, "fallback"


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML every `period` seconds (read-only)."""

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
def resolve(args, world: int):
    """(workload name, scaling, tp, kv heads per GPU are derived later): what `auto` means for this GPU count.
    Both arms call this, so they always agree on the configuration."""
    name, scaling = args.workload, args.scaling
    if name == "auto":
        name = "cfg2" if world == 1 and not args.shard_of else "cfg3"
    if scaling == "auto":
        scaling = "strong" if (world > 1 and name == "cfg3") or args.shard_of else "weak"
    tp = args.shard_of if args.shard_of else (world if scaling == "strong" else 1)
    return name, scaling, tp


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


def workload_config(w, world: int, tp: int, scaling: str):
    """The `config` object of the JSON line; a pure function of the workload and the split, so that both arms
    print the same one."""
    kvh_local = w.num_kv_heads // tp
    n_sets = len(page_sets(w))
    return {"workload": f"{w.name}: paged decode attention, {w.num_heads} q heads / {w.num_kv_heads} kv heads, "
                        f"head_dim {w.head_dim}, batch {w.batch}, ctx {int(w.context_lens.min())}.."
                        f"{int(w.context_lens.max())} (mean {float(w.context_lens.mean()):.0f}), block {w.block_size}, "
                        f"pool {w.num_blocks} blocks, plus store_kvcache of {w.batch} new tokens",
            "kv_heads_per_gpu": kvh_local, "q_heads_per_gpu": kvh_local * (w.num_heads // w.num_kv_heads),
            "parallelism": (f"kv heads cut {tp} ways, one shard per GPU, no collective in the path" if tp > 1 else
                            f"{world} replica(s) of the whole workload, no collective in the path"),
            "gpus": world,
            "l2": (f"{n_sets} disjoint page set(s) rotated between steps; each step streams "
                   f"{w.kv_bytes(kvh_local) / 1e6:.0f} MB per GPU > 126 MB L2"),
            "seed": w.seed}


# ----------------------------------------------------------------------------------------------
# CPU baseline (the oracle as the timed thing -- the only place bench.py times it)
# ----------------------------------------------------------------------------------------------
class CpuReference:
    """Times the torch-CPU restatement of the reference's decode path on (sequence, kv head) samples."""

    def __init__(self, w, kvh_total: int):
        import torch
        torch.set_num_threads(host_cores())  # torch.distributed.run exports OMP_NUM_THREADS=1: undo that here
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
    world = args.gpus
    name, scaling, tp = resolve(args, world)
    w = pick_workload(name, args.pool_blocks)
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
    sample = (f"restated reference jnp path (torch CPU, {ref.threads} threads) per step on the first {n_seqs} of "
              f"{w.batch} sequences x {n_kvh} of {w.num_kv_heads} kv heads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(w, world, tp, scaling),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": ref.threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm: timing helpers
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


class Dist:
    """The little of torch.distributed the bench needs; a no-op with one process."""

    def __init__(self, world, dev):
        self.world, self.dev = world, dev
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=dev)
            self.dist = dist

    def barrier(self):
        import torch
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max(self, *vals):
        import torch
        if self.world == 1:
            return [float(v) for v in vals]
        t = torch.tensor(list(vals), device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def time_blocks(fn, steps: int, min_seconds: float, dd: Dist, max_blocks: int = 4000):
    """Runs blocks of exactly `steps` calls of fn(i), each block between two CUDA events, until `min_seconds` of GPU
    time have passed (the block count is fixed beforehand from one calibration block, so every rank runs the same
    number).  Returns (per-block milliseconds of this rank, total ms between the first and the last event)."""
    import torch
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dd.barrier()
    a.record()
    for i in range(steps):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    (calib,) = dd.max(a.elapsed_time(b))
    blocks = int(min(max_blocks, max(1, np.ceil(min_seconds * 1e3 / max(calib, 1e-3)))))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    dd.barrier()
    ev[0].record()
    i = 0
    for blk in range(blocks):
        for _ in range(steps):
            fn(i)
            i += 1
        ev[blk + 1].record()
    torch.cuda.synchronize()
    per_block = [ev[j].elapsed_time(ev[j + 1]) for j in range(blocks)]
    total = ev[0].elapsed_time(ev[blocks])
    dd.barrier()
    return per_block, total


def time_pass(fn, launches: int, warm: int):
    """`warm` untimed calls, then `launches` back-to-back calls inside ONE event pair (mean per call), then the same
    number again with an event pair per call (spread; the events keep consecutive calls from overlapping their
    launches, so these run a little slower than the mean).  Returns (mean_us, [p10, p50, p90] us)."""
    import torch
    for i in range(warm):
        fn(i)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for i in range(launches):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    mean_us = a.elapsed_time(b) / launches * 1e3
    ea = [torch.cuda.Event(enable_timing=True) for _ in range(launches)]
    eb = [torch.cuda.Event(enable_timing=True) for _ in range(launches)]
    for i in range(launches):
        ea[i].record()
        fn(i)
        eb[i].record()
    torch.cuda.synchronize()
    each = [x.elapsed_time(y) * 1e3 for x, y in zip(ea, eb)]
    return mean_us, [float(v) for v in np.percentile(each, [10, 50, 90])]


class DecodeRig:
    """One rank's decode workload on the device: cache shard, rotating page sets, the three ways to run a step."""

    def __init__(self, w, kvh, dev, rank, pin=True):
        import torch
        from nanovllm_jax_b200.layers.attention import Attention
        from nanovllm_jax_b200.utils.context import create_decode_context
        self.w, self.kvh, self.dev = w, kvh, dev
        self.g = w.num_heads // w.num_kv_heads
        self.h = kvh * self.g
        self.sets = page_sets(w)
        self.n_sets = len(self.sets)
        gen = torch.Generator(device=dev)
        gen.manual_seed(w.seed * 100 + rank)
        shape = (w.num_blocks, w.block_size, kvh, w.head_dim)
        self.kc = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        self.vc = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        fill_normal_bf16(self.kc, gen)
        fill_normal_bf16(self.vc, gen)
        self.attn = Attention(self.h, w.head_dim, w.scale, kvh, w.block_size)
        self.attn.set_kv_cache(self.kc, self.vc)
        self.host, self.devflat, self.devin = make_step_inputs(w, self.sets, self.h, kvh, dev, pin=pin)
        self.ctxs = [create_decode_context(context_lens=d[4], slot_mapping=d[3], block_tables=d[5]) for d in self.devin]
        self.out = torch.empty((w.batch, self.h, w.head_dim), dtype=torch.bfloat16, device=dev)
        self.out_host = torch.empty((w.batch, self.h, w.head_dim), dtype=torch.bfloat16).pin_memory() if pin else None
        self.decode_bytes = w.kv_bytes(kvh)
        self.step_bytes = self.decode_bytes + w.batch * (kvh * w.head_dim * 2 * 2 * 2 + 4)

    def step(self, i):
        """store + decode with device-resident inputs: the fused C call behind Attention.__call__."""
        from nanovllm_jax_b200 import ops
        q, k, v, sl, cl, bt = self.devin[i % self.n_sets]
        return ops.decode_step(q, k, v, self.kc, self.vc, sl, bt, cl, self.w.scale, self.w.block_size, out=self.out)

    def decode_only(self, i):
        from nanovllm_jax_b200 import ops
        q, _, _, _, cl, bt = self.devin[i % self.n_sets]
        return ops.paged_decode(q, self.kc, self.vc, bt, cl, self.w.scale, self.w.block_size, out=self.out)

    def e2e_step(self, i):
        import torch
        s = i % self.n_sets
        self.devflat[s].copy_(self.host[s], non_blocking=True)
        o = self.attn(self.devin[s][0], self.devin[s][1], self.devin[s][2], self.ctxs[s])
        self.out_host.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def parity(self, n_seqs: int = 4):
        """Oracle check of this rank's shard: the shortest, the longest and random sequences of page set 0,
        re-computed on the host from the pages they own (bench.py's checker leg; nothing timed uses it)."""
        import torch
        from oracle import reference_attention as ref
        w = self.w
        out = self.step(0).clone()
        torch.cuda.synchronize()
        q = self.devin[0][0]
        tables0 = self.sets[0][0]
        order = np.argsort(w.context_lens)
        rng = np.random.Generator(np.random.PCG64(w.seed + 5))
        pick = [int(order[0]), int(order[-1])] + rng.choice(w.batch, max(0, n_seqs - 2), replace=False).tolist()
        mx, mean = 0.0, 0.0
        for b in pick:
            ids = [int(i) for i in tables0[b] if i >= 0]
            idx = torch.tensor(ids, device=self.dev, dtype=torch.long)
            kb = self.kc[idx].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            vb = self.vc[idx].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            want = ref.paged_decode_attention_streamed(q[b:b + 1].float().cpu().numpy(), kb, vb,
                                                       np.arange(len(ids), dtype=np.int32)[None, :],
                                                       w.context_lens[b:b + 1], w.scale, w.block_size, kv_dtype_bits=True)
            diff = np.abs(out[b:b + 1].float().cpu().numpy() - want)
            mx, mean = max(mx, float(diff.max())), max(mean, float(diff.mean()))
        return mx, mean, len(pick)


def decode_roofline(rig, peak, peak_kind, launches, warm, step_us, traffic):
    mean_us, pct = time_pass(rig.decode_only, launches, warm)
    if step_us is not None and mean_us > step_us * 1.01:  # a noisy pass: the call cannot outlast the step around it
        mean_us, pct = time_pass(rig.decode_only, launches, warm)
    achieved = rig.decode_bytes / (mean_us / 1e6) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": traffic,
            "kernel": "decode_prepare_kernel + paged_decode_kernel (one nvllm_b200_paged_decode call)",
            "bytes_per_launch": rig.decode_bytes, "us_per_launch": mean_us, "us_per_launch_p10_p50_p90": pct,
            "launches_timed": launches, "warmup_launches": warm,
            "how": "mean of back-to-back calls inside one CUDA event pair; percentiles from a second pass with an "
                   "event pair per call",
            "le_step": (None if step_us is None else bool(mean_us <= step_us * 1.01)),
            "peak_kind": f"{peak_kind} copy bandwidth", "frac_of_nominal_8tbs": achieved / 8000.0}


# ----------------------------------------------------------------------------------------------
# prefill rig (cfg4)
# ----------------------------------------------------------------------------------------------
class PrefillRig:
    def __init__(self, kvh, dev, rank):
        import torch
        from nanovllm_jax_b200 import workloads
        from nanovllm_jax_b200.layers.attention import Attention
        from nanovllm_jax_b200.utils.context import create_prefill_context
        w = workloads.config4()
        self.w, self.kvh, self.dev = w, kvh, dev
        self.g = w.num_heads // w.num_kv_heads
        self.h = kvh * self.g
        t = w.total_tokens
        gen = torch.Generator(device=dev)
        gen.manual_seed(w.seed * 100 + rank)
        self.q = torch.empty((t, self.h, w.head_dim), dtype=torch.bfloat16, device=dev)
        self.k = torch.empty((t, kvh, w.head_dim), dtype=torch.bfloat16, device=dev)
        self.v = torch.empty_like(self.k)
        for x in (self.q, self.k, self.v):
            fill_normal_bf16(x, gen)
        self.kc = torch.zeros((w.num_blocks, w.block_size, kvh, w.head_dim), dtype=torch.bfloat16, device=dev)
        self.vc = torch.zeros_like(self.kc)
        self.attn = Attention(self.h, w.head_dim, w.scale, kvh, w.block_size)
        self.attn.set_kv_cache(self.kc, self.vc)
        self.cu = torch.from_numpy(w.cu_seqlens).to(dev)
        self.slots = torch.from_numpy(w.slot_mapping).to(dev)
        self.max_len = int(w.seq_lens.max())
        self.ctx = create_prefill_context(self.cu, self.cu, self.max_len, self.max_len, self.slots,
                                          cu_seqlens_host=w.cu_seqlens)
        self.out = torch.empty_like(self.q)
        self.flat = (w.num_blocks * w.block_size, kvh, w.head_dim)
        self.flops = w.flops(self.h)
        self.store_bytes = w.store_bytes(kvh)

    def step(self, i=0):
        return self.attn(self.q, self.k, self.v, self.ctx)

    def prefill_only(self, i=0):
        from nanovllm_jax_b200 import ops
        return ops.varlen_prefill(self.q, self.k, self.v, self.cu, self.max_len, self.w.scale, out=self.out,
                                  cu_seqlens_host=self.w.cu_seqlens)

    def store_only(self, i=0):
        from nanovllm_jax_b200 import ops
        ops.store_kvcache(self.k, self.v, self.kc.view(self.flat), self.vc.view(self.flat), self.slots)

    # ---- the step before attention in a Qwen3 layer: q-norm, k-norm, rotary embedding, store (one pass) ----
    def setup_pre_attention(self):
        import torch
        w, dev = self.w, self.dev
        inv = 1.0 / (1e6 ** (torch.arange(0, w.head_dim, 2, device=dev, dtype=torch.float32) / w.head_dim))
        ang = torch.arange(int(w.seq_lens.max()), device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos_sin = torch.cat([ang.cos(), ang.sin()], dim=-1).contiguous()
        pos = np.concatenate([np.arange(n, dtype=np.int32) for n in w.seq_lens])
        self.positions = torch.from_numpy(pos).to(dev)
        self.q_w = torch.ones(w.head_dim, dtype=torch.float32, device=dev)
        self.k_w = torch.ones(w.head_dim, dtype=torch.float32, device=dev)
        self.q2, self.k2 = self.q.clone(), self.k.clone()  # rotated in place: the prefill's inputs stay as they are
        t = w.total_tokens
        self.pre_bytes = t * ((self.h + 2 * self.kvh) + (self.h + self.kvh) + 2 * self.kvh) * w.head_dim * 2

    def pre_attention_only(self, i=0):
        from nanovllm_jax_b200 import ops
        ops.qk_norm_rope_store(self.q2, self.k2, self.v, self.q_w, self.k_w, self.cos_sin, self.positions,
                               self.kc.view(self.flat), self.vc.view(self.flat), self.slots)

    # ---- prefill over a cached prefix: the first half of every sequence is cached, the second half is new ----
    def setup_prefix(self):
        import torch
        w, dev = self.w, self.dev
        lens = w.seq_lens.astype(np.int64)
        prefix = lens // 2
        new = lens - prefix
        self.store_only()  # every token's K/V row sits in the pages
        width = max(len(b) for b in w.block_lists)
        tables = np.full((w.batch, width), -1, np.int32)
        for b, blocks in enumerate(w.block_lists):
            tables[b, : len(blocks)] = blocks
        self.tables = torch.from_numpy(tables).to(dev)
        self.cu_q_host = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
        self.cu_q = torch.from_numpy(self.cu_q_host).to(dev)
        self.cu_k = torch.from_numpy(w.cu_seqlens).to(dev)
        self.max_new = int(new.max())
        rows = np.concatenate([np.arange(w.cu_seqlens[b] + prefix[b], w.cu_seqlens[b + 1]) for b in range(w.batch)])
        self.q_new = self.q[torch.from_numpy(rows).to(dev)].contiguous()
        self.out_new = torch.empty_like(self.q_new)
        self.prefix_flops = int(4 * w.head_dim * self.h * int((new * prefix + new * (new + 1) // 2).sum()))
        self.prefix_desc = (f"{w.batch} sequences, {int(prefix.sum())} cached + {int(new.sum())} new tokens "
                            f"(the second half of each sequence of the prefill workload)")

    def prefix_prefill_only(self, i=0):
        from nanovllm_jax_b200 import ops
        return ops.paged_prefill(self.q_new, self.kc, self.vc, self.tables, self.cu_q, self.cu_k, self.max_new,
                                 self.w.scale, self.w.block_size, out=self.out_new, cu_seqlens_host=self.cu_q_host)


def prefill_roofline(rig, launches, warm):
    _, sustained, burst, kind = load_peaks()
    mean_us, pct = time_pass(rig.prefill_only, launches, warm)
    achieved = rig.flops / (mean_us / 1e6) / 1e12
    return {"bound": "tensor", "achieved": achieved, "peak": sustained, "unit": "TFLOP/s", "frac": achieved / sustained,
            "frac_of_burst": achieved / burst, "peak_burst": burst, "traffic": NCU_TRAFFIC_BYTES.get("cfg4"),
            "kernel": "prefill_plan_kernel + varlen_prefill_kernel (one nvllm_b200_varlen_prefill call)",
            "flops_per_launch": rig.flops, "us_per_launch": mean_us, "us_per_launch_p10_p50_p90": pct,
            "launches_timed": launches, "warmup_launches": warm,
            "peak_kind": f"{kind} cuBLAS bf16, sustained (burst beside it)"}


def prefill_config(w, world, h, kvh):
    return {"workload": f"{w.name}: varlen causal prefill attention, {w.num_heads} q heads / {w.num_kv_heads} kv heads, "
                        f"head_dim {w.head_dim}, {w.batch} packed sequences of {int(w.seq_lens.min())}.."
                        f"{int(w.seq_lens.max())} tokens (T = {w.total_tokens}), plus store_kvcache of all T tokens "
                        f"(block {w.block_size})",
            "kv_heads_per_gpu": kvh, "q_heads_per_gpu": h,
            "parallelism": f"kv-head shards x{world}, no collective in the path", "gpus": world,
            "l2": f"q/k/v/out of one step are {(2 * h + 2 * kvh) * w.total_tokens * w.head_dim * 2 / 1e6:.0f} MB "
                  f"> 126 MB L2; K/V tile reuse inside a step is meant to hit L2",
            "seed": w.seed}


def secondary_block(dev, rank, launches, warm):
    """The workloads the headline does not run, each in its own pass (one GPU): sizes, event-timed means, fractions."""
    import gc

    import torch
    peak, sustained, burst, kind = load_peaks()
    out = {}
    w3 = pick_workload("cfg3")
    rig = DecodeRig(w3, w3.num_kv_heads, dev, rank, pin=False)
    step_us, _ = time_pass(rig.step, launches, warm)
    roof = decode_roofline(rig, peak, kind, launches, warm, step_us, None)
    out["cfg3_decode"] = {"workload": w3.name, "kv_heads": w3.num_kv_heads, "step_us": step_us,
                          "step_gbps": rig.step_bytes / (step_us / 1e6) / 1e9, "roofline": roof}
    del rig
    gc.collect()
    torch.cuda.empty_cache()
    pr = PrefillRig(8, dev, rank)
    # the kernel-only pass first: the step (store + prefill) is then timed on a GPU that is at least as warm
    proof = prefill_roofline(pr, max(10, launches // 2), max(3, warm // 2))
    step_us, _ = time_pass(pr.step, max(10, launches // 2), max(3, warm // 2))
    out["prefill"] = {"workload": pr.w.name, "step_us": step_us, "step_tflops": pr.flops / (step_us / 1e6) / 1e12,
                      "roofline": proof}
    st_us, st_pct = time_pass(pr.store_only, launches, warm)
    gbps = pr.store_bytes / (st_us / 1e6) / 1e9
    out["store_kvcache"] = {"workload": f"{pr.w.total_tokens} tokens x 8 kv heads (the prefill's K/V rows)",
                            "bytes_per_launch": pr.store_bytes, "us_per_launch": st_us,
                            "us_per_launch_p10_p50_p90": st_pct, "launches_timed": launches,
                            "roofline": {"bound": "hbm", "achieved": gbps, "peak": peak, "unit": "GB/s",
                                         "frac": gbps / peak, "traffic": None,
                                         "note": "325 MB read + 325 MB written per launch; with back-to-back launches "
                                                 "part of the source rows is still in the 126 MB L2"}}
    pr.setup_pre_attention()
    pa_us, pa_pct = time_pass(pr.pre_attention_only, launches, warm)
    gbps = pr.pre_bytes / (pa_us / 1e6) / 1e9
    out["pre_attention"] = {"workload": f"q-norm + k-norm + rotary embedding + store of {pr.w.total_tokens} tokens, "
                                        f"{pr.h} q heads / {pr.kvh} kv heads (one nvllm_b200_qk_norm_rope_store call)",
                            "bytes_per_launch": pr.pre_bytes, "us_per_launch": pa_us,
                            "us_per_launch_p10_p50_p90": pa_pct, "launches_timed": launches,
                            "roofline": {"bound": "hbm", "achieved": gbps, "peak": peak, "unit": "GB/s",
                                         "frac": gbps / peak, "traffic": None,
                                         "note": "q, k, v read; q, k written back; rotated k and v scattered into the pages"}}
    pr.setup_prefix()
    n_l, n_w = max(10, launches // 2), max(3, warm // 2)
    px_us, px_pct = time_pass(pr.prefix_prefill_only, n_l, n_w)
    tfl = pr.prefix_flops / (px_us / 1e6) / 1e12
    out["prefix_prefill"] = {"workload": pr.prefix_desc + ", keys and values read from the pages through block tables "
                                         "(one nvllm_b200_paged_prefill call)",
                             "flops_per_launch": pr.prefix_flops, "us_per_launch": px_us,
                             "us_per_launch_p10_p50_p90": px_pct, "launches_timed": n_l,
                             "roofline": {"bound": "tensor", "achieved": tfl, "peak": sustained, "unit": "TFLOP/s",
                                          "frac": tfl / sustained, "frac_of_burst": tfl / burst, "peak_burst": burst,
                                          "traffic": None}}
    del pr
    gc.collect()
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def run_b200(args):
    import torch
    from nanovllm_jax_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dd = Dist(world, dev)
    _lib.load()  # fail loudly before anything is timed

    name, scaling, tp = resolve(args, world)
    w = pick_workload(name, args.pool_blocks)
    if w.num_kv_heads % tp:
        raise SystemExit("the kv heads must divide by the number of shards")
    kvh = w.num_kv_heads // tp
    shard_rank = rank if (scaling == "strong" and not args.shard_of) else 0
    rig = DecodeRig(w, kvh, dev, shard_rank if tp > 1 else rank)

    for i in range(max(args.warmup, 3)):
        rig.step(i)
    dd.barrier()
    if args.profile_steps:  # a short untimed run for a profiler to attach to: nothing is measured or printed
        for i in range(args.profile_steps):
            rig.step(i)
        torch.cuda.synchronize()
        dd.close()
        return

    # --- timed region: blocks of K steps, device-resident inputs --------------------------------
    with ClockSampler(local) as clocks:
        per_block, total_ms = time_blocks(rig.step, args.steps, args.min_seconds, dd)
    blocks = len(per_block)
    ms_local = total_ms / (blocks * args.steps)
    med_local = float(np.median(per_block)) / args.steps
    first_local = per_block[0] / args.steps
    ms_per_step, ms_median, ms_first = dd.max(ms_local, med_local, first_local)
    status = _lib.device_status()

    # --- the decode C call alone, in its own pass ------------------------------------------------
    peak, _, _, peak_kind = load_peaks()
    roof = decode_roofline(rig, peak, peak_kind, args.pass_launches, args.pass_warmup, ms_local * 1e3,
                           NCU_TRAFFIC_BYTES.get(name) if kvh == w.num_kv_heads else None)
    (roof_us,) = dd.max(roof["us_per_launch"])
    if world > 1:  # the line reports the slowest rank
        roof["us_per_launch_rank0"] = roof["us_per_launch"]
        roof["us_per_launch"] = roof_us
        roof["achieved"] = rig.decode_bytes / (roof_us / 1e6) / 1e9
        roof["frac"] = roof["achieved"] / peak
        roof["frac_of_nominal_8tbs"] = roof["achieved"] / 8000.0
        roof["le_step"] = bool(roof_us <= ms_per_step * 1e3 * 1.01)

    # --- end to end: host inputs in, host result out, every step --------------------------------
    e2e_steps = max(args.steps, min(2000, int(0.5 / max(ms_local * 1.5e-3, 1e-6))))
    for i in range(5):
        rig.e2e_step(i)
    dd.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        rig.e2e_step(i)
    torch.cuda.synchronize()
    (e2e_ms,) = dd.max((time.perf_counter() - t0) / e2e_steps * 1e3)
    dd.barrier()

    # --- parity of what was timed (checker leg) --------------------------------------------------
    parity = None
    if world > 1 or args.parity:
        mx, mean, n = rig.parity(4)
        mx, mean = dd.max(mx, mean)
        parity = {"parity_max_abs": mx, "parity_mean_abs": mean, "sequences_per_rank": n, "tolerance": [2e-2, 2e-3],
                  "ok": bool(mx <= 2e-2 and mean <= 2e-3),
                  "what": "every rank re-computes sequences of its kv-head shard with the fp32 CPU oracle from the "
                          "pages they own; max over ranks"}

    secondary = None
    if world == 1 and not args.no_secondary and not args.shard_of and name == "cfg2":
        secondary = secondary_block(dev, rank, args.pass_launches, args.pass_warmup)

    if rank == 0:
        h2d = rig.devin[0][0].numel() * 2 + 2 * rig.devin[0][1].numel() * 2 + 4 * (2 * w.batch + rig.devin[0][5].numel())
        line = {
            "metric": METRIC, "value": world * rig.step_bytes / (ms_per_step / 1e3) / 1e9, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(w, world, tp, scaling),
            "timing": {"blocks": blocks, "steps_per_block": args.steps, "timed_ms": total_ms,
                       "ms_per_step_median_block": ms_median, "ms_per_step_first_block": ms_first,
                       "min_seconds": args.min_seconds,
                       "what": "the block of `steps` steps is repeated back to back until min_seconds of GPU time "
                               "have passed; ms_per_step = total / (blocks * steps), max over ranks"},
            "per_gpu_gbps": rig.step_bytes / (ms_per_step / 1e3) / 1e9,
            "per_gpu_frac_of_peak": rig.step_bytes / (ms_per_step / 1e3) / 1e9 / peak,
            "roofline": roof,
            "e2e": {"value": world * rig.step_bytes / (e2e_ms / 1e3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": rig.out_host.numel() * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "what": "Attention.__call__ (one nvllm_b200_decode_step call) with q/k/v/slot_mapping/context_lens/"
                            "block_tables copied from pinned host memory (one packed copy) and the output copied "
                            "back, stream-synchronised every step; the KV cache stays in HBM"},
            "clocks": clocks.summary(), "gpu_launches": 2 * args.steps * blocks, "launches_per_step": 2,
            "device_status": status,
        }
        if args.shard_of:
            line["config"]["shard_of"] = args.shard_of
        if parity:
            line["parity"] = parity
        if secondary:
            line["secondary"] = secondary
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg(w, kvh)
        print(json.dumps(line), flush=True)
    dd.close()


# ----------------------------------------------------------------------------------------------
# prefill workload (cfg4) as the headline: metric = causal attention TFLOP/s, tensor-core roofline
# ----------------------------------------------------------------------------------------------
def prefill_cpu_sample(w, budget_s: float):
    """Times the torch-CPU restatement of the reference prefill on the shortest sequences that fit the budget."""
    import torch
    from oracle import reference_attention_torch as reft
    torch.set_num_threads(host_cores())
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


def run_prefill(args):
    import torch
    from nanovllm_jax_b200 import _lib, workloads

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    w = workloads.config4()
    scaling = "weak" if args.scaling == "auto" else args.scaling
    if args.impl == "reference":
        if rank != 0:
            return
        budget = min(20.0, 150.0 / max(args.steps + args.warmup, 1))
        vals = [prefill_cpu_sample(w, budget) for _ in range(min(args.steps + args.warmup, 3))]
        tf, used, dt, threads = vals[-1]
        sample = f"restated reference prefill (torch CPU, fp32) on the {len(used)} shortest sequences ({used} tokens)"
        print(json.dumps({"impl": "reference", "metric": PREFILL_METRIC, "value": tf, "unit": PREFILL_UNIT,
                          "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
                          "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16",
                          "data": "synthetic", "config": prefill_config(w, args.gpus, w.num_heads, w.num_kv_heads),
                          "cpu_baseline": {"value": tf, "unit": PREFILL_UNIT, "cores": threads, "kind": "port",
                                           "sample": sample},
                          "e2e": {"value": tf, "unit": PREFILL_UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                          "gpu_launches": 0}), flush=True)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dd = Dist(world, dev)
    _lib.load()
    kvh = w.num_kv_heads // world if scaling == "strong" else w.num_kv_heads
    rig = PrefillRig(kvh, dev, rank)
    for _ in range(max(args.warmup, 3)):
        rig.step()
    if args.profile_steps:  # a short untimed run for a profiler to attach to: nothing is measured or printed
        for _ in range(args.profile_steps):
            rig.step()
        rig.setup_pre_attention()
        rig.setup_prefix()
        for _ in range(args.profile_steps):  # the two kernels of the secondary block that share this workload
            rig.pre_attention_only()
            rig.prefix_prefill_only()
        torch.cuda.synchronize()
        dd.close()
        return
    with ClockSampler(local) as clocks:
        per_block, total_ms = time_blocks(rig.step, args.steps, args.min_seconds, dd)
    blocks = len(per_block)
    (ms,) = dd.max(total_ms / (blocks * args.steps))
    status = _lib.device_status()
    roof = prefill_roofline(rig, max(10, args.pass_launches // 2), max(3, args.pass_warmup // 2))

    hq, hk, hv = (x.cpu().pin_memory() for x in (rig.q, rig.k, rig.v))
    hout = torch.empty_like(hq).pin_memory()
    e2e_steps = max(1, min(args.steps, 10))

    def e2e_step():
        rig.q.copy_(hq, non_blocking=True)
        rig.k.copy_(hk, non_blocking=True)
        rig.v.copy_(hv, non_blocking=True)
        o = rig.step()
        hout.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step()
    dd.barrier()
    tw = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    (e2e_ms,) = dd.max((time.perf_counter() - tw) / e2e_steps * 1e3)
    dd.barrier()
    if rank == 0:
        line = {"metric": PREFILL_METRIC, "value": world * rig.flops / (ms / 1e3) / 1e12, "unit": PREFILL_UNIT,
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": prefill_config(w, world, rig.h, kvh),
                "timing": {"blocks": blocks, "steps_per_block": args.steps, "timed_ms": total_ms},
                "roofline": roof,
                "e2e": {"value": world * rig.flops / (e2e_ms / 1e3) / 1e12, "unit": PREFILL_UNIT,
                        "h2d_bytes_per_step": sum(x.numel() * 2 for x in (hq, hk, hv)),
                        "d2h_bytes_per_step": hout.numel() * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                        "what": "Attention.__call__ (store_kvcache + varlen prefill) with q/k/v copied from pinned host "
                                "memory and the output copied back every step"},
                "clocks": clocks.summary(), "gpu_launches": 3 * args.steps * blocks, "device_status": status}
        if world == 1 and not args.no_cpu_baseline:
            tf, used, dt, threads = prefill_cpu_sample(w, 12.0)
            line["cpu_baseline"] = {"value": tf, "unit": PREFILL_UNIT, "cores": threads, "kind": "port",
                                    "sample": f"restated reference prefill (torch CPU, fp32) on the {len(used)} shortest "
                                              f"sequences ({used} tokens), {dt:.1f} s; JAX itself is not installed"}
        print(json.dumps(line), flush=True)
    dd.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", choices=["auto", "cfg1", "cfg2", "cfg3", "cfg4"], default="auto")
    ap.add_argument("--scaling", choices=["auto", "weak", "strong"], default="auto")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="one GPU only: run rank 0's shard of a kv-head split this many ways")
    ap.add_argument("--min-seconds", type=float, default=2.0, help="GPU time the repeated K-step block must cover")
    ap.add_argument("--pass-launches", type=int, default=100, help="back-to-back launches of the kernel-only passes")
    ap.add_argument("--pass-warmup", type=int, default=10)
    ap.add_argument("--parity", action="store_true", help="run the oracle check of the timed workload at one GPU too")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--profile-steps", type=int, default=0,
                    help="run this many untimed steps after the warm-up and exit (for profiler captures)")
    ap.add_argument("--pool-blocks", type=int, default=0,
                    help="shrink the physical page pool (same sequences); for profiler captures only")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    args.pass_launches = max(args.pass_launches, 50)
    args.pass_warmup = max(args.pass_warmup, 10)
    if args.shard_of and args.gpus != 1:
        raise SystemExit("--shard-of emulates one shard on ONE GPU")
    if args.impl == "reference":
        return run_prefill(args) if args.workload == "cfg4" else run_reference(args)
    if args.gpus > 1 and "RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__)] + sys.argv[1:]
        os.execv(sys.executable, cmd)
    if args.workload == "cfg4":
        return run_prefill(args)
    run_b200(args)


if __name__ == "__main__":
    main()
