#!/usr/bin/env python
"""End-to-end decode throughput (tokens/s) of a random-init Qwen3-8B-shaped model whose attention runs on this
library, at 1/2/4/8 GPUs with tensor parallelism.

    python bench_serving.py [--gpus N] [--requests 128] [--prompt-len 512] [--gen-len 256] [--layers 36]
                            [--no-graph] [--allreduce peer|nccl] [--unfused]
    (N > 1: python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench_serving.py --gpus N)

What is measured is the serving loop of the reference (engine/llm_engine.py:120-165): prefill first, in batches of at
most 16 384 prompt tokens, then one decode step per generated token for all requests, greedy sampling, token ids
read back to the host every step.  Everything AROUND attention is deliberately plain: torch bf16 GEMMs (cuBLAS),
torch RMSNorm / SiLU, replicated embedding and LM head.  What comes from this library:

  * attention -- ``Attention.__call__`` with per-rank head counts and a per-rank KV-cache shard, exactly as the
    reference's model calls it (models/qwen3.py:114-120, 166); by default the step between the QKV projection and
    attention (q_norm, k_norm, rotary_emb, store_kv_to_cache: models/qwen3.py:157-166) runs as this library's fused
    kernels (``--unfused`` puts the torch ops back);
  * the decode step's metadata -- fixed-shape buffers (``DecodeMetadata``), one host -> device copy per step;
  * the sum over ranks after o_proj and down_proj (layers/linear.py:486-510) -- ``PeerAllReduce`` (one-shot NVLink
    kernel, residual add fused) unless ``--allreduce nccl``.

Pages are dealt the way the reference's block manager deals them (engine/block_manager.py:137-182, 215-244: free list
in order, a new block when a sequence crosses a block boundary); ``tests/test_serving_tables.py`` holds this to
tables produced by the reference's own code.

The decode step is replayed from a CUDA graph.  With more than one rank that holds only when the reductions are this
library's kernels (``--allreduce peer``: ordinary kernels that number their calls on the device, so a replay is a new
call; their waits are bounded, so a rank that falls out of step ends in a status bit, not a hang); with
``--allreduce nccl`` the step is launched eagerly -- NCCL collectives of several ranks are not captured.  The model is NOT part of the library; it exists so that
the attention path can be timed inside a realistic decode step.  Weights are N(0, 0.02) random (there is no checkpoint
in the image), drawn per head group so that the full model is the same at every tensor-parallel size; prompts are
uniform random token ids.  Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from nanovllm_jax_b200 import ops  # noqa: E402
from nanovllm_jax_b200.layers.attention import Attention  # noqa: E402
from nanovllm_jax_b200.utils.context import create_prefill_context  # noqa: E402
from nanovllm_jax_b200.utils.decode_metadata import DecodeMetadata  # noqa: E402

SHARDS = 8  # weights are drawn in 8 head groups / column chunks: the largest tensor-parallel size (config.py:39)


class Qwen3Config:
    """Qwen3-8B sizes (dense, GQA, QK-norm, RoPE, SwiGLU)."""

    def __init__(self, layers=36, hidden=4096, heads=32, kv_heads=8, head_dim=128, intermediate=12288, vocab=151936,
                 rope_theta=1e6, eps=1e-6, block_size=256, max_position=4096):
        self.layers, self.hidden, self.heads, self.kv_heads, self.head_dim = layers, hidden, heads, kv_heads, head_dim
        self.intermediate, self.vocab, self.rope_theta, self.eps, self.block_size = (intermediate, vocab, rope_theta, eps,
                                                                                     block_size)
        self.max_position = max_position


def _rand(shape, gen, dev, std=0.02):
    return (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std).to(torch.bfloat16)


def _sharded(rows_per_shard, cols, seed, my_shards, dev, transpose=False):
    """Concatenation of this rank's shards of a matrix drawn shard by shard (shard s from seed + s), so that the matrix
    assembled from all ranks is the same whatever the tensor-parallel size.  transpose: shards are column blocks."""
    parts = []
    for s in my_shards:
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed * 64 + s)
        parts.append(_rand((rows_per_shard, cols), gen, dev))
    w = torch.cat(parts, dim=0)
    return w.t().contiguous() if transpose else w


class Layer:
    def __init__(self, cfg, tp, rank, index, dev):
        h, d = cfg.hidden, cfg.head_dim
        self.hq, self.hk = cfg.heads // tp, cfg.kv_heads // tp
        shards = min(SHARDS, cfg.kv_heads)   # models with fewer than 8 kv heads are drawn in as many groups
        if shards % tp or cfg.kv_heads % shards or cfg.intermediate % shards:
            raise ValueError("tensor-parallel size must divide the number of weight shards")
        mine = list(range(rank * shards // tp, (rank + 1) * shards // tp))
        g = cfg.heads // cfg.kv_heads
        kv_per_shard = cfg.kv_heads // shards
        seed = 1000 + index * 16
        wq = _sharded(kv_per_shard * g * d, h, seed + 0, mine, dev)
        wk = _sharded(kv_per_shard * d, h, seed + 1, mine, dev)
        wv = _sharded(kv_per_shard * d, h, seed + 2, mine, dev)
        self.w_qkv = torch.cat([wq, wk, wv], dim=0)                                   # column-parallel
        self.w_o = _sharded(kv_per_shard * g * d, h, seed + 3, mine, dev, transpose=True)   # row-parallel [h, hq*d]
        inter = cfg.intermediate // shards
        self.w_gate_up = torch.cat([_sharded(inter, h, seed + 4, mine, dev), _sharded(inter, h, seed + 5, mine, dev)], 0)
        self.w_down = _sharded(inter, h, seed + 6, mine, dev, transpose=True)          # row-parallel [h, inter/tp]
        self.ln1 = torch.ones(h, dtype=torch.bfloat16, device=dev)
        self.ln2 = torch.ones(h, dtype=torch.bfloat16, device=dev)
        self.q_norm = torch.ones(d, dtype=torch.bfloat16, device=dev)
        self.k_norm = torch.ones(d, dtype=torch.bfloat16, device=dev)
        self.q_norm_f32, self.k_norm_f32 = self.q_norm.float(), self.k_norm.float()
        self.attn = Attention(self.hq, d, 1.0 / math.sqrt(d), self.hk, cfg.block_size)


class Qwen3:
    """Forward pass only.  `fused`: the library's fused pre-attention kernels; `reducer`: a PeerAllReduce or None (NCCL)."""

    def __init__(self, cfg: Qwen3Config, tp: int, rank: int, dev, seed: int = 0, fused: bool = True, reducer=None):
        self.cfg, self.tp, self.rank, self.dev, self.fused, self.reducer = cfg, tp, rank, dev, fused, reducer
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)                          # embedding / head replicated: same draw on every rank
        self.embed = _rand((cfg.vocab, cfg.hidden), gen, dev)
        self.lm_head = _rand((cfg.vocab, cfg.hidden), gen, dev)
        self.final_ln = torch.ones(cfg.hidden, dtype=torch.bfloat16, device=dev)
        self.layers = [Layer(cfg, tp, rank, i, dev) for i in range(cfg.layers)]
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=dev, dtype=torch.float32) / cfg.head_dim))
        self.inv_freq = inv
        ang = torch.arange(cfg.max_position, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos_sin = torch.cat([ang.cos(), ang.sin()], dim=-1).contiguous()   # layers/rotary_embedding.py:57-75
        self.allreduce_calls = 0

    def allocate_cache(self, num_blocks: int):
        cfg = self.cfg
        for layer in self.layers:
            shape = (num_blocks, cfg.block_size, layer.hk, cfg.head_dim)
            layer.attn.set_kv_cache(torch.zeros(shape, dtype=torch.bfloat16, device=self.dev),
                                    torch.zeros(shape, dtype=torch.bfloat16, device=self.dev))

    def _rope(self, x, positions):
        ang = positions.to(torch.float32)[:, None] * self.inv_freq[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x1, x2 = x.float().chunk(2, dim=-1)
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(torch.bfloat16)

    def _reduce_add(self, partial, residual):
        """residual + sum over ranks of partial (the row-parallel reduction followed by the residual add)."""
        if self.tp == 1:
            return residual + partial
        self.allreduce_calls += 1
        if self.reducer is not None:
            return self.reducer.all_reduce_(partial, residual=residual)
        dist.all_reduce(partial)
        return residual + partial

    def _attention(self, layer, q, k, v, positions, ctx, dense_attention):
        d = self.cfg.head_dim
        q, k, v = q.view(-1, layer.hq, d), k.view(-1, layer.hk, d), v.reshape(-1, layer.hk, d)
        if dense_attention is not None or not self.fused:
            q = F.rms_norm(q, (d,), layer.q_norm, self.cfg.eps)
            k = F.rms_norm(k, (d,), layer.k_norm, self.cfg.eps)
            q, k = self._rope(q, positions), self._rope(k, positions)
            if dense_attention is not None:
                return dense_attention(layer, q, k, v)
            return layer.attn(q.contiguous(), k.contiguous(), v.contiguous(), ctx)
        a = layer.attn
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        pos32 = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
        if not ctx.is_prefill:  # norm + rope + store + decode attention: one C call, two launches
            return ops.fused_decode_step(q, k, v, layer.q_norm_f32, layer.k_norm_f32, self.cos_sin, pos32, a.k_cache,
                                         a.v_cache, ctx.slot_mapping, ctx.block_tables, ctx.context_lens, a.scale,
                                         a.block_size, eps=self.cfg.eps)
        ops.qk_norm_rope_store(q, k, v, layer.q_norm_f32, layer.k_norm_f32, self.cos_sin, pos32, a.k_cache, a.v_cache,
                               ctx.slot_mapping, eps=self.cfg.eps)
        return a._prefill_attention(q, k, v, ctx)  # the rows are stored already

    def forward(self, ids, positions, ctx, dense_attention=None):
        """ids, positions: [T] on device.  Returns hidden states [T, hidden]."""
        cfg = self.cfg
        d = cfg.head_dim
        x = self.embed[ids]
        for layer in self.layers:
            h = F.rms_norm(x, (cfg.hidden,), layer.ln1, cfg.eps)
            qkv = h @ layer.w_qkv.t()
            q, k, v = qkv.split([layer.hq * d, layer.hk * d, layer.hk * d], dim=-1)
            o = self._attention(layer, q, k, v, positions, ctx, dense_attention)
            x = self._reduce_add(o.reshape(-1, layer.hq * d) @ layer.w_o.t(), x)
            h = F.rms_norm(x, (cfg.hidden,), layer.ln2, cfg.eps)
            gate, up = (h @ layer.w_gate_up.t()).chunk(2, dim=-1)
            x = self._reduce_add((F.silu(gate) * up) @ layer.w_down.t(), x)
        return F.rms_norm(x, (cfg.hidden,), self.final_ln, cfg.eps)

    def logits(self, hidden):
        return hidden @ self.lm_head.t()


def deal_pages(requests: int, prompt_len: int, gen_len: int, block: int):
    """Block tables [requests, blocks] as the reference's block manager deals them for this workload: ``allocate`` takes
    the free list in order, request by request (engine/block_manager.py:137-182); during decode a sequence takes the
    next free block when its length crosses a block boundary, in request order within a step (:215-232).  No prompt
    shares a full block with another (random tokens), so the prefix cache never hits."""
    per_prompt = -(-prompt_len // block)
    total = -(-(prompt_len + gen_len - 1) // block)
    tables = np.full((requests, total), -1, dtype=np.int32)
    nxt = 0
    for r in range(requests):
        tables[r, :per_prompt] = np.arange(nxt, nxt + per_prompt)
        nxt += per_prompt
    for j in range(per_prompt, total):       # the j-th block of every sequence is taken in the same decode step
        tables[:, j] = np.arange(nxt, nxt + requests)
        nxt += requests
    return tables, nxt


class Engine:
    """Static-batch serving loop: every request prefills, then all decode together (what the reference's scheduler does
    with max_num_seqs >= requests: prefill first, engine/scheduler.py:81-100, then decode, :103-125)."""

    def __init__(self, model: Qwen3, prompts: np.ndarray, gen_len: int, max_batched_tokens: int = 16384):
        self.m, self.prompts, self.gen_len = model, prompts, gen_len
        self.n, self.plen = prompts.shape
        cfg = model.cfg
        self.blk = cfg.block_size
        self.tables, used = deal_pages(self.n, self.plen, gen_len, self.blk)
        self.max_blocks = self.tables.shape[1]
        model.allocate_cache(used + 8)
        self.per_prefill = max(1, max_batched_tokens // self.plen)
        dev = model.dev
        self.meta = DecodeMetadata(self.n, self.max_blocks, dev)   # fixed-shape decode metadata, one copy per step
        self.h_tokens = torch.zeros(self.n, dtype=torch.int32).pin_memory()
        self.graph = None
        self.graph_error = None

    # ---- prefill ----
    def prefill(self):
        dev = self.m.dev
        first = torch.empty(self.n, dtype=torch.int32, device=dev)
        self.fingerprint = torch.zeros(2, dtype=torch.float64, device=dev)  # sum |hidden|, sum of the top logits
        for s0 in range(0, self.n, self.per_prefill):
            s1 = min(self.n, s0 + self.per_prefill)
            b = s1 - s0
            ids = torch.from_numpy(self.prompts[s0:s1].reshape(-1).astype(np.int64)).to(dev)
            pos = torch.arange(self.plen, device=dev, dtype=torch.int32).repeat(b)
            cu_host = (np.arange(b + 1) * self.plen).astype(np.int32)
            slots = (self.tables[s0:s1, :, None] * self.blk + np.arange(self.blk)[None, None, :]).reshape(b, -1)[:, : self.plen]
            ctx = create_prefill_context(torch.from_numpy(cu_host).to(dev), torch.from_numpy(cu_host).to(dev), self.plen,
                                         self.plen, torch.from_numpy(slots.reshape(-1).astype(np.int32)).to(dev),
                                         cu_seqlens_host=cu_host)
            hidden = self.m.forward(ids, pos, ctx)
            last = hidden[torch.from_numpy(cu_host[1:].astype(np.int64) - 1).to(dev)]
            logits = self.m.logits(last)
            first[s0:s1] = logits.argmax(dim=-1).to(torch.int32)
            self.fingerprint[0] += last.float().abs().sum().double()
            self.fingerprint[1] += logits.float().amax(dim=-1).sum().double()
        return first

    # ---- decode ----
    def _decode_step_device(self):
        ids, pos = self.meta.inputs(self.n)
        hidden = self.m.forward(ids, pos, self.meta.context(self.n))
        ids.copy_(self.m.logits(hidden).argmax(dim=-1).to(torch.int32))

    def _set_meta(self, step, tokens=None):
        """Metadata of decode step `step` (1-based): the token fed sits at position plen + step - 1."""
        length = self.plen + step
        pos = length - 1
        j = pos // self.blk
        slots = self.tables[:, j] * self.blk + pos % self.blk
        tables = self.tables[:, : j + 1]
        ids = tokens if tokens is not None else np.zeros(self.n, np.int32)
        self.meta.update(ids, np.full(self.n, pos, np.int32), slots, np.full(self.n, length, np.int32), tables,
                         max_num_seqs=self.n)

    def decode(self, first_tokens, use_graph: bool):
        n = self.n
        first_host = first_tokens.cpu().numpy().astype(np.int32)
        out = np.zeros((n, self.gen_len), dtype=np.int64)
        out[:, 0] = first_host
        if use_graph and self.graph is None:
            self._set_meta(1, first_host)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._decode_step_device()      # warm-up on the side stream (allocations, cuBLAS handles)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            try:
                g = torch.cuda.CUDAGraph()
                # thread_local: another thread of the process (NCCL's watchdog) may touch CUDA during the capture
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    self._decode_step_device()
                self.graph = g
            except Exception as exc:  # capture unsupported here: run the step eagerly and say so
                self.graph = None
                self.graph_error = f"{type(exc).__name__}: {exc}"[:200]
                torch.cuda.synchronize()
        tokens = first_host
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for step in range(1, self.gen_len):
            # the ids fed at this step are already on the device (the previous step's argmax) except at step 1
            self._set_meta(step, tokens)
            if self.graph is not None:
                self.graph.replay()
            else:
                self._decode_step_device()
            self.h_tokens.copy_(self.meta.input_ids[:n], non_blocking=True)
            torch.cuda.current_stream().synchronize()   # the scheduler needs the tokens (EOS / max_tokens checks)
            tokens = self.h_tokens.numpy().copy()
            out[:, step] = tokens
        return out, time.perf_counter() - t0


def _stage(msg: str) -> None:
    """Progress marker on stderr (NVLLM_SERVING_VERBOSE=1): shows how far each rank got if a run stalls."""
    if os.environ.get("NVLLM_SERVING_VERBOSE", "0") == "1":
        print(f"[rank {os.environ.get('RANK', '0')} +{time.perf_counter() - _T0:7.1f}s] {msg}", file=sys.stderr, flush=True)


_T0 = time.perf_counter()


def time_allreduce(model: Qwen3, tokens: int, calls: int = 144):
    """Device time of one decode-size reduction (+ residual add) as the model issues it, event-timed over `calls`
    back-to-back calls: (microseconds per call, which implementation)."""
    x = torch.zeros((tokens, model.cfg.hidden), dtype=torch.bfloat16, device=model.dev)
    res = torch.zeros_like(x)
    for _ in range(8):
        model._reduce_add(x, res)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for _ in range(calls):
        model._reduce_add(x, res)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / calls * 1e3], device=model.dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--gen-len", type=int, default=256)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--no-graph", action="store_true", help="launch the decode step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--allreduce", choices=["peer", "nccl"], default="peer")
    ap.add_argument("--unfused", action="store_true", help="torch q_norm / k_norm / RoPE and separate store instead of the fused kernels")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if SHARDS % world:
        raise SystemExit("the tensor-parallel size must divide 8")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    _stage("start")
    reducer = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        _stage("process group up")
        if args.allreduce == "peer":
            from nanovllm_jax_b200.comm import PeerAllReduce
            reducer = PeerAllReduce(args.requests * 4096 * 2)
            _stage("peer buffers mapped")
    cfg = Qwen3Config(layers=args.layers, max_position=max(4096, args.prompt_len + args.gen_len))
    model = Qwen3(cfg, world, rank, dev, fused=not args.unfused, reducer=reducer)
    _stage("weights drawn")
    rng = np.random.Generator(np.random.PCG64(5000))
    prompts = rng.integers(0, cfg.vocab, size=(args.requests, args.prompt_len))
    eng = Engine(model, prompts, args.gen_len)
    torch.cuda.synchronize()
    _stage("cache allocated")
    if world > 1:
        dist.barrier()
        _stage("barrier passed")
    t0 = time.perf_counter()
    first = eng.prefill()
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0
    _stage(f"prefill done in {t_prefill:.2f}s")
    use_graph = (not args.no_graph) and (world == 1 or reducer is not None)
    model.allreduce_calls = 0
    tokens, t_decode = eng.decode(first, use_graph=use_graph)
    _stage(f"decode done in {t_decode:.2f}s")
    ar_per_step = model.allreduce_calls // max(args.gen_len - 1, 1) if eng.graph is None else 2 * cfg.layers * (world > 1)
    ar_us = None
    if world > 1:
        t = torch.tensor([t_prefill, t_decode], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_prefill, t_decode = float(t[0]), float(t[1])
        ar_us = time_allreduce(model, args.requests)
        _stage("all-reduce timed")
    if rank == 0:
        n_dec = args.requests * (args.gen_len - 1)
        ms_step = t_decode / (args.gen_len - 1) * 1e3
        line = {
            "metric": "decode_tokens_per_s", "value": n_dec / t_decode, "unit": "tokens/s", "n_gpus": world,
            "decode_steps": args.gen_len - 1, "ms_per_decode_step": ms_step,
            "prefill_s": t_prefill, "prefill_tokens_per_s": args.requests * args.prompt_len / t_prefill,
            "end_to_end_tokens_per_s": args.requests * args.gen_len / (t_prefill + t_decode),
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "cuda_graph": eng.graph is not None,
            "cuda_graph_error": eng.graph_error,
            "allreduce": None if world == 1 else {
                "implementation": "PeerAllReduce (one-shot NVLink kernel, residual add fused)" if reducer is not None
                                  else "torch.distributed all_reduce (NCCL) + residual add",
                "calls_per_step": ar_per_step, "message_bytes": args.requests * cfg.hidden * 2,
                "us_per_call": ar_us, "share_of_decode_step": ar_us * ar_per_step / (ms_step * 1e3),
                "how": "CUDA events around 144 back-to-back calls of the decode-size reduction, max over ranks"},
            "config": {"model": f"random-init Qwen3-8B shape, {args.layers} layers, hidden 4096, 32/8 heads x 128, "
                                "intermediate 12288, vocab 151936", "requests": args.requests,
                       "prompt_len": args.prompt_len, "gen_len": args.gen_len, "parallelism": f"tp{world}",
                       "sampling": "greedy argmax on device, token ids copied to the host every step",
                       "pre_attention": "torch ops" if args.unfused else "fused qk-norm + rope + store kernels",
                       "outside_attention": "torch bf16 GEMMs, torch RMSNorm/SiLU"},
            "tokens_checksum": int(tokens.sum() % 1000003),
            "first_tokens_checksum": int(tokens[:, 0].sum() % 1000003),
            "prefill_hidden_mean_abs": float(eng.fingerprint[0]) / (args.requests * cfg.hidden),
            "prefill_top_logit_mean": float(eng.fingerprint[1]) / args.requests,
            "checksum_note": "weights are identical at every tensor-parallel size, but the order of the bf16 sums over "
                             "ranks is not, and the argmax over 151936 random-init logits has near-ties at that noise "
                             "level: the token checksums differ between tensor-parallel sizes, the two float "
                             "fingerprints of the prefill (mean |hidden| of the last positions, mean top logit) agree "
                             "to about three digits"}
        print(json.dumps(line), flush=True)
    if reducer is not None:
        reducer.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
