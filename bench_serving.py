#!/usr/bin/env python
"""End-to-end decode throughput (tokens/s) of a random-init Qwen3-8B-shaped model whose attention runs on this
library, at 1/2/4/8 GPUs with tensor parallelism.

    python bench_serving.py [--gpus N] [--requests 128] [--prompt-len 512] [--gen-len 256] [--layers 36] [--no-graph]
    (N > 1: python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench_serving.py --gpus N)

What is measured is the serving loop of the reference (engine/llm_engine.py:120-165): prefill first, in batches of at
most 16 384 prompt tokens, then one decode step per generated token for all requests, greedy sampling, token ids
read back to the host every step.  Everything AROUND attention is deliberately plain: torch bf16 GEMMs (cuBLAS),
torch RMSNorm / RoPE / SiLU, NCCL all-reduce after o_proj and down_proj (the row-parallel reductions of
layers/linear.py:497-503), replicated embedding and LM head, sequential page allocation.  Attention -- store_kvcache,
paged decode, varlen prefill -- goes through ``nanovllm_jax_b200.layers.attention.Attention`` with per-rank head
counts and a per-rank KV-cache shard, exactly as the reference's model would call it (models/qwen3.py:114-120,166).

Status of the numbers: the single-GPU run (CUDA graph replay of the decode step) is measured.  With more than one
rank the decode step is launched eagerly unless --graph is given: the only multi-rank attempt so far captured the step
(NCCL all-reduces included) into a CUDA graph on every rank and did not finish, and no GPU time was left to find out
why (one candidate: a capture that fails on one rank only, which would leave that rank issuing live all-reduces
against ranks that merely recorded theirs).  Multi-GPU tokens/s are therefore NOT measured yet.

The model is NOT part of the library; it exists so that the attention path can be timed inside a realistic decode
step.  Weights are N(0, 0.02) random (there is no checkpoint in the image), prompts are uniform random token ids.
Prints one JSON line on rank 0.
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

from nanovllm_jax_b200.layers.attention import Attention  # noqa: E402
from nanovllm_jax_b200.utils.context import create_decode_context, create_prefill_context  # noqa: E402


class Qwen3Config:
    """Qwen3-8B sizes (dense, GQA, QK-norm, RoPE, SwiGLU)."""

    def __init__(self, layers=36, hidden=4096, heads=32, kv_heads=8, head_dim=128, intermediate=12288, vocab=151936,
                 rope_theta=1e6, eps=1e-6, block_size=256):
        self.layers, self.hidden, self.heads, self.kv_heads, self.head_dim = layers, hidden, heads, kv_heads, head_dim
        self.intermediate, self.vocab, self.rope_theta, self.eps, self.block_size = (intermediate, vocab, rope_theta, eps,
                                                                                     block_size)


def _rand(shape, gen, dev, std=0.02):
    return (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * std).to(torch.bfloat16)


class Layer:
    def __init__(self, cfg, tp, gen, dev):
        h, d = cfg.hidden, cfg.head_dim
        self.hq, self.hk = cfg.heads // tp, cfg.kv_heads // tp
        self.w_qkv = _rand(((self.hq + 2 * self.hk) * d, h), gen, dev)         # column-parallel
        self.w_o = _rand((h, self.hq * d), gen, dev)                           # row-parallel
        self.w_gate_up = _rand((2 * cfg.intermediate // tp, h), gen, dev)      # column-parallel
        self.w_down = _rand((h, cfg.intermediate // tp), gen, dev)             # row-parallel
        self.ln1 = torch.ones(h, dtype=torch.bfloat16, device=dev)
        self.ln2 = torch.ones(h, dtype=torch.bfloat16, device=dev)
        self.q_norm = torch.ones(d, dtype=torch.bfloat16, device=dev)
        self.k_norm = torch.ones(d, dtype=torch.bfloat16, device=dev)
        self.attn = Attention(self.hq, d, 1.0 / math.sqrt(d), self.hk, cfg.block_size)


class Qwen3:
    """Forward pass only; `attention` selects this library ('b200') or a dense torch reference ('torch', tests only)."""

    def __init__(self, cfg: Qwen3Config, tp: int, rank: int, dev, seed: int = 0):
        self.cfg, self.tp, self.rank, self.dev = cfg, tp, rank, dev
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)                          # embedding / head replicated: same draw on every rank
        self.embed = _rand((cfg.vocab, cfg.hidden), gen, dev)
        self.lm_head = _rand((cfg.vocab, cfg.hidden), gen, dev)
        self.final_ln = torch.ones(cfg.hidden, dtype=torch.bfloat16, device=dev)
        gen.manual_seed(seed * 1000 + 17 + rank)       # sharded weights: each rank draws its own slice
        self.layers = [Layer(cfg, tp, gen, dev) for _ in range(cfg.layers)]
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=dev, dtype=torch.float32) / cfg.head_dim))
        self.inv_freq = inv

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

    def _all_reduce(self, x):
        if self.tp > 1:
            dist.all_reduce(x)
        return x

    def forward(self, ids, positions, ctx, dense_attention=None):
        """ids, positions: [T] on device.  Returns hidden states [T, hidden]."""
        cfg = self.cfg
        d = cfg.head_dim
        x = self.embed[ids]
        for layer in self.layers:
            h = F.rms_norm(x, (cfg.hidden,), layer.ln1, cfg.eps)
            qkv = h @ layer.w_qkv.t()
            q, k, v = qkv.split([layer.hq * d, layer.hk * d, layer.hk * d], dim=-1)
            q = F.rms_norm(q.view(-1, layer.hq, d), (d,), layer.q_norm, cfg.eps)
            k = F.rms_norm(k.view(-1, layer.hk, d), (d,), layer.k_norm, cfg.eps)
            q, k = self._rope(q, positions), self._rope(k, positions)
            v = v.reshape(-1, layer.hk, d)
            if dense_attention is None:
                o = layer.attn(q.contiguous(), k.contiguous(), v.contiguous(), ctx)
            else:
                o = dense_attention(layer, q, k, v)
            x = x + self._all_reduce(o.reshape(-1, layer.hq * d) @ layer.w_o.t())
            h = F.rms_norm(x, (cfg.hidden,), layer.ln2, cfg.eps)
            gate, up = (h @ layer.w_gate_up.t()).chunk(2, dim=-1)
            x = x + self._all_reduce((F.silu(gate) * up) @ layer.w_down.t())
        return F.rms_norm(x, (cfg.hidden,), self.final_ln, cfg.eps)

    def logits(self, hidden):
        return hidden @ self.lm_head.t()


class Engine:
    """Static-batch serving loop: every request prefills, then all decode together (what the reference's scheduler does
    with max_num_seqs >= requests: prefill first, engine/scheduler.py:81-100, then decode, :103-125)."""

    def __init__(self, model: Qwen3, prompts: np.ndarray, gen_len: int, max_batched_tokens: int = 16384, seed: int = 0):
        self.m, self.prompts, self.gen_len = model, prompts, gen_len
        self.n, self.plen = prompts.shape
        cfg = model.cfg
        self.blk = cfg.block_size
        self.max_blocks = -(-(self.plen + gen_len) // self.blk)
        rng = np.random.Generator(np.random.PCG64(seed))
        num_blocks = self.n * self.max_blocks + 8
        perm = rng.permutation(num_blocks).astype(np.int32)
        self.tables = perm[: self.n * self.max_blocks].reshape(self.n, self.max_blocks)  # pages pre-assigned per request
        model.allocate_cache(num_blocks)
        self.per_prefill = max(1, max_batched_tokens // self.plen)
        dev = model.dev
        # static device buffers for the decode step (graph-replayable: same shapes every step)
        self.d_ids = torch.zeros(self.n, dtype=torch.int64, device=dev)
        self.d_pos = torch.zeros(self.n, dtype=torch.int64, device=dev)
        self.d_ctx = torch.zeros(self.n, dtype=torch.int32, device=dev)
        self.d_slots = torch.zeros(self.n, dtype=torch.int32, device=dev)
        self.d_tables = torch.from_numpy(self.tables).to(dev)
        self.h_meta = torch.zeros((3, self.n), dtype=torch.int32).pin_memory()
        self.h_tokens = torch.zeros(self.n, dtype=torch.int64).pin_memory()
        self.decode_ctx = create_decode_context(self.d_ctx, self.d_slots, self.d_tables)
        self.graph = None
        self.graph_error = None

    # ---- prefill ----
    def prefill(self):
        dev, cfg = self.m.dev, self.m.cfg
        first = torch.empty(self.n, dtype=torch.int64, device=dev)
        for s0 in range(0, self.n, self.per_prefill):
            s1 = min(self.n, s0 + self.per_prefill)
            b = s1 - s0
            ids = torch.from_numpy(self.prompts[s0:s1].reshape(-1).astype(np.int64)).to(dev)
            pos = torch.arange(self.plen, device=dev).repeat(b)
            cu_host = (np.arange(b + 1) * self.plen).astype(np.int32)
            slots = (self.tables[s0:s1, :, None] * self.blk + np.arange(self.blk)[None, None, :]).reshape(b, -1)[:, : self.plen]
            ctx = create_prefill_context(torch.from_numpy(cu_host).to(dev), torch.from_numpy(cu_host).to(dev), self.plen,
                                         self.plen, torch.from_numpy(slots.reshape(-1).astype(np.int32)).to(dev),
                                         cu_seqlens_host=cu_host)
            hidden = self.m.forward(ids, pos, ctx)
            last = hidden[torch.from_numpy(cu_host[1:].astype(np.int64) - 1).to(dev)]
            first[s0:s1] = self.m.logits(last).argmax(dim=-1)
        return first

    # ---- decode ----
    def _decode_step_device(self):
        hidden = self.m.forward(self.d_ids, self.d_pos, self.decode_ctx)
        self.d_ids.copy_(self.m.logits(hidden).argmax(dim=-1))

    def decode(self, first_tokens, use_graph: bool):
        n, blk = self.n, self.blk
        self.d_ids.copy_(first_tokens)
        out = np.zeros((n, self.gen_len), dtype=np.int64)
        out[:, 0] = first_tokens.cpu().numpy()
        rows = np.arange(n)

        def set_meta(step):  # token generated at `step` sits at position plen + step - 1 ... the one fed now is step-1
            length = self.plen + step               # context length once this step's token is stored
            pos = length - 1
            self.h_meta[0].fill_(pos)
            self.h_meta[1].fill_(length)
            self.h_meta[2].copy_(torch.from_numpy(self.tables[rows, pos // blk] * blk + pos % blk))
            self.d_pos.copy_(self.h_meta[0], non_blocking=True)
            self.d_ctx.copy_(self.h_meta[1], non_blocking=True)
            self.d_slots.copy_(self.h_meta[2], non_blocking=True)

        if use_graph and self.graph is None:
            set_meta(1)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._decode_step_device()      # warm-up on the side stream (allocations, cuBLAS handles)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.d_ids.copy_(first_tokens)
            try:
                g = torch.cuda.CUDAGraph()
                # thread_local: the NCCL watchdog thread may touch CUDA while this thread captures
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    self._decode_step_device()
                self.graph = g
            except Exception as exc:  # capture unsupported here: run the step eagerly and say so
                self.graph = None
                self.graph_error = f"{type(exc).__name__}: {exc}"[:200]
                torch.cuda.synchronize()
            if self.m.tp > 1:
                # Every rank must take the same path: a rank replaying a graph never meets a rank that issues its
                # all-reduces live.  One failed capture sends everybody to the eager step.
                agreed = torch.tensor([1 if self.graph is not None else 0], device=self.m.dev)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
                if int(agreed.item()) == 0:
                    self.graph = None
                    self.graph_error = self.graph_error or "capture failed on another rank"
            self.d_ids.copy_(first_tokens)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for step in range(1, self.gen_len):
            set_meta(step)
            if self.graph is not None:
                self.graph.replay()
            else:
                self._decode_step_device()
            self.h_tokens.copy_(self.d_ids, non_blocking=True)
            torch.cuda.current_stream().synchronize()   # the scheduler needs the tokens (EOS / max_tokens checks)
            out[:, step] = self.h_tokens.numpy()
        return out, time.perf_counter() - t0


def _stage(msg: str) -> None:
    """Progress marker on stderr (NVLLM_SERVING_VERBOSE=1): shows how far each rank got if a run stalls."""
    if os.environ.get("NVLLM_SERVING_VERBOSE", "0") == "1":
        print(f"[rank {os.environ.get('RANK', '0')} +{time.perf_counter() - _T0:7.1f}s] {msg}", file=sys.stderr, flush=True)


_T0 = time.perf_counter()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--gen-len", type=int, default=256)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--no-graph", action="store_true", help="launch the decode step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--graph", action="store_true", help="with more than one rank: capture the decode step anyway")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    _stage("start")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        _stage("process group up")
    cfg = Qwen3Config(layers=args.layers)
    model = Qwen3(cfg, world, rank, dev)
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
    use_graph = (not args.no_graph) and (world == 1 or args.graph)
    tokens, t_decode = eng.decode(first, use_graph=use_graph)
    _stage(f"decode done in {t_decode:.2f}s")
    if world > 1:
        t = torch.tensor([t_prefill, t_decode], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_prefill, t_decode = float(t[0]), float(t[1])
    if rank == 0:
        n_dec = args.requests * (args.gen_len - 1)
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": n_dec / t_decode, "unit": "tokens/s", "n_gpus": world,
            "decode_steps": args.gen_len - 1, "ms_per_decode_step": t_decode / (args.gen_len - 1) * 1e3,
            "prefill_s": t_prefill, "prefill_tokens_per_s": args.requests * args.prompt_len / t_prefill,
            "end_to_end_tokens_per_s": args.requests * args.gen_len / (t_prefill + t_decode),
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "cuda_graph": eng.graph is not None, "cuda_graph_error": eng.graph_error,
            "config": {"model": f"random-init Qwen3-8B shape, {args.layers} layers, hidden 4096, 32/8 heads x 128, "
                                "intermediate 12288, vocab 151936", "requests": args.requests,
                       "prompt_len": args.prompt_len, "gen_len": args.gen_len, "parallelism": f"tp{world}",
                       "sampling": "greedy argmax on device, token ids copied to the host every step",
                       "outside_attention": "torch bf16 GEMMs, torch RMSNorm/RoPE/SiLU, NCCL all-reduce"},
            "tokens_checksum": int(tokens.sum() % 1000003)}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
