"""One-shot NVLink all-reduce for decode-size messages (csrc/allreduce.cu) behind torch.distributed plumbing.

The reference sums the partial outputs of its row-parallel projections over the tensor-parallel ranks
(RowParallelLinear.__call__, layers/linear.py:486-510; o_proj at models/qwen3.py:170, down_proj at :230).  At decode
sizes (batch x hidden bf16: a megabyte or less) the sum is latency-bound, and there are 72 of them per step of a
36-layer model.  ``PeerAllReduce`` gives every rank of ONE node a buffer that all other ranks map through CUDA IPC and
reduces with a single kernel per call: copy in, flag the peers, wait for their flags, add up everybody's copy in rank
order (so every rank gets bit-identical sums), optionally adding the residual stream in the same pass.

torch.distributed is used once, at construction, to exchange the 64-byte IPC handles (any backend: the handles travel
as Python objects).  Larger messages fall back to the process group's own all-reduce (NCCL).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib


class PeerAllReduce:
    """Sum over the ranks of ``group`` (all on one node, one GPU each) for bf16 tensors of up to ``max_bytes``."""

    def __init__(self, max_bytes: int, group=None, device=None, max_spins: int = 1 << 22):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("PeerAllReduce serves the GPUs of one node (at most 8 ranks)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_bytes = int(max_bytes)
        self.max_spins = int(max_spins)
        self.epoch = 0
        lib = _lib.load()
        self._lib = lib
        handle = ctypes.create_string_buffer(64)
        mine = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(lib.nvllm_b200_comm_alloc(self.max_bytes, ctypes.byref(mine), handle))
        self._mine = mine.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self._opened = []
        ptrs = (ctypes.c_void_p * self.world)()
        with torch.cuda.device(self.device):
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs[r] = self._mine
                else:
                    p = ctypes.c_void_p()
                    _lib.check(lib.nvllm_b200_comm_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)))
                    self._opened.append(p.value)
                    ptrs[r] = p.value
        self._ptrs = ptrs
        dist.barrier(group=group)  # nobody signals a peer whose buffer is not mapped yet

    def all_reduce_(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """In place: x = sum over ranks of x (+ residual).  bf16, contiguous, numel a multiple of 8."""
        nbytes = x.numel() * x.element_size()
        if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.numel() % 8 or nbytes > self.max_bytes:
            dist.all_reduce(x, group=self.group)  # not a decode-size bf16 message: the process group's collective
            if residual is not None:
                x.add_(residual)
            return x
        if residual is not None and (residual.dtype != x.dtype or residual.shape != x.shape or not residual.is_contiguous()):
            raise ValueError("residual must match x")
        self.epoch += 1  # bookkeeping only: the kernel numbers the calls itself (epoch 0), which survives graph replay
        with torch.cuda.device(self.device):
            _lib.check(self._lib.nvllm_b200_allreduce_sum(
                x.data_ptr(), x.data_ptr(), residual.data_ptr() if residual is not None else None, self._ptrs,
                self.rank, self.world, x.numel(), self.max_bytes, 0, self.max_spins,
                torch.cuda.current_stream(self.device).cuda_stream))
        return x

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (after every rank has stopped using them)."""
        if self._mine is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self._lib.nvllm_b200_comm_close(ctypes.c_void_p(p))
            dist.barrier(group=self.group)
            self._lib.nvllm_b200_comm_free(ctypes.c_void_p(self._mine))
        self._opened, self._mine = [], None
