"""Fixed-shape decode metadata: what makes a decode step replayable (CUDA graph, jit cache hit).

The reference pads nothing: every decode step builds ``input_ids``, ``positions``, ``slot_mapping``, ``context_lens``
and a ``block_tables`` array whose width is the longest block table of the batch (engine/model_runner.py:225-246,
340-374), so each new (batch, width) pair is a new XLA program -- the launch overhead the reference names as its first
gap (docs/pytorch_vs_jax_comparison.md:47-66, 102-121).  Its only concession is the list of batch sizes it means to
pre-compile (``compiled_bs``, engine/model_runner.py:209-210).

This module holds the step's metadata in ONE device buffer of fixed layout, filled from one pinned host buffer with a
single asynchronous copy per step:

  * the batch is padded up to the reference's own bucket list (1, 2, 4, 8, 16, 32, ... in steps of 16);
  * the block-table width is padded up to a power of two;
  * padded rows are inert for the kernels of this library: ``context_lens = 0`` (the row attends to nothing and comes
    back as zeros), ``slot_mapping = -1`` (nothing is stored), ``block_tables = -1``, ``input_ids = positions = 0``.

The tensors handed out are views of the same storage for the lifetime of the object, so a step captured once per
(bucketed batch, bucketed width) replays with whatever the next ``update`` copied in.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .context import AttentionContext, create_decode_context
from .staging import packed_like


def compiled_batch_sizes(max_num_seqs: int) -> list[int]:
    """The batch sizes the reference pre-compiles (engine/model_runner.py:209-210)."""
    max_bs = min(int(max_num_seqs), 512)
    return [b for b in (1, 2, 4, 8) if b <= max(max_bs, 1)] + list(range(16, max_bs + 1, 16))


def bucket_batch(n: int, max_num_seqs: int) -> int:
    """Smallest compiled batch size >= n (n itself beyond the list: the reference would compile it on the fly)."""
    for b in compiled_batch_sizes(max_num_seqs):
        if b >= n:
            return b
    return n


def bucket_blocks(n: int, min_blocks: int = 1) -> int:
    """Block-table width rounded up to a power of two."""
    n = max(int(n), min_blocks, 1)
    return 1 << (n - 1).bit_length()


class DecodeMetadata:
    """Pointer-stable decode metadata for up to ``max_batch`` sequences with up to ``max_blocks`` pages each.

    ``update(...)`` writes one step's metadata (padding included) into pinned host memory and enqueues ONE host ->
    device copy on the current stream; ``context(batch, width)`` returns an AttentionContext whose tensors alias the
    device buffer for that bucket.  Host-side logic works with ``device='cpu'`` too (used by the CPU tests).
    """

    def __init__(self, max_batch: int, max_blocks: int, device, pin: bool | None = None):
        self.max_batch = int(max_batch)
        self.max_blocks = bucket_blocks(max_blocks)
        self.device = torch.device(device)
        pin = self.device.type == "cuda" if pin is None else pin
        b, w = self.max_batch, self.max_blocks
        like = (torch.empty(b, dtype=torch.int32), torch.empty(b, dtype=torch.int32), torch.empty(b, dtype=torch.int32),
                torch.empty(b, dtype=torch.int32), torch.empty((b, w), dtype=torch.int32))
        self._host_flat, hv = packed_like(like, "cpu", pin=pin)
        self._dev_flat, dv = packed_like(like, self.device)
        self.h_ids, self.h_pos, self.h_slots, self.h_ctx, self.h_tables = hv
        self.input_ids, self.positions, self.slot_mapping, self.context_lens, self.block_tables = dv
        self._host_flat.zero_()
        self.h_slots.fill_(-1)
        self.h_tables.fill_(-1)
        self._dev_flat.copy_(self._host_flat)
        self.batch = 0          # live sequences of the last update
        self.padded_batch = 0   # its bucket
        self.width = 1          # bucketed block-table width of the last update

    def update(self, input_ids: Sequence[int], positions: Sequence[int], slot_mapping: Sequence[int],
               context_lens: Sequence[int], block_tables: Sequence[Sequence[int]], max_num_seqs: int | None = None):
        """One step's metadata, as engine/model_runner.py:340-374 computes it, into the fixed buffers.
        Returns (padded_batch, width): the bucket a captured step is keyed by."""
        n = len(input_ids)
        if not (len(positions) == len(slot_mapping) == len(context_lens) == len(block_tables) == n):
            raise ValueError("per-sequence lists differ in length")
        if n > self.max_batch:
            raise ValueError(f"{n} sequences exceed the buffers' {self.max_batch}")
        longest = max((len(t) for t in block_tables), default=1)
        if longest > self.max_blocks:
            raise ValueError(f"a block table of {longest} pages exceeds the buffers' {self.max_blocks}")
        nb = min(bucket_batch(max(n, 1), max_num_seqs if max_num_seqs is not None else self.max_batch), self.max_batch)
        nb = max(nb, n)
        self.h_ids[:n] = torch.as_tensor(np.asarray(input_ids, dtype=np.int32))
        self.h_pos[:n] = torch.as_tensor(np.asarray(positions, dtype=np.int32))
        self.h_slots[:n] = torch.as_tensor(np.asarray(slot_mapping, dtype=np.int32))
        self.h_ctx[:n] = torch.as_tensor(np.asarray(context_lens, dtype=np.int32))
        # rows that were live in an earlier, larger batch become padding again
        hi = max(self.padded_batch, nb)
        self.h_ids[n:hi] = 0
        self.h_pos[n:hi] = 0
        self.h_slots[n:hi] = -1
        self.h_ctx[n:hi] = 0
        self.h_tables[:hi].fill_(-1)
        for i, t in enumerate(block_tables):
            if len(t):
                self.h_tables[i, :len(t)] = torch.as_tensor(np.asarray(t, dtype=np.int32))
        self._dev_flat.copy_(self._host_flat, non_blocking=True)  # the step's single host -> device copy
        self.batch, self.padded_batch, self.width = n, nb, bucket_blocks(longest)
        return nb, self.width

    def context(self, padded_batch: int | None = None, width: int | None = None) -> AttentionContext:
        """AttentionContext over the first ``padded_batch`` rows.  The block tables keep the buffers' full width (a
        narrower view would not be contiguous); ``width`` only names the bucket -- columns beyond a row's pages hold -1
        and are never read."""
        nb = self.padded_batch if padded_batch is None else padded_batch
        return create_decode_context(context_lens=self.context_lens[:nb], slot_mapping=self.slot_mapping[:nb],
                                     block_tables=self.block_tables[:nb])

    def inputs(self, padded_batch: int | None = None):
        """(input_ids, positions) views for the model's embedding / RoPE, same rows as ``context``."""
        nb = self.padded_batch if padded_batch is None else padded_batch
        return self.input_ids[:nb], self.positions[:nb]
