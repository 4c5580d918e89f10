"""One buffer for a step's inputs: several tensors laid out in a single allocation so that a step's host -> device
transfer is ONE copy instead of one per tensor (six small copies cost more host time than the bytes they move)."""
from __future__ import annotations

import torch


def packed_like(tensors, device, pin: bool = False, align: int = 256):
    """Returns ``(flat, views)``: a uint8 buffer on ``device`` and, for every tensor of ``tensors``, a tensor of the same
    shape and dtype that aliases a 256-byte-aligned slice of ``flat`` (contents uninitialised).

    Copying one ``flat`` onto another built from the same ``tensors`` moves all of them at once; with ``pin`` the
    (CPU) buffer is page-locked so that the copy can be asynchronous.
    """
    offsets, total = [], 0
    for t in tensors:
        total = (total + align - 1) // align * align
        offsets.append(total)
        total += t.numel() * t.element_size()
    flat = torch.empty(max(total, 1), dtype=torch.uint8, device=device)
    if pin:
        flat = flat.pin_memory()
    views = [flat[o:o + t.numel() * t.element_size()].view(t.dtype).view(t.shape) for o, t in zip(offsets, tensors)]
    return flat, views
