import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _has_cuda() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# ---- helpers shared by the GPU tests ---------------------------------------------------------


def bits_to_torch(bits: np.ndarray, device="cuda"):
    """uint16 bf16 bit patterns -> torch.bfloat16 tensor on `device`."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).to(device)


def torch_to_bits(t) -> np.ndarray:
    """torch.bfloat16 tensor -> uint16 bit patterns (numpy, host)."""
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def torch_to_f32(t) -> np.ndarray:
    return t.detach().float().cpu().numpy()


# Acceptance tolerances for bf16 attention outputs against the fp32 oracle.
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3


def assert_attention_close(got_f32: np.ndarray, want_f32: np.ndarray, what: str = ""):
    diff = np.abs(got_f32.astype(np.float64) - want_f32.astype(np.float64))
    assert np.isfinite(got_f32).all(), f"{what}: non-finite output"
    mx, mean = float(diff.max(initial=0.0)), float(diff.mean()) if diff.size else 0.0
    assert mx <= MAX_ABS_TOL and mean <= MEAN_ABS_TOL, f"{what}: max-abs {mx:.3e} mean-abs {mean:.3e}"
    return mx, mean
