"""Shared fixtures. Tests that need a GPU carry ``@pytest.mark.gpu``; everything else runs on the CPU."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.x (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _as_tensor(array: np.ndarray, dtype: torch.dtype | None = None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(array))
    if dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu):
        return t.view(torch.uint8).view(dtype)
    if dtype == torch.bfloat16:
        return t.view(torch.bfloat16)
    return t if dtype is None else t.to(dtype)


class Golden:
    """A ``tests/golden/<name>.npz`` fixture; ``g("key", dtype)`` returns the stored bytes as a tensor of ``dtype``."""

    def __init__(self, name: str) -> None:
        self.data = np.load(GOLDEN / f"{name}.npz")

    def __contains__(self, key: str) -> bool:
        return key in self.data.files

    def __call__(self, key: str, dtype: torch.dtype | None = None) -> torch.Tensor:
        return _as_tensor(self.data[key], dtype)

    def get(self, key: str, dtype: torch.dtype | None = None):
        return self(key, dtype) if key in self else None


@pytest.fixture(scope="session")
def golden():
    cache: dict[str, Golden] = {}

    def load(name: str) -> Golden:
        if name not in cache:
            cache[name] = Golden(name)
        return cache[name]

    return load


def same_bytes(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Bitwise equality of two tensors of the same dtype family (fp8 / bf16 compared as integers)."""
    if a.shape != b.shape:
        return False
    size = a.element_size()
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[size]
    return torch.equal(a.contiguous().view(view), b.contiguous().view(view))


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 units in the last place between two bf16 tensors (monotone integer mapping of the bits)."""
    def key(t):
        bits = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(bits < 0, -(bits & 0x7FFF), bits)
    return (key(a) - key(b)).abs()


# Tests check the device status word after every launch (a kernel whose bounded wait ran out reports there).
import os  # noqa: E402

os.environ.setdefault("FLASHIM_B200_CHECK", "1")

DEV = "cuda"


def to_dev(*tensors):
    out = tuple(None if t is None else t.to(DEV) for t in tensors)
    return out if len(out) > 1 else out[0]


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def code_mismatch(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.cpu().contiguous().view(torch.uint8) != b.cpu().contiguous().view(torch.uint8)).float().mean())
