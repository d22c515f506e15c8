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


# the comparison helpers live in fim_testlib.py (this directory is on sys.path while pytest collects it)
sys.path.insert(0, str(Path(__file__).resolve().parent))
import fim_testlib  # noqa: E402,F401  (sets FLASHIM_B200_CHECK for the whole session)
