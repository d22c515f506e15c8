"""Backend loading, after flashim/backends/_loader.py:14-71: each backend is a module that registers implementations
into the op registry when imported. This package has exactly one, the sm_100a CUDA backend."""

from __future__ import annotations

import importlib
import logging
from dataclasses import dataclass

logger = logging.getLogger("flashim_b200.backends")


@dataclass(frozen=True)
class Backend:
    name: str
    modules: tuple[str, ...]


BACKENDS: tuple[Backend, ...] = (Backend("sm100", ("sm100.kernels",)),)
LOADED: list[str] = []
_done = False


def load() -> None:
    global _done
    if _done:
        return
    _done = True
    for backend in BACKENDS:
        for module in backend.modules:
            importlib.import_module(f"flashim_b200.backends.{module}").register()
        LOADED.append(backend.name)
