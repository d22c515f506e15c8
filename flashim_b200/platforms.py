"""Platform description used by op dispatch: the device, its compute capability and the features kernels may require.

Mirrors the surface of FlashIM's ``flashim.platforms`` that the conv path touches (``Feature``, ``Platform``,
``platform_for``, ``register_detector``; flashim/platforms/base.py:18-80, flashim/platforms/detect.py:25-75,
flashim/platforms/nvidia.py:83-121) and adds the one probe this backend needs: whether the sm_100a kernel library is
built (``Feature.SM100A_KERNELS``).
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass, field
from enum import Enum

import torch

from flashim_b200 import _native


class Feature(str, Enum):
    NVCC = "nvcc"
    MMA_SYNC = "mma_sync"
    TMA = "tma"
    WGMMA = "wgmma"
    TCGEN05 = "tcgen05"
    FP8_E4M3 = "fp8_e4m3"
    MXFP8_SCALED_MM = "mxfp8_scaled_mm"
    CUDA_GRAPHS = "cuda_graphs"
    #: ``libflashim_sm100.so`` (tcgen05 / TMA kernels compiled for sm_100a) is present and loadable
    SM100A_KERNELS = "sm100a_kernels"


@dataclass(frozen=True)
class Platform:
    device_type: str
    device_index: int | None = None
    name: str = ""
    capability: tuple[int, int] | None = None
    features: frozenset[Feature] = field(default_factory=frozenset)
    arch: str = ""

    @property
    def device(self) -> torch.device:
        return torch.device(self.device_type, self.device_index)

    def supports(self, *features: Feature) -> bool:
        return all(f in self.features for f in features)

    def has_capability(self, minimum: tuple[int, int]) -> bool:
        return self.capability is not None and self.capability >= minimum

    def describe(self) -> str:
        feats = ",".join(sorted(f.value for f in self.features)) or "-"
        return f"{self.device_type}{' ' + self.arch if self.arch else ''} ({self.name or 'unknown'}) features={feats}"


def isa_features(capability: tuple[int, int]) -> set[Feature]:
    """Hardware features of a compute capability (flashim/platforms/nvidia.py:83-94)."""
    features: set[Feature] = set()
    if capability >= (8, 0):
        features.add(Feature.MMA_SYNC)
    if capability >= (9, 0):
        features.add(Feature.TMA)
    if capability == (9, 0):
        features.add(Feature.WGMMA)
    if capability[0] in (10, 11):
        features.add(Feature.TCGEN05)
    return features


def sm100a_kernels_usable(capability: tuple[int, int]) -> bool:
    """The sm_100a build only runs on compute capability 10.0 (arch-specific code is not forward compatible)."""
    return capability == (10, 0) and _native.available()


def detect_cuda(index: int) -> Platform:
    capability = torch.cuda.get_device_capability(index)
    features = {Feature.CUDA_GRAPHS, *isa_features(capability)}
    if hasattr(torch, "float8_e4m3fn") and capability >= (8, 9):
        features.add(Feature.FP8_E4M3)
    if capability >= (10, 0) and hasattr(torch, "float8_e8m0fnu"):
        features.add(Feature.MXFP8_SCALED_MM)
    if sm100a_kernels_usable(capability):
        features.add(Feature.SM100A_KERNELS)
    return Platform("cuda", index, torch.cuda.get_device_name(index), capability, frozenset(features),
                    f"sm_{capability[0]}{capability[1]}")


Detector = Callable[[int], Platform]
_DETECTORS: dict[str, Detector] = {"cuda": detect_cuda}
_PLATFORMS: dict[tuple[str, int | None], Platform] = {}


def register_detector(device_type: str, detector: Detector) -> None:
    _DETECTORS[device_type] = detector
    _PLATFORMS.clear()


def default_device() -> torch.device:
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


def platform_for(device: torch.device | str | None = None) -> Platform:
    device = torch.device(device if device is not None else default_device())
    index = device.index
    if device.type == "cuda" and index is None:
        index = torch.cuda.current_device()
    key = (device.type, index)
    platform = _PLATFORMS.get(key)
    if platform is None:
        detector = _DETECTORS.get(device.type)
        platform = Platform(device.type, index, device.type) if detector is None or device.type == "cpu" else detector(index)
        _PLATFORMS[key] = platform
    return platform
