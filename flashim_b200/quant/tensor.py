"""Quantized tensor containers and the load-time weight packing of the conv path.

Same containers and field names as FlashIM (flashim/quant/tensor.py:16-145) so modules written against them work
unchanged: ``QuantizedTensor`` (E4M3 activations + one static exponent per 32 channels), ``QuantizedWeight`` (E4M3
``[N, K]`` + one exponent per (row, 32 inputs)), ``Int8Tensor``. Weight packing runs once when a model is built, in
torch on the weights' own device; activations are only ever quantized by the CUDA kernels.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import Tensor

BLOCK = 32
FP8_MAX = 448.0
INT8_MAX = 127.0


def padded_channels(channels: int) -> int:
    return -(-channels // BLOCK) * BLOCK


def scale_exponent_from_amax(amax: Tensor) -> Tensor:
    """int8 exponent ``clamp(ceil(log2(amax / 448)))``, ``-127`` for zero (flashim/quant/formats/mx.py:22-26)."""
    e = torch.ceil(torch.log2(amax / FP8_MAX))
    e = torch.where(amax == 0, torch.full_like(e, -127.0), e)
    return e.clamp(-127, 127).to(torch.int8)


def exponent_to_e8m0(exponent: Tensor) -> Tensor:
    """Biased E8M0 bytes (uint8) of int8 exponents."""
    return (exponent.to(torch.int16) + 127).to(torch.uint8)


def swizzle_scales(exponent: Tensor) -> Tensor:
    """``[rows, groups]`` int8 exponents -> flat uint8 E8M0 bytes in 512-byte tiles of 128 rows x 4 groups (32 rows of 16
    bytes: row ``r % 32``, then ``(r % 128) // 32``, then group), zero padded: the layout tcgen05.cp moves to tensor
    memory unchanged and cuBLAS calls SWIZZLE_32_4_4 (flashim/quant/formats/mx.py:67-86)."""
    raw = exponent_to_e8m0(exponent)
    rows, groups = raw.shape
    pr, pg = -(-rows // 128) * 128, -(-groups // 4) * 4
    padded = torch.zeros((pr, pg), dtype=torch.uint8, device=raw.device)
    padded[:rows, :groups] = raw
    return padded.view(pr // 128, 4, 32, pg // 4, 4).permute(0, 3, 2, 1, 4).reshape(-1).contiguous()


def swizzled_scale_bytes(rows: int, groups: int) -> int:
    return (-(-rows // 128)) * (-(-groups // 4)) * 512


@dataclass(frozen=True)
class QuantizedTensor:
    values: Tensor
    scale_exponent: Tensor
    logical_shape: tuple[int, ...]

    def __post_init__(self) -> None:
        if self.values.dtype != torch.float8_e4m3fn:
            raise ValueError(f"Expected float8_e4m3fn values, got {self.values.dtype}")
        if self.scale_exponent.dtype != torch.int8:
            raise ValueError("scale_exponent must be int8 unbiased exponents")
        channels = self.values.shape[-1]
        if channels % BLOCK or channels < self.logical_shape[-1]:
            raise ValueError(f"Bad physical channels {channels} for {self.logical_shape}")
        if tuple(self.scale_exponent.shape) != (channels // BLOCK,):
            raise ValueError(f"Expected scale shape {(channels // BLOCK,)}")

    @property
    def device(self) -> torch.device:
        return self.values.device

    @property
    def channels(self) -> int:
        return self.values.shape[-1]

    @property
    def rows(self) -> int:
        return math.prod(self.values.shape[:-1])

    def matrix(self) -> Tensor:
        return self.values.reshape(-1, self.channels)

    def dequantize(self, dtype: torch.dtype = torch.float32) -> Tensor:
        blocks = self.values.reshape(self.rows, self.channels // BLOCK, BLOCK).float()
        dense = (blocks * torch.exp2(self.scale_exponent.float())[..., None]).reshape(self.rows, -1)
        return dense[:, : self.logical_shape[-1]].reshape(self.logical_shape).to(dtype)


@dataclass(frozen=True)
class QuantizedWeight:
    values: Tensor
    scale_exponent: Tensor
    logical_shape: tuple[int, int]

    @property
    def out_features(self) -> int:
        return self.values.shape[0]

    @property
    def in_features(self) -> int:
        return self.values.shape[1]

    @classmethod
    def from_float(cls, weight: Tensor) -> "QuantizedWeight":
        """Pad both dimensions to 32, one exponent per (row, 32 inputs), ``w / 2**e`` saturated, E4M3
        (flashim/quant/tensor.py:76-87)."""
        if weight.ndim != 2:
            raise ValueError(f"Unsupported weight shape: {tuple(weight.shape)}")
        if not torch.isfinite(weight).all():
            raise ValueError("Cannot quantize non-finite weights")
        n, k = padded_channels(weight.shape[0]), padded_channels(weight.shape[1])
        blocks = F.pad(weight.float(), (0, k - weight.shape[1], 0, n - weight.shape[0])).reshape(n, k // BLOCK, BLOCK)
        exponent = scale_exponent_from_amax(blocks.abs().amax(dim=-1))
        q = (blocks / torch.exp2(exponent.float())[..., None]).clamp(-FP8_MAX, FP8_MAX)
        return cls(q.reshape(n, k).to(torch.float8_e4m3fn), exponent, tuple(weight.shape))

    @classmethod
    def from_conv(cls, weight: Tensor) -> "QuantizedWeight":
        """``[Cout, Cin, kh, kw]`` -> K order ``(ky, kx, c)`` with ``Cin`` padded to 32 per tap
        (flashim/quant/methods/conv2d.py:193-205)."""
        cout, cin = weight.shape[:2]
        w = F.pad(weight.detach().permute(0, 2, 3, 1), (0, padded_channels(cin) - cin))
        return cls.from_float(w.reshape(cout, -1))

    def swizzled_scales(self) -> Tensor:
        return swizzle_scales(self.scale_exponent)

    def dequantize(self, dtype: torch.dtype = torch.float32) -> Tensor:
        blocks = self.values.reshape(self.out_features, self.in_features // BLOCK, BLOCK).float()
        dense = (blocks * torch.exp2(self.scale_exponent.float())[..., None]).reshape(self.out_features, self.in_features)
        return dense[: self.logical_shape[0], : self.logical_shape[1]].to(dtype)


@dataclass(frozen=True)
class Int8Tensor:
    values: Tensor
    scale: Tensor

    def __post_init__(self) -> None:
        if self.values.dtype != torch.int8:
            raise ValueError(f"Expected int8 values, got {self.values.dtype}")
        if self.scale.dtype != torch.float32 or self.scale.numel() != 1:
            raise ValueError("scale must be a single FP32 value")

    @property
    def logical_shape(self) -> tuple[int, ...]:
        return tuple(self.values.shape)

    def matrix(self) -> Tensor:
        return self.values.reshape(-1, self.values.shape[-1])

    def dequantize(self, dtype: torch.dtype = torch.float32) -> Tensor:
        return (self.values.float() * self.scale).to(dtype)


_EPS = torch.finfo(torch.float32).eps


def safe_scale(scale: Tensor) -> Tensor:
    scale = scale.float()
    return torch.where(torch.isfinite(scale) & (scale > _EPS), scale, torch.full_like(scale, _EPS))


def int8_weight_from_conv(weight: Tensor) -> tuple[Tensor, Tensor]:
    """``[Cout, Cin, kh, kw]`` -> int8 ``[Cout, kh*kw*Cin]`` (ky, kx, c) and fp32 per-row scales ``amax / 127``
    (flashim/quant/methods/conv2d.py:91-100, flashim/quant/formats/int8.py:19-26)."""
    w = weight.detach().permute(0, 2, 3, 1).reshape(weight.shape[0], -1)
    scale = safe_scale(w.float().abs().amax(dim=1) / INT8_MAX)
    q = (w.float() / scale[:, None]).round().clamp(-INT8_MAX, INT8_MAX).to(torch.int8)
    return q.contiguous(), scale
