"""Containers for quantised operands and the load-time packing of conv weights.

The three containers carry the field names FlashIM's carry (flashim/quant/tensor.py:16-145: ``values`` /
``scale_exponent`` / ``logical_shape``, ``values`` / ``scale``) so a module written against those reads these the same
way: ``QuantizedTensor`` is an E4M3 activation whose 32-channel blocks share one static power-of-two scale across all
rows, ``QuantizedWeight`` an E4M3 ``[N, K]`` matrix with a scale per (row, 32 inputs), ``Int8Tensor`` int8 values under
one fp32 scale. Packing a weight happens once, when a model is built, in torch on the weight's own device; activations
are only ever quantised by the CUDA kernels.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import Tensor

BLOCK = 32          # elements that share one E8M0 scale
FP8_MAX = 448.0     # largest finite E4M3 magnitude
INT8_MAX = 127.0
_SCALE_TILE_ROWS, _SCALE_TILE_GROUPS = 128, 4  # one 512-byte tile of the swizzled scale layout


def _round_up(value: int, multiple: int) -> int:
    return (value + multiple - 1) // multiple * multiple


def padded_channels(channels: int) -> int:
    """Channels as stored: the next multiple of the 32-element block."""
    return _round_up(channels, BLOCK)


# ---- E8M0 scales -----------------------------------------------------------------------------------------------------


def scale_exponent_from_amax(amax: Tensor) -> Tensor:
    """The int8 exponent ``e`` with ``amax / 2**e <= 448``, i.e. ``ceil(log2(amax / 448))`` in fp32, limited to
    [-127, 127]; an all-zero block gets -127 (the rule of flashim/quant/formats/mx.py:22-26)."""
    exponent = torch.log2(amax.float() / FP8_MAX).ceil()
    exponent = exponent.masked_fill(amax == 0, -127.0)
    return exponent.clamp_(-127.0, 127.0).to(torch.int8)


def calibrate_block32_exponent(value: Tensor) -> Tensor:
    """Static per-32-channel exponents of an activation ``[..., C]``: the largest magnitude of each block of 32 channels
    over every row (a trailing ragged block is zero-padded), through :func:`scale_exponent_from_amax`; int8 ``[Cp / 32]``
    (the helper of flashim/quant/formats/mx.py:41-47, as the calibrator uses it, flashim/quant/calibration.py:122-128)."""
    channels = value.shape[-1]
    rows = value.reshape(-1, channels).float()
    padded = padded_channels(channels)
    if padded != channels:
        rows = torch.nn.functional.pad(rows, (0, padded - channels))
    return scale_exponent_from_amax(rows.abs().reshape(-1, padded // BLOCK, BLOCK).amax(dim=(0, 2)))


def exponent_to_e8m0(exponent: Tensor) -> Tensor:
    """int8 exponents -> the biased bytes E8M0 stores (uint8, bias 127)."""
    return (exponent.to(torch.int16) + 127).to(torch.uint8)


def swizzled_scale_bytes(rows: int, groups: int) -> int:
    """Size of the swizzled layout of a ``[rows, groups]`` scale matrix: whole 128 x 4 tiles of 512 bytes."""
    return (_round_up(rows, _SCALE_TILE_ROWS) // _SCALE_TILE_ROWS) * (_round_up(groups, _SCALE_TILE_GROUPS) // _SCALE_TILE_GROUPS) * 512


def swizzle_scales(exponent: Tensor) -> Tensor:
    """``[rows, groups]`` int8 exponents -> flat E8M0 bytes in the tiled order the tensor cores read.

    The matrix is cut into tiles of 128 rows x 4 groups (zero-padded at the edges); a tile is stored as 32 lines of 16
    bytes, line ``r % 32`` holding, for the four 32-row quarters ``q = (r % 128) // 32`` in turn, the 4 group bytes of row
    ``32 q + r % 32``. Tiles follow each other group-tile fastest. ``tcgen05.cp.32x128b.warpx4`` moves such a tile into
    4 tensor-memory columns unchanged; cuBLAS names the order SWIZZLE_32_4_4 and FlashIM's ``swizzle_scales`` produces
    it (flashim/quant/formats/mx.py:67-86)."""
    rows, groups = exponent.shape
    tall, wide = _round_up(rows, _SCALE_TILE_ROWS), _round_up(groups, _SCALE_TILE_GROUPS)
    plane = exponent.new_zeros((tall, wide), dtype=torch.uint8)
    plane[:rows, :groups] = exponent_to_e8m0(exponent)
    # axes: row tile, quarter, line, group tile, group  ->  row tile, group tile, line, quarter, group
    tiles = plane.reshape(tall // _SCALE_TILE_ROWS, 4, 32, wide // _SCALE_TILE_GROUPS, _SCALE_TILE_GROUPS)
    return tiles.permute(0, 3, 2, 1, 4).contiguous().reshape(-1)


def _apply_block_scales(values: Tensor, exponent: Tensor) -> Tensor:
    """``values [R, K]`` (E4M3) times ``2**exponent`` per 32-element block; ``exponent`` is ``[K/32]`` or ``[R, K/32]``."""
    rows, width = values.shape
    scale = torch.exp2(exponent.float()).unsqueeze(-1)
    return (values.float().reshape(rows, width // BLOCK, BLOCK) * scale).reshape(rows, width)


# ---- containers ------------------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class QuantizedTensor:
    """E4M3 ``[*leading, Cp]`` with ``Cp`` the padded channel count, one int8 exponent per 32 channels shared by every
    row, and the unpadded shape the values stand for."""

    values: Tensor
    scale_exponent: Tensor
    logical_shape: tuple[int, ...]

    def __post_init__(self) -> None:
        if self.values.dtype != torch.float8_e4m3fn:
            raise ValueError(f"QuantizedTensor.values must be float8_e4m3fn, not {self.values.dtype}")
        if self.scale_exponent.dtype != torch.int8:
            raise ValueError(f"QuantizedTensor.scale_exponent holds int8 exponents, not {self.scale_exponent.dtype}")
        stored = self.values.shape[-1]
        if stored % BLOCK != 0 or stored < self.logical_shape[-1]:
            raise ValueError(f"{stored} stored channels cannot hold logical shape {self.logical_shape} in blocks of {BLOCK}")
        if self.scale_exponent.shape != (stored // BLOCK,):
            raise ValueError(f"{stored} channels need {stored // BLOCK} exponents, got shape {tuple(self.scale_exponent.shape)}")

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
        """The values as ``[rows, Cp]``."""
        return self.values.reshape(self.rows, self.channels)

    def dequantize(self, dtype: torch.dtype = torch.float32) -> Tensor:
        dense = _apply_block_scales(self.matrix(), self.scale_exponent)
        return dense[:, : self.logical_shape[-1]].reshape(self.logical_shape).to(dtype)


@dataclass(frozen=True)
class QuantizedWeight:
    """E4M3 ``[Np, Kp]`` (both padded to 32) with int8 exponents ``[Np, Kp / 32]``."""

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
        """Quantise a dense ``[N, K]`` matrix: zero-pad to multiples of 32, take each (row, 32 inputs) block's exponent
        from its largest magnitude, divide, saturate at +-448 and round to E4M3 (as flashim/quant/tensor.py:76-87)."""
        if weight.dim() != 2:
            raise ValueError(f"a weight matrix has two dimensions; got shape {tuple(weight.shape)}")
        if not bool(torch.isfinite(weight).all()):
            raise ValueError("the weight contains inf or nan and cannot be quantised")
        n, k = weight.shape
        stored = weight.new_zeros((padded_channels(n), padded_channels(k)), dtype=torch.float32)
        stored[:n, :k] = weight
        blocks = stored.unflatten(1, (-1, BLOCK))
        exponent = scale_exponent_from_amax(blocks.abs().amax(dim=2))
        scaled = (blocks / torch.exp2(exponent.float()).unsqueeze(-1)).clamp_(-FP8_MAX, FP8_MAX)
        return cls(scaled.flatten(1).to(torch.float8_e4m3fn), exponent, (n, k))

    @classmethod
    def from_conv(cls, weight: Tensor) -> "QuantizedWeight":
        """A conv weight ``[Cout, Cin, kh, kw]`` as the GEMM operand of the implicit-GEMM conv: taps outermost, channels
        innermost along K — ``(ky, kx, c)`` — with ``Cin`` zero-padded to 32 inside every tap
        (flashim/quant/methods/conv2d.py:193-205)."""
        cout, cin, kh, kw = weight.shape
        taps_last = weight.detach().new_zeros((cout, kh, kw, padded_channels(cin)))
        taps_last[..., :cin] = weight.detach().movedim(1, -1)
        return cls.from_float(taps_last.flatten(1))

    def swizzled_scales(self) -> Tensor:
        return swizzle_scales(self.scale_exponent)

    def dequantize(self, dtype: torch.dtype = torch.float32) -> Tensor:
        dense = _apply_block_scales(self.values, self.scale_exponent)
        return dense[: self.logical_shape[0], : self.logical_shape[1]].to(dtype)


@dataclass(frozen=True)
class Int8Tensor:
    """int8 values under one fp32 scale (``value = code * scale``)."""

    values: Tensor
    scale: Tensor

    def __post_init__(self) -> None:
        if self.values.dtype != torch.int8:
            raise ValueError(f"Int8Tensor.values must be int8, not {self.values.dtype}")
        if self.scale.dtype != torch.float32 or self.scale.numel() != 1:
            raise ValueError("Int8Tensor.scale is one float32 number")

    @property
    def logical_shape(self) -> tuple[int, ...]:
        return tuple(self.values.shape)

    def matrix(self) -> Tensor:
        return self.values.reshape(-1, self.values.shape[-1])

    def dequantize(self, dtype: torch.dtype = torch.float32) -> Tensor:
        return (self.values.float() * self.scale).to(dtype)


# ---- INT8 conv weights -----------------------------------------------------------------------------------------------


def safe_scale(scale: Tensor) -> Tensor:
    """Scales that are zero, negative, tiny or non-finite become fp32 epsilon, so a division by them stays finite."""
    scale = scale.float()
    floor = torch.finfo(torch.float32).eps
    usable = torch.isfinite(scale) & (scale > floor)
    return torch.where(usable, scale, scale.new_full((), floor))


def int8_weight_from_conv(weight: Tensor) -> tuple[Tensor, Tensor]:
    """A conv weight ``[Cout, Cin, kh, kw]`` -> int8 ``[Cout, kh * kw * Cin]`` in ``(ky, kx, c)`` order and one fp32
    scale per output channel, ``max|w| / 127`` (flashim/quant/methods/conv2d.py:91-100,
    flashim/quant/formats/int8.py:19-26)."""
    rows = weight.detach().movedim(1, -1).flatten(1).float()
    scale = safe_scale(rows.abs().amax(dim=1) / INT8_MAX)
    codes = torch.round(rows / scale.unsqueeze(1)).clamp_(-INT8_MAX, INT8_MAX)
    return codes.to(torch.int8).contiguous(), scale
