"""CPU restatement of FlashIM's torch reference for the quantized conv / depthwise path. TEST INFRASTRUCTURE ONLY:
the product (``flashim_b200``) never imports this file.

Every function names the reference source it follows as ``<file>:<lines>`` (paths inside the FlashIM project). The
reference expresses its oracle in CPU torch arithmetic, so this restatement does the same: the roundings that matter
(fp32 ``log2`` / ``ceil`` of the E8M0 rule, IEEE division before the INT8 rounding, the bf16 rounding points of the
epilogues) are then the same machine operations as the reference's.

Pinned by ``tests/test_oracle_golden.py`` against (1) the known-answer vectors of the reference's own tests and (2)
outputs of the reference implementation stored in ``tests/golden/*.npz``.

Functions whose name ends in ``_ext`` restate behaviour the reference does not have as one op (a GELU epilogue, per-row
activation scales, dynamic requantisation in the epilogue, fp32 / int32 outputs). They are compositions of the
reference's primitives with the rounding points written out below; their parity is pinned by this repository's tests only.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

E4M3_MAX = 448.0
MX_BLOCK = 32
INT8_LIMIT = 127.0
E4M3 = torch.float8_e4m3fn

__all__ = [
    "E4M3_MAX", "MX_BLOCK", "round_up32", "e8m0_exponent", "divide_by_block_scales", "static_block_exponent",
    "quantize_rows_dynamic", "e8m0_bytes", "swizzle_32_4_4", "unswizzle_32_4_4", "quantize_static_mx",
    "pack_mx_weight", "pack_mx_conv_weight", "floor_scale", "int8_weight_scales", "quantize_int8",
    "pack_int8_conv_weight", "gather_taps", "conv_out_size", "mx_matmul_fp32", "int8_matmul_int32",
    "mxfp8_conv2d", "int8_conv2d", "add_residual", "depthwise5x5_fp32", "depthwise5x5_relu_mxfp8",
    "depthwise5x5_relu_int8", "depthwise5x5_act_ext", "depthwise5x5_act_mxfp8_ext", "mxfp8_conv2d_ext",
    "int8_conv2d_accumulators_ext", "int8_conv2d_maxpool", "romav2_refiner_input", "romav2_refiner_heads", "mxfp8_scaled_mm", "int8_linear", "refiner_block_ext", "refiner_level_ext", "make_refiner_level_weights",
    "dequantize_mx", "mxfp8_linear", "gelu_quantize", "mxfp8_gelu_mlp", "depthwise5x5_relu_pointwise",
    "depthwise5x5_relu_pointwise_mxfp8", "depthwise5x5_relu_pointwise_int8",
]


# ---------------------------------------------------------------------------------------------------------------
# MX (E4M3 values, one E8M0 power-of-two scale per 32 elements)          flashim/quant/formats/mx.py
# ---------------------------------------------------------------------------------------------------------------


def round_up32(n: int) -> int:
    """Channel count padded to the MX block (flashim/quant/formats/mx.py:18-19)."""
    return -(-n // MX_BLOCK) * MX_BLOCK


def e8m0_exponent(amax: Tensor) -> Tensor:
    """Unbiased exponent ``e`` of the block scale ``2**e``: fp32 ``ceil(log2(amax / 448))``, ``-127`` for an all-zero
    block, clamped to ``[-127, 127]``, int8 (flashim/quant/formats/mx.py:22-26). The fp32 ``log2`` makes a block whose
    amax sits a few ulp above ``448 * 2**k`` keep exponent ``k``; that behaviour is part of the contract."""
    e = torch.ceil(torch.log2(amax / E4M3_MAX))
    e = torch.where(amax == 0, torch.full_like(e, -127.0), e)
    return e.clamp(-127, 127).to(torch.int8)


def divide_by_block_scales(blocks: Tensor, exponent: Tensor) -> Tensor:
    """``[..., groups, 32]`` blocks divided by ``2**exponent`` and saturated to +-448, fp32
    (flashim/quant/formats/mx.py:29-38). ``exponent`` is ``[groups]`` (shared by all rows) or ``[rows, groups]``."""
    scale = torch.exp2(exponent.float())
    if exponent.ndim == 1:
        scale = scale[None, :, None]
    elif exponent.ndim == 2:
        scale = scale[..., None]
    else:
        raise ValueError(f"scale rank {exponent.ndim} is not supported")
    return (blocks / scale).clamp(-E4M3_MAX, E4M3_MAX)


def static_block_exponent(value: Tensor) -> Tensor:
    """One exponent per padded 32-channel block from the amax over every row
    (flashim/quant/formats/mx.py:41-47)."""
    cp = round_up32(value.shape[-1])
    blocks = F.pad(value.float(), (0, cp - value.shape[-1])).reshape(-1, cp // MX_BLOCK, MX_BLOCK)
    return e8m0_exponent(blocks.abs().amax(dim=(0, 2)))


def quantize_rows_dynamic(matrix: Tensor) -> tuple[Tensor, Tensor]:
    """Per-(row, 32-block) dynamic MXFP8 of ``[rows, K]``: E4M3 ``[rows, K]`` and int8 exponents ``[rows, K/32]``
    (flashim/quant/formats/mx.py:50-60). Note the multiply by ``2**-e`` (not a division)."""
    rows, k = matrix.shape
    if k % MX_BLOCK:
        raise ValueError(f"K={k} is not a multiple of 32")
    blocks = matrix.float().contiguous().reshape(rows, k // MX_BLOCK, MX_BLOCK)
    e = e8m0_exponent(blocks.abs().amax(dim=-1))
    q = (blocks * torch.exp2(-e.float())[..., None]).clamp(-E4M3_MAX, E4M3_MAX)
    return q.to(E4M3).reshape(rows, k), e


def e8m0_bytes(exponent: Tensor) -> Tensor:
    """Biased E8M0 byte ``e + 127`` as uint8 (flashim/quant/formats/mx.py:63-64)."""
    return (exponent.to(torch.int16) + 127).to(torch.uint8)


def swizzle_32_4_4(exponent: Tensor) -> Tensor:
    """``[rows, groups]`` int8 exponents -> flat uint8 E8M0 bytes in 128-row x 4-group tiles of 512 bytes, rows padded to
    128 and groups to 4 with zero bytes; byte offset of ``(r, g)`` is
    ``((r // 128) * tiles + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4``
    (flashim/quant/formats/mx.py:67-86)."""
    raw = e8m0_bytes(exponent)
    rows, groups = raw.shape
    pr, pg = -(-rows // 128) * 128, -(-groups // 4) * 4
    padded = torch.zeros((pr, pg), dtype=torch.uint8)
    padded[:rows, :groups] = raw
    return padded.view(pr // 128, 4, 32, pg // 4, 4).permute(0, 3, 2, 1, 4).reshape(-1).contiguous()


def unswizzle_32_4_4(flat: Tensor, rows: int, groups: int) -> Tensor:
    """Inverse of :func:`swizzle_32_4_4`: int8 exponents ``[rows, groups]`` (flashim/ops/gemm.py:21-37)."""
    pr, pg = -(-rows // 128) * 128, -(-groups // 4) * 4
    tiles = flat.view(torch.uint8).reshape(pr // 128, pg // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(pr, pg)
    return (tiles[:rows, :groups].to(torch.int16) - 127).to(torch.int8)


def quantize_static_mx(value: Tensor, exponent: Tensor) -> Tensor:
    """Static block-32 quantisation of ``[..., C]`` with a shared int8 ``[Cp/32]`` exponent vector: channels zero-padded
    to ``Cp``, ``x / 2**e``, saturate, round to nearest even E4M3 ``[..., Cp]`` (flashim/quant/tensor.py:97-121)."""
    cp = round_up32(value.shape[-1])
    if tuple(exponent.shape) != (cp // MX_BLOCK,):
        raise ValueError(f"expected {(cp // MX_BLOCK,)} exponents, got {tuple(exponent.shape)}")
    dense = value.contiguous().float()
    if cp != value.shape[-1]:
        dense = F.pad(dense, (0, cp - value.shape[-1]))
    q = divide_by_block_scales(dense.reshape(-1, cp // MX_BLOCK, MX_BLOCK), exponent.to(torch.int8))
    return q.reshape(*value.shape[:-1], cp).to(E4M3)


def pack_mx_weight(weight: Tensor) -> tuple[Tensor, Tensor]:
    """``[N, K]`` float weight -> E4M3 ``[Np, Kp]`` (both padded to 32) and int8 exponents ``[Np, Kp/32]``, one per
    (row, 32 inputs) (flashim/quant/tensor.py:76-87)."""
    n, k = weight.shape
    np_, kp = round_up32(n), round_up32(k)
    padded = F.pad(weight.float(), (0, kp - k, 0, np_ - n))
    blocks = padded.reshape(np_, kp // MX_BLOCK, MX_BLOCK)
    e = e8m0_exponent(blocks.abs().amax(dim=-1))
    return divide_by_block_scales(blocks, e).reshape(np_, kp).to(E4M3), e


def pack_mx_conv_weight(weight: Tensor) -> tuple[Tensor, Tensor]:
    """``[Cout, Cin, kh, kw]`` -> K order ``(ky, kx, c)`` with ``Cin`` padded to 32 per tap, then :func:`pack_mx_weight`
    (flashim/quant/methods/conv2d.py:193-205)."""
    cout, cin = weight.shape[:2]
    w = F.pad(weight.permute(0, 2, 3, 1), (0, round_up32(cin) - cin))
    return pack_mx_weight(w.reshape(cout, -1))


def dequantize_mx(values: Tensor, exponent: Tensor) -> Tensor:
    """fp32 ``values * 2**exponent`` with ``exponent`` ``[K/32]`` (shared) or ``[rows, K/32]``
    (flashim/quant/tensor.py:52-55,89-94)."""
    rows = values.reshape(-1, values.shape[-1])
    scale = torch.exp2(exponent.float()).repeat_interleave(MX_BLOCK, dim=-1)
    return (rows.float() * scale).reshape(values.shape)


# ---------------------------------------------------------------------------------------------------------------
# symmetric INT8                                                        flashim/quant/formats/int8.py
# ---------------------------------------------------------------------------------------------------------------

_EPS = torch.finfo(torch.float32).eps


def floor_scale(scale: Tensor) -> Tensor:
    """Non-finite or vanishing scales become fp32 eps (flashim/quant/formats/int8.py:13-16)."""
    scale = scale.float()
    return torch.where(torch.isfinite(scale) & (scale > _EPS), scale, torch.full_like(scale, _EPS))


def int8_weight_scales(weight: Tensor) -> Tensor:
    """Per-output-row ``amax / 127`` (flashim/quant/formats/int8.py:19-21)."""
    return floor_scale(weight.float().abs().amax(dim=1) / INT8_LIMIT)


def quantize_int8(value: Tensor, scale: Tensor) -> Tensor:
    """``round_half_even(value / scale)`` saturated to +-127, int8, in fp32 arithmetic with a true division
    (flashim/quant/formats/int8.py:24-26; flashim/quant/tensor.py:148-151)."""
    return (value.float() / scale).round().clamp(-INT8_LIMIT, INT8_LIMIT).to(torch.int8).contiguous()


def pack_int8_conv_weight(weight: Tensor) -> tuple[Tensor, Tensor]:
    """``[Cout, Cin, kh, kw]`` -> int8 ``[Cout, kh*kw*Cin]`` in ``(ky, kx, c)`` order and fp32 ``[Cout]`` scales
    (flashim/quant/methods/conv2d.py:91-100)."""
    w = weight.permute(0, 2, 3, 1).reshape(weight.shape[0], -1)
    s = int8_weight_scales(w)
    return quantize_int8(w, s[:, None]), s


# ---------------------------------------------------------------------------------------------------------------
# implicit-GEMM conv oracles                                            flashim/ops/conv.py, flashim/ops/gemm.py
# ---------------------------------------------------------------------------------------------------------------


def conv_out_size(size: int, k: int, s: int, p: int, d: int) -> int:
    return (size + 2 * p - d * (k - 1) - 1) // s + 1


def gather_taps(x: Tensor, kh, kw, sh, sw, ph, pw, dh, dw) -> Tensor:
    """Byte im2col: ``[B, H, W, C]`` of a 1-byte dtype -> ``[B*Ho*Wo, kh*kw*C]`` in ``(ky, kx, c)`` order, zero bytes
    for the padding (flashim/ops/conv.py:144-165)."""
    b, h, w, c = x.shape
    raw = x.view(torch.uint8)
    if ph or pw:
        raw = F.pad(raw, (0, 0, pw, pw, ph, ph))
    ho, wo = conv_out_size(h, kh, sh, ph, dh), conv_out_size(w, kw, sw, pw, dw)
    cols = [
        raw[:, ky * dh: ky * dh + (ho - 1) * sh + 1: sh, kx * dw: kx * dw + (wo - 1) * sw + 1: sw]
        for ky in range(kh) for kx in range(kw)
    ]
    out = cols[0] if len(cols) == 1 else torch.cat(cols, dim=-1)
    return out.reshape(b * ho * wo, -1).view(x.dtype)


def mx_matmul_fp32(a: Tensor, a_exp: Tensor, w: Tensor, w_exp: Tensor) -> Tensor:
    """fp32 ``deq(a) @ deq(w)^T`` of E4M3 ``a [M, K]`` (exponents ``[K/32]`` shared or ``[M, K/32]``) and ``w [N, K]``
    (exponents ``[N, K/32]``) (flashim/ops/gemm.py:58-66)."""
    return dequantize_mx(a, a_exp) @ dequantize_mx(w, w_exp).t()


def int8_matmul_int32(a: Tensor, w: Tensor) -> Tensor:
    """Exact ``a [M, K] @ w [N, K]^T`` in integers, returned as int32. The reference does the product in int64
    (flashim/ops/gemm.py:87); a float64 matmul is exact for the same operands (|sum| < 2**53) and uses BLAS."""
    acc = a.double() @ w.double().t()
    return acc.to(torch.int64).to(torch.int32)


def add_residual(out: Tensor, residual: Tensor, relu: bool) -> Tensor:
    """``relu(out + residual)`` in fp32 -> bf16; ``residual`` may carry fewer channels
    (flashim/ops/conv.py:198-203)."""
    c = residual.shape[-1]
    s = out.float().clone()
    s[..., :c] += residual.float()
    return (s.relu() if relu else s).to(torch.bfloat16)


def mxfp8_conv2d(x, channel_exponent, weight, weight_exponent, bias, kh, kw, sh, sw, ph, pw, dh, dw, *,
                 relu=False, residual=None, out_exponent=None) -> Tensor:
    """Static block-scaled MXFP8 conv: E4M3 NHWC ``x`` with ``[Cin/32]`` exponents shared by every pixel and tap, E4M3
    weight ``[Cout, kh*kw*Cin]`` with ``[Cout, kh*kw*Cin/32]`` exponents -> bf16 ``[B, Ho, Wo, Cout]``: fp32 product,
    ``+ bias``, one bf16 rounding, then residual / ReLU, then optionally the static requantisation of that bf16 tensor
    (flashim/ops/conv.py:309-339, flashim/ops/gemm.py:58-69)."""
    b, h, w, _ = x.shape
    ho, wo = conv_out_size(h, kh, sh, ph, dh), conv_out_size(w, kw, sw, pw, dw)
    cols = gather_taps(x, kh, kw, sh, sw, ph, pw, dh, dw)
    out = mx_matmul_fp32(cols, channel_exponent.repeat(kh * kw), weight, weight_exponent)
    if bias is not None:
        out = out + bias.float()
    out = out.to(torch.bfloat16).reshape(b, ho, wo, -1)
    if residual is not None:
        out = add_residual(out, residual, relu)
    elif relu:
        out = F.relu(out)
    return out if out_exponent is None else quantize_static_mx(out, out_exponent)


def int8_conv2d(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, *,
                relu=False, residual=None, out_scale=None) -> Tensor:
    """INT8 conv: exact int32 sums, ``float(acc) * (a_scale * w_scale[n])`` then ``+ bias`` (two fp32 roundings),
    ReLU, one bf16 rounding, residual, optional static INT8 requantisation
    (flashim/ops/conv.py:174-195, flashim/ops/gemm.py:82-98)."""
    b, h, w, _ = x.shape
    ho, wo = conv_out_size(h, kh, sh, ph, dh), conv_out_size(w, kw, sw, pw, dw)
    acc = int8_matmul_int32(gather_taps(x, kh, kw, sh, sw, ph, pw, dh, dw), weight)
    out = acc.float() * (a_scale.float() * w_scale.float())
    if bias is not None:
        out = out + bias.float()
    if relu and residual is None:
        out = out.relu()
    out = out.to(torch.bfloat16).reshape(b, ho, wo, -1)
    if residual is not None:
        out = add_residual(out, residual, relu)
    return out if out_scale is None else quantize_int8(out, out_scale.float().reshape(()))


def int8_conv2d_maxpool(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu=False, out_scale):
    """:func:`int8_conv2d` (bf16 output) and its ``MaxPool2d(2)`` quantised with ``out_scale``: ``(out, pooled int8
    [B, Ho // 2, Wo // 2, Cout])``; a trailing odd row / column is dropped (flashim/ops/conv.py:209-222)."""
    out = int8_conv2d(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, relu=relu)
    pooled = F.max_pool2d(out.permute(0, 3, 1, 2).float(), 2).permute(0, 2, 3, 1).to(torch.bfloat16)
    return out, quantize_int8(pooled, out_scale.float().reshape(()))


def romav2_refiner_input(f_a, f_b, warp, emb_weight, emb_bias, scale_factor, radius, pair=0):
    """RoMaV2 refiner input, bf16 channels-last ``[B, 2P + E + K, h, w]`` from fp32 ``f_a`` / ``f_b [B, h, w, P]`` and
    ``warp [B, h, w, 2]``: ``f_a``; ``f_b`` sampled at the warp (bilinear, zeros padding, ``align_corners=False``); the 1x1
    conv ``[E, 2]`` of ``scale_factor * (warp - identity grid)``; and, for ``radius >= 0``, the dot products of
    ``f_a / sqrt(P)`` with ``f_b`` sampled on the ``(2r+1)^2`` window of one-pixel steps around the warp, ``k = ky (2r+1) +
    kx``. ``pair > 0``: image ``i`` of ``f_a`` is matched with image ``(i + pair) % (2 pair)`` of ``f_a``
    (flashim/ops/romav2.py:36-66, flashim/ops/correlation.py:13-39)."""
    if pair > 0:
        f_b = torch.roll(f_a, shifts=pair, dims=0)
    b, h, w, p = f_a.shape
    a, other = f_a.permute(0, 3, 1, 2), f_b.permute(0, 3, 1, 2)
    sample = lambda grid: F.grid_sample(other, grid, mode="bilinear", padding_mode="zeros", align_corners=False)  # noqa: E731
    gy, gx = torch.meshgrid(torch.linspace(-1 + 1 / h, 1 - 1 / h, h), torch.linspace(-1 + 1 / w, 1 - 1 / w, w), indexing="ij")
    displacement = (warp - torch.stack((gx, gy), dim=-1)).permute(0, 3, 1, 2)
    embedding = F.conv2d(scale_factor[None, :, None, None] * displacement, emb_weight.reshape(-1, 2, 1, 1), emb_bias)
    parts = [a, sample(warp), embedding]
    if radius >= 0:
        steps = 2 * radius + 1
        oy, ox = torch.meshgrid(torch.linspace(-2 * radius / h, 2 * radius / h, steps),
                                torch.linspace(-2 * radius / w, 2 * radius / w, steps), indexing="ij")
        offsets = torch.stack((ox, oy), dim=-1).reshape(-1, 2)                       # [K, 2], x first
        coords = (warp[:, :, :, None, :] + offsets).reshape(b, h, w * steps * steps, 2)
        sampled = sample(coords).reshape(b, p, h, w, steps * steps)
        parts.append(((a[..., None] / p**0.5) * sampled).sum(dim=1).permute(0, 3, 1, 2))
    return torch.cat(parts, dim=1).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)


def romav2_refiner_heads(z, weight, bias, prev_warp, prev_confidence, refine_init):
    """RoMaV2 refiner heads: fp32 1x1 conv of ``z [B, C, h, w]`` to 2 displacement + 4 precision channels,
    ``warp = prev_warp + disp / (refine_init * (w, h))``, ``l00 = softplus(d1) + 1e-6``, ``l10 = d2``,
    ``l11 = softplus(d3) + 1e-6``, ``confidence = prev_confidence (zero-padded to 4) + (d0, l00^2, l00 l10, l10^2 + l11^2)``;
    fp32 ``[B, h, w, 2]`` and ``[B, h, w, 4]`` (flashim/ops/romav2.py:95-120)."""
    _, _, h, w = z.shape
    out = F.conv2d(z.float(), weight.float().reshape(6, -1)[:, :, None, None], bias.float()).permute(0, 2, 3, 1)
    warp = prev_warp + out[..., :2] / (refine_init * torch.tensor([w, h], dtype=prev_warp.dtype))
    d = out[..., 2:]
    l00, l10, l11 = F.softplus(d[..., 1]) + 1e-6, d[..., 2], F.softplus(d[..., 3]) + 1e-6
    delta = torch.stack([d[..., 0], l00 * l00, l00 * l10, l10 * l10 + l11 * l11], dim=-1)
    previous = prev_confidence if prev_confidence.shape[-1] == 4 else F.pad(prev_confidence, (0, 3))
    return warp, previous + delta


def mxfp8_scaled_mm(a: Tensor, b_t: Tensor, a_scale: Tensor, b_scale: Tensor, bias: Tensor | None = None) -> Tensor:
    """Block-scaled MXFP8 GEMM ``a [M, K] x b_t [K, N]`` with swizzled E8M0 scales of both operands (rows of ``a``, rows
    of ``b_t.t()``), fp32 product, ``+ bias`` in fp32, one bf16 rounding (flashim/ops/gemm.py:21-52)."""
    def dense(values: Tensor, swizzled: Tensor) -> Tensor:
        rows, k = values.shape
        exponent = unswizzle_32_4_4(swizzled.view(torch.uint8), rows, k // MX_BLOCK).float()
        return (values.float().reshape(rows, k // MX_BLOCK, MX_BLOCK) * torch.exp2(exponent)[..., None]).reshape(rows, k)

    out = dense(a, a_scale) @ dense(b_t.t(), b_scale).t()
    if bias is not None:
        out = out + bias.float()
    return out.to(torch.bfloat16)


def int8_linear(a, weight, a_scale, w_scale, bias, *, relu=False, gelu=False, residual=None) -> Tensor:
    """``[M, K] int8 x [N, K] int8^T`` in int32, ``float(acc) * (a_scale * w_scale) + bias``, ReLU, one bf16 rounding,
    GELU of the bf16 value (rounded to bf16), residual added in bf16 (flashim/ops/gemm.py:82-98)."""
    out = int8_matmul_int32(a, weight).float() * (a_scale.float() * w_scale.float())
    if bias is not None:
        out = out + bias.float()
    if relu:
        out = out.relu()
    out = out.to(torch.bfloat16)
    if gelu:
        out = F.gelu(out)
    if residual is not None:
        out = residual + out
    return out


def mxfp8_linear(values: Tensor, scale_exponent: Tensor, bias: Tensor | None, weight: Tensor, weight_exponent: Tensor) -> Tensor:
    """Static MXFP8 linear: E4M3 ``values [rows, K]`` under the shared exponents ``[K/32]``, E4M3 ``weight [N, K]`` under
    ``[N, K/32]`` exponents; fp32 product, ``+ bias`` in fp32, one bf16 rounding (flashim/ops/gemm.py:58-69)."""
    out = mx_matmul_fp32(values, scale_exponent, weight, weight_exponent)
    if bias is not None:
        out = out + bias.float()
    return out.to(torch.bfloat16)


def gelu_quantize(value: Tensor, scale_exponent: Tensor, *, input_bias: Tensor | None = None) -> Tensor:
    """``quantize_static(GELU(value [+ input_bias]))``, erf form: in fp32 when a bias is fused, else in ``value``'s dtype;
    rounded to ``value``'s dtype before the static block-32 quantiser (flashim/ops/quantize.py:62-71)."""
    if input_bias is not None:
        activated = F.gelu(value.float() + input_bias.float()).to(value.dtype)
    else:
        activated = F.gelu(value)
    return quantize_static_mx(activated, scale_exponent)


def mxfp8_gelu_mlp(values, scale_exponent, w1, w1_exponent, b1, hidden_exponent, w2, w2_exponent) -> Tensor:
    """``linear(quantize_static(GELU(linear(x, W1) [bf16] + b1) [bf16], hidden_exponent), W2)`` -> bf16; neither linear adds
    a bias of its own (flashim/ops/gemm.py:146-154)."""
    hidden = mxfp8_linear(values, scale_exponent, None, w1, w1_exponent)
    return mxfp8_linear(gelu_quantize(hidden, hidden_exponent, input_bias=b1), hidden_exponent, None, w2, w2_exponent)


def depthwise5x5_relu_pointwise(value, dw_weight, dw_bias, pw_weight, pw_bias) -> Tensor:
    """bf16 refiner block: depthwise 5x5 + bias + ReLU in fp32, one bf16 rounding, pointwise ``[Cout, Cin]`` product in
    fp32 plus bias, one bf16 rounding; NHWC ``[B, H, W, Cout]`` (the memory of the reference's channels-last result,
    flashim/ops/conv.py:67-84)."""
    hidden = F.relu(depthwise5x5_fp32(value, dw_weight, dw_bias)).to(torch.bfloat16).float()
    out = F.conv2d(hidden, pw_weight.float()[:, :, None, None], pw_bias.float())
    return out.to(torch.bfloat16).permute(0, 2, 3, 1).contiguous()


def depthwise5x5_relu_pointwise_mxfp8(value, dw_weight, dw_bias, pw_weight, pw_scale_swizzled, pw_bias) -> Tensor:
    """:func:`depthwise5x5_relu_mxfp8` then :func:`mxfp8_scaled_mm` with the pointwise weight ``[N, K]``; NHWC
    ``[B, H, W, N]`` (flashim/ops/conv.py:93-110)."""
    b, _, h, w = value.shape
    q, scale = depthwise5x5_relu_mxfp8(value, dw_weight, dw_bias)
    return mxfp8_scaled_mm(q, pw_weight.t(), scale, pw_scale_swizzled, pw_bias).reshape(b, h, w, -1)


def depthwise5x5_relu_pointwise_int8(value, dw_weight, dw_bias, pw_weight, pw_wscale, pw_bias, scale) -> Tensor:
    """:func:`depthwise5x5_relu_int8` then :func:`int8_linear`; NHWC ``[B, H, W, N]`` (flashim/ops/conv.py:119-135)."""
    b, _, h, w = value.shape
    q = depthwise5x5_relu_int8(value, dw_weight, dw_bias, scale)
    return int8_linear(q, pw_weight, scale, pw_wscale, pw_bias).reshape(b, h, w, -1)


def int8_conv2d_accumulators_ext(x, weight, kh, kw, sh, sw, ph, pw, dh, dw) -> Tensor:
    """The raw int32 sums ``[B, Ho, Wo, Cout]`` of :func:`int8_conv2d` before any scaling (extension: the reference keeps
    them internal, flashim/ops/gemm.py:87)."""
    b, h, w, _ = x.shape
    ho, wo = conv_out_size(h, kh, sh, ph, dh), conv_out_size(w, kw, sw, pw, dw)
    return int8_matmul_int32(gather_taps(x, kh, kw, sh, sw, ph, pw, dh, dw), weight).reshape(b, ho, wo, -1)


def mxfp8_conv2d_ext(x, act_exponent, weight, weight_exponent, bias, kh, kw, sh, sw, ph, pw, dh, dw, *,
                     act="none", residual=None, out_exponent=None, dynamic_out=False, out_fp32=False):
    """:func:`mxfp8_conv2d` with the extensions the B200 epilogue offers. Rounding points, in order:

    1. fp32 product (activation exponents ``[Cin/32]`` static, or ``[B*H*W, Cin/32]`` per pixel for a 1x1 conv fed by a
       dynamic producer), ``+ bias`` in fp32; ``out_fp32`` returns this.
    2. one bf16 rounding.
    3. ``act``: ``"relu"`` or ``"gelu"`` (erf form evaluated in fp32 on the bf16 value, rounded to bf16 again: the
       ``gelu=True`` convention of flashim/ops/gemm.py:82-98).
    4. ``residual`` added in fp32 to the bf16 value, one more bf16 rounding (flashim/ops/conv.py:198-203); with
       ``act="relu"`` the ReLU moves after the sum as in the reference.
    5. ``out_exponent``: static requantisation (:func:`quantize_static_mx`), returns E4M3; or ``dynamic_out``: per
       (pixel, 32 channels) dynamic requantisation (:func:`quantize_rows_dynamic`), returns ``(E4M3, int8 exponents
       [B*Ho*Wo, Cout/32])``.
    """
    b, h, w, cin = x.shape
    ho, wo = conv_out_size(h, kh, sh, ph, dh), conv_out_size(w, kw, sw, pw, dw)
    cols = gather_taps(x, kh, kw, sh, sw, ph, pw, dh, dw)
    if act_exponent.ndim == 2:
        if (kh, kw, sh, sw, ph, pw) != (1, 1, 1, 1, 0, 0):
            raise ValueError("per-pixel activation scales need a 1x1 conv")
        a_exp = act_exponent
    else:
        a_exp = act_exponent.repeat(kh * kw)
    out = mx_matmul_fp32(cols, a_exp, weight, weight_exponent)
    if bias is not None:
        out = out + bias.float()
    out = out.reshape(b, ho, wo, -1)
    if out_fp32:
        return out
    out = out.to(torch.bfloat16)
    if act == "gelu":
        out = F.gelu(out.float()).to(torch.bfloat16)
    if residual is not None:
        out = add_residual(out, residual, act == "relu")
    elif act == "relu":
        out = F.relu(out)
    if out_exponent is not None:
        return quantize_static_mx(out, out_exponent)
    if dynamic_out:
        q, e = quantize_rows_dynamic(out.reshape(-1, out.shape[-1]))
        return q.reshape(out.shape), e
    return out


# ---------------------------------------------------------------------------------------------------------------
# depthwise 5x5                                                         flashim/ops/conv.py:30-61
# ---------------------------------------------------------------------------------------------------------------


def depthwise5x5_fp32(value: Tensor, weight: Tensor, bias: Tensor) -> Tensor:
    """fp32 depthwise 5x5 (pad 2) of the bf16-rounded ``value [B, C, H, W]`` with the packed bf16 ``weight [25, C]``
    (tap-major: ``ky * 5 + kx``) plus fp32 ``bias [C]`` -> fp32 ``[B, C, H, W]`` (flashim/ops/conv.py:36-39)."""
    c = value.shape[1]
    kernel = weight.float().t().reshape(c, 1, 5, 5)
    return F.conv2d(value.to(torch.bfloat16).float(), kernel, bias.float(), padding=2, groups=c)


def depthwise5x5_relu_mxfp8(value, weight, bias) -> tuple[Tensor, Tensor]:
    """Depthwise + bias + ReLU, the fp32 result quantised per (pixel, 32 channels) without an intermediate bf16
    rounding: E4M3 ``[B*H*W, C]`` and the swizzled E8M0 bytes (flashim/ops/conv.py:30-41)."""
    c = value.shape[1]
    out = F.relu(depthwise5x5_fp32(value, weight, bias))
    q, e = quantize_rows_dynamic(out.permute(0, 2, 3, 1).reshape(-1, c))
    return q, swizzle_32_4_4(e)


def depthwise5x5_relu_int8(value, weight, bias, scale) -> Tensor:
    """Depthwise + bias + ReLU rounded to bf16, then static INT8 ``[B*H*W, C]`` (flashim/ops/conv.py:50-58)."""
    c = value.shape[1]
    out = F.relu(depthwise5x5_fp32(value, weight, bias)).to(torch.bfloat16)
    return quantize_int8(out.permute(0, 2, 3, 1).reshape(-1, c), scale)


def _activate(x: Tensor, act: str) -> Tensor:
    if act == "relu":
        return F.relu(x)
    if act == "gelu":
        return F.gelu(x)
    if act == "none":
        return x
    raise ValueError(f"unknown activation {act!r}")


def depthwise5x5_act_ext(value, weight, bias, act="gelu") -> Tensor:
    """Depthwise + bias + activation (in fp32) -> one bf16 rounding, NHWC ``[B, H, W, C]``. Extension: the reference's
    depthwise ops end in a quantiser; the conv and its operand layout are those of flashim/ops/conv.py:30-41."""
    return _activate(depthwise5x5_fp32(value, weight, bias), act).to(torch.bfloat16).permute(0, 2, 3, 1).contiguous()


def depthwise5x5_act_mxfp8_ext(value, weight, bias, act="gelu") -> tuple[Tensor, Tensor]:
    """:func:`depthwise5x5_relu_mxfp8` with a selectable activation; returns E4M3 ``[B*H*W, C]`` and the *plain* int8
    exponents ``[B*H*W, C/32]`` (swizzle with :func:`swizzle_32_4_4`)."""
    c = value.shape[1]
    out = _activate(depthwise5x5_fp32(value, weight, bias), act)
    return quantize_rows_dynamic(out.permute(0, 2, 3, 1).reshape(-1, c))


# ---------------------------------------------------------------------------------------------------------------
# synthetic refiner stack (the benchmark's stack workload); block structure after flashim/models/romav2/refiner.py:45-148 and
# flashim/quant/passes/separable_conv_block.py:69-110, widened to the C -> 2C -> C residual MLP the benchmark names.
# ---------------------------------------------------------------------------------------------------------------


def make_refiner_level_weights(channels: int, blocks: int, generator: torch.Generator) -> dict:
    """Random-init weights of one pyramid level: ``proj`` 1x1 C->C, ``blocks`` x (depthwise 5x5, 1x1 C->2C, 1x1 2C->C),
    ``head`` 1x1 C->4 (padded to 32 outputs by the MX weight packing). Kaiming-normal convs, biases ~ N(0, 0.02)."""

    def conv(cout, cin):
        w = torch.empty(cout, cin, 1, 1)
        torch.nn.init.kaiming_normal_(w, generator=generator)
        q, e = pack_mx_conv_weight(w)
        return {"w": q, "e": e, "b": (torch.randn(round_up32(cout), generator=generator) * 0.02).to(torch.bfloat16),
                "cout": cout}

    level = {"channels": channels, "proj": conv(channels, channels), "head": conv(4, channels), "blocks": []}
    for _ in range(blocks):
        level["blocks"].append({
            "dw_w": (torch.randn(25, channels, generator=generator) * 0.05).to(torch.bfloat16),
            "dw_b": torch.randn(channels, generator=generator) * 0.02,
            "up": conv(2 * channels, channels),
            "down": conv(channels, 2 * channels),
        })
    return level


def _pointwise(q, e, layer, **kw):
    return mxfp8_conv2d_ext(q, e, layer["w"], layer["e"], layer["b"], 1, 1, 1, 1, 0, 0, 1, 1, **kw)


def refiner_block_ext(x: Tensor, block: dict) -> Tensor:
    """One refiner block on bf16 NHWC ``x``: depthwise 5x5 + bias + GELU -> dynamic MXFP8 -> 1x1 C->2C + bias + GELU ->
    dynamic MXFP8 -> 1x1 2C->C + bias + residual ``x`` -> bf16 NHWC."""
    b, h, w, c = x.shape
    q, e = depthwise5x5_act_mxfp8_ext(x.permute(0, 3, 1, 2), block["dw_w"], block["dw_b"], "gelu")
    hq, he = _pointwise(q.reshape(b, h, w, c), e, block["up"], act="gelu", dynamic_out=True)
    return _pointwise(hq, he, block["down"], residual=x)


def refiner_level_ext(x: Tensor, level: dict) -> Tensor:
    """One pyramid level: dynamic MXFP8 of the bf16 input -> ``proj`` -> blocks -> dynamic MXFP8 -> ``head``; returns the
    bf16 ``[B, H, W, 32]`` head output whose first 4 channels are warp (2) + confidence (2)."""
    b, h, w, c = x.shape
    q, e = quantize_rows_dynamic(x.reshape(-1, c))
    y = _pointwise(q.reshape(b, h, w, c), e, level["proj"])
    for block in level["blocks"]:
        y = refiner_block_ext(y, block)
    q, e = quantize_rows_dynamic(y.reshape(-1, c))
    return _pointwise(q.reshape(b, h, w, c), e, level["head"])


def _self_check() -> None:  # pragma: no cover - convenience for ``python -m oracle.flashim_oracle``
    amax = torch.tensor([0.0, 448.0, 449.0, 1.0, 1e-30])
    assert e8m0_exponent(amax).tolist() == [-127, 0, 1, -8, -108]
    assert quantize_int8(torch.tensor([0.5, 1.5, 2.5, -0.5, 1000.0, -1000.0, 0.0]), torch.tensor(1.0)).tolist() == [
        0, 2, 2, 0, 127, -127, 0]
    e = torch.randint(-20, 10, (300, 7), dtype=torch.int8)
    assert torch.equal(unswizzle_32_4_4(swizzle_32_4_4(e), 300, 7), e)
    print("oracle self-check ok", math.pi > 3)


if __name__ == "__main__":
    _self_check()
