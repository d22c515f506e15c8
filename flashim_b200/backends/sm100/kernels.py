"""The sm_100a CUDA backend: ``torch.library`` custom ops around the C ABI of ``libflashim_sm100.so`` and their
registration into the op registry (the role flashim/backends/cuda/conv.py plays for FlashIM's JIT CUDA kernels: ctypes
launch on torch's current stream, non-zero return code -> ``RuntimeError``, fake implementations for tracing).

Implementations are registered as ``"sm100"`` for compute capability 10.0 only and require ``Feature.TCGEN05`` and
``Feature.SM100A_KERNELS``; :func:`register` takes the registry to register into, so the same code can register into
FlashIM's own ``flashim.ops`` (see ``flashim_b200.integration``).
"""

from __future__ import annotations

import ctypes
import os
from collections import OrderedDict

import torch
from torch import Tensor

from flashim_b200 import _native
from flashim_b200.quant.tensor import (
    BLOCK, Int8Tensor, QuantizedTensor, padded_channels, swizzle_scales, swizzled_scale_bytes,
)

E4M3 = torch.float8_e4m3fn
_IN_DTYPES = {torch.float32: _native.DTYPE_F32, torch.bfloat16: _native.DTYPE_BF16}
_CHECK_EVERY_CALL = os.environ.get("FLASHIM_B200_CHECK", "0") == "1"

# ---- status word --------------------------------------------------------------------------------------------------------
_STATUS: dict[int, Tensor] = {}


def status_word(device: torch.device) -> Tensor:
    """The per-device int32 word the kernels' bounded waits report to (zero while everything is healthy)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _STATUS.get(index)
    if word is None:
        word = _STATUS[index] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
    return word


def check_status(device: torch.device | str | None = None) -> None:
    """Synchronise and raise if a kernel on ``device`` abandoned work because one of its waits ran out."""
    device = torch.device(device if device is not None else "cuda")
    word = status_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        raise RuntimeError(f"sm100 kernel gave up waiting: {_native.STATUS.get(code, hex(code))}; outputs are invalid")


def _swizzled_scale_buffer(rows: int, groups: int, device) -> Tensor:
    """Byte buffer of the swizzled E8M0 layout. Its padding (rows up to a multiple of 128, groups up to a multiple of 4) is
    zero like the reference's ``swizzle_scales``; a kernel writes every other byte, so a buffer without padding needs no
    fill."""
    size = swizzled_scale_bytes(rows, groups)
    if rows % 128 == 0 and groups % 4 == 0:
        return torch.empty(size, device=device, dtype=torch.uint8)
    return torch.zeros(size, device=device, dtype=torch.uint8)


def _stream(t: Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _finish(code: int, what: str, device: torch.device) -> None:
    _native.check(code, what)
    if _CHECK_EVERY_CALL and not torch.cuda.is_current_stream_capturing():
        check_status(device)


def _nhwc(value: Tensor) -> Tensor:
    """``[B, C, H, W]`` -> its bf16 ``[B, H, W, C]`` memory (zero-copy for channels-last bf16 input)."""
    if value.dtype != torch.bfloat16:
        value = value.to(torch.bfloat16)
    pixels = value.permute(0, 2, 3, 1)
    if not pixels.is_contiguous() or pixels.data_ptr() % 16:
        pixels = pixels.contiguous() if not pixels.is_contiguous() else pixels.clone()
    return pixels


# ---- custom ops: depthwise -------------------------------------------------------------------------------------------


@torch.library.custom_op("flashim_b200::dw5x5_bf16", mutates_args=())
def dw5x5_bf16(pixels: Tensor, weight: Tensor, bias: Tensor, act: int) -> Tensor:
    b, h, w, c = pixels.shape
    out = torch.empty((b, h, w, c), device=pixels.device, dtype=torch.bfloat16)
    code = _native.library().fim_dw5x5_bf16(
        pixels.data_ptr(), weight.data_ptr(), bias.data_ptr(), out.data_ptr(), b, h, w, c, act,
        status_word(pixels.device).data_ptr(), _stream(pixels))
    _finish(code, f"dw5x5_bf16 {tuple(pixels.shape)}", pixels.device)
    return out


@dw5x5_bf16.register_fake
def _(pixels, weight, bias, act):
    return pixels.new_empty(pixels.shape, dtype=torch.bfloat16)


@torch.library.custom_op("flashim_b200::dw5x5_mxfp8", mutates_args=())
def dw5x5_mxfp8(pixels: Tensor, weight: Tensor, bias: Tensor, act: int, swizzled: bool) -> tuple[Tensor, Tensor]:
    b, h, w, c = pixels.shape
    rows = b * h * w
    out = torch.empty((rows, c), device=pixels.device, dtype=E4M3)
    if swizzled:
        scales = _swizzled_scale_buffer(rows, c // BLOCK, pixels.device)
    else:
        scales = torch.empty((rows, c // BLOCK), device=pixels.device, dtype=torch.uint8)
    code = _native.library().fim_dw5x5_mxfp8(
        pixels.data_ptr(), weight.data_ptr(), bias.data_ptr(), out.data_ptr(), scales.data_ptr(), int(swizzled), b, h, w, c,
        act, status_word(pixels.device).data_ptr(), _stream(pixels))
    _finish(code, f"dw5x5_mxfp8 {tuple(pixels.shape)}", pixels.device)
    return out, scales


@dw5x5_mxfp8.register_fake
def _(pixels, weight, bias, act, swizzled):
    b, h, w, c = pixels.shape
    rows = b * h * w
    scales = pixels.new_empty((swizzled_scale_bytes(rows, c // BLOCK),) if swizzled else (rows, c // BLOCK), dtype=torch.uint8)
    return pixels.new_empty((rows, c), dtype=E4M3), scales


@torch.library.custom_op("flashim_b200::dw5x5_relu_int8", mutates_args=())
def dw5x5_relu_int8(pixels: Tensor, weight: Tensor, bias: Tensor, scale: Tensor) -> Tensor:
    b, h, w, c = pixels.shape
    out = torch.empty((b * h * w, c), device=pixels.device, dtype=torch.int8)
    code = _native.library().fim_dw5x5_relu_int8(
        pixels.data_ptr(), weight.data_ptr(), bias.data_ptr(), scale.data_ptr(), out.data_ptr(), b, h, w, c,
        status_word(pixels.device).data_ptr(), _stream(pixels))
    _finish(code, f"dw5x5_relu_int8 {tuple(pixels.shape)}", pixels.device)
    return out


@dw5x5_relu_int8.register_fake
def _(pixels, weight, bias, scale):
    b, h, w, c = pixels.shape
    return pixels.new_empty((b * h * w, c), dtype=torch.int8)


# ---- custom ops: quantisers -------------------------------------------------------------------------------------------


@torch.library.custom_op("flashim_b200::quantize_mxfp8_static", mutates_args=())
def quantize_mxfp8_static(value: Tensor, exponent: Tensor) -> Tensor:
    value = _aligned(value)
    channels = value.shape[-1]
    rows = value.numel() // channels
    out = torch.empty((*value.shape[:-1], padded_channels(channels)), device=value.device, dtype=E4M3)
    code = _native.library().fim_quantize_mxfp8_static(
        value.data_ptr(), _IN_DTYPES[value.dtype], exponent.data_ptr(), out.data_ptr(), rows, channels, _stream(value))
    _finish(code, f"quantize_mxfp8_static {tuple(value.shape)}", value.device)
    return out


@quantize_mxfp8_static.register_fake
def _(value, exponent):
    return value.new_empty((*value.shape[:-1], padded_channels(value.shape[-1])), dtype=E4M3)


@torch.library.custom_op("flashim_b200::quantize_mxfp8_dynamic", mutates_args=())
def quantize_mxfp8_dynamic(value: Tensor, swizzled: bool) -> tuple[Tensor, Tensor]:
    value = _aligned(value)
    channels = value.shape[-1]
    rows = value.numel() // channels
    out = torch.empty(value.shape, device=value.device, dtype=E4M3)
    if swizzled:
        scales = _swizzled_scale_buffer(rows, channels // BLOCK, value.device)
    else:
        scales = torch.empty((rows, channels // BLOCK), device=value.device, dtype=torch.uint8)
    code = _native.library().fim_quantize_mxfp8_dynamic(
        value.data_ptr(), _IN_DTYPES[value.dtype], out.data_ptr(), scales.data_ptr(), int(swizzled), rows, channels,
        _stream(value))
    _finish(code, f"quantize_mxfp8_dynamic {tuple(value.shape)}", value.device)
    return out, scales


@quantize_mxfp8_dynamic.register_fake
def _(value, swizzled):
    channels = value.shape[-1]
    rows = value.numel() // channels
    scales = value.new_empty((swizzled_scale_bytes(rows, channels // BLOCK),) if swizzled else (rows, channels // BLOCK),
                             dtype=torch.uint8)
    return value.new_empty(value.shape, dtype=E4M3), scales


@torch.library.custom_op("flashim_b200::quantize_int8_static", mutates_args=())
def quantize_int8_static(value: Tensor, scale: Tensor) -> Tensor:
    value = _aligned(value)
    out = torch.empty(value.shape, device=value.device, dtype=torch.int8)
    code = _native.library().fim_quantize_int8_static(
        value.data_ptr(), _IN_DTYPES[value.dtype], scale.data_ptr(), out.data_ptr(), value.numel(), _stream(value))
    _finish(code, f"quantize_int8_static {tuple(value.shape)}", value.device)
    return out


@quantize_int8_static.register_fake
def _(value, scale):
    return value.new_empty(value.shape, dtype=torch.int8)


@torch.library.custom_op("flashim_b200::quantize_mxfp8_static_nchw", mutates_args=())
def quantize_mxfp8_static_nchw(source: Tensor, exponent: Tensor) -> Tensor:
    """``source`` NCHW-contiguous ``[B, C, H, W]`` -> E4M3 NHWC ``[B, H, W, Cp]`` (the quantiser does the layout change)."""
    b, c, h, w = source.shape
    out = torch.empty((b, h, w, padded_channels(c)), device=source.device, dtype=E4M3)
    code = _native.library().fim_quantize_mxfp8_static_nchw(
        source.data_ptr(), _IN_DTYPES[source.dtype], exponent.data_ptr(), out.data_ptr(), b, c, h * w, _stream(source))
    _finish(code, f"quantize_mxfp8_static_nchw {tuple(source.shape)}", source.device)
    return out


@quantize_mxfp8_static_nchw.register_fake
def _(source, exponent):
    b, c, h, w = source.shape
    return source.new_empty((b, h, w, padded_channels(c)), dtype=E4M3)


@torch.library.custom_op("flashim_b200::quantize_int8_static_nchw", mutates_args=())
def quantize_int8_static_nchw(source: Tensor, scale: Tensor) -> Tensor:
    b, c, h, w = source.shape
    out = torch.empty((b, h, w, c), device=source.device, dtype=torch.int8)
    code = _native.library().fim_quantize_int8_static_nchw(
        source.data_ptr(), _IN_DTYPES[source.dtype], scale.data_ptr(), out.data_ptr(), b, c, h * w, _stream(source))
    _finish(code, f"quantize_int8_static_nchw {tuple(source.shape)}", source.device)
    return out


@quantize_int8_static_nchw.register_fake
def _(source, scale):
    b, c, h, w = source.shape
    return source.new_empty((b, h, w, c), dtype=torch.int8)


@torch.library.custom_op("flashim_b200::maxpool2_quantize_int8", mutates_args=())
def maxpool2_quantize_int8(value: Tensor, scale: Tensor) -> Tensor:
    """bf16 NHWC ``[B, H, W, C]`` -> int8 ``[B, H // 2, W // 2, C]``: MaxPool2d(2) and the static INT8 quantiser."""
    b, h, w, c = value.shape
    out = torch.empty((b, h // 2, w // 2, c), device=value.device, dtype=torch.int8)
    code = _native.library().fim_maxpool2_quantize_int8(
        value.data_ptr(), scale.data_ptr(), out.data_ptr(), b, h, w, c, _stream(value))
    _finish(code, f"maxpool2_quantize_int8 {tuple(value.shape)}", value.device)
    return out


@maxpool2_quantize_int8.register_fake
def _(value, scale):
    b, h, w, c = value.shape
    return value.new_empty((b, h // 2, w // 2, c), dtype=torch.int8)


@torch.library.custom_op("flashim_b200::romav2_refiner_input", mutates_args=())
def romav2_refiner_input_launch(f_a: Tensor, f_b: Tensor, warp: Tensor, emb_weight: Tensor, emb_bias: Tensor, scale_x: float,
                                scale_y: float, radius: int, pair: int) -> Tensor:
    """Returns the NHWC memory ``[B, h, w, 2P + E + K]`` (bf16)."""
    b, h, w, features = f_a.shape
    embedding = emb_weight.shape[0]
    k = (2 * radius + 1) ** 2 if radius >= 0 else 0
    out = torch.empty((b, h, w, 2 * features + embedding + k), device=f_a.device, dtype=torch.bfloat16)
    code = _native.library().fim_romav2_refiner_input(
        f_a.data_ptr(), f_b.data_ptr(), warp.data_ptr(), emb_weight.data_ptr(), emb_bias.data_ptr(), scale_x, scale_y,
        out.data_ptr(), b, h, w, features, embedding, radius, pair, _stream(f_a))
    _finish(code, f"romav2_refiner_input {tuple(f_a.shape)} r={radius}", f_a.device)
    return out


@romav2_refiner_input_launch.register_fake
def _(f_a, f_b, warp, emb_weight, emb_bias, scale_x, scale_y, radius, pair):
    b, h, w, features = f_a.shape
    k = (2 * radius + 1) ** 2 if radius >= 0 else 0
    return f_a.new_empty((b, h, w, 2 * features + emb_weight.shape[0] + k), dtype=torch.bfloat16)


@torch.library.custom_op("flashim_b200::romav2_refiner_heads", mutates_args=())
def romav2_refiner_heads_launch(z: Tensor, weight: Tensor, bias: Tensor, prev_warp: Tensor, prev_confidence: Tensor,
                                inv_norm_x: float, inv_norm_y: float) -> tuple[Tensor, Tensor]:
    """``z`` is the NHWC memory ``[B, h, w, C]`` (bf16) of the channels-last feature map."""
    b, h, w, c = z.shape
    warp = torch.empty((b, h, w, 2), device=z.device, dtype=torch.float32)
    confidence = torch.empty((b, h, w, 4), device=z.device, dtype=torch.float32)
    code = _native.library().fim_romav2_refiner_heads(
        z.data_ptr(), weight.data_ptr(), bias.data_ptr(), prev_warp.data_ptr(), prev_confidence.data_ptr(),
        prev_confidence.shape[-1], warp.data_ptr(), confidence.data_ptr(), b * h * w, c, inv_norm_x, inv_norm_y, _stream(z))
    _finish(code, f"romav2_refiner_heads {tuple(z.shape)}", z.device)
    return warp, confidence


@romav2_refiner_heads_launch.register_fake
def _(z, weight, bias, prev_warp, prev_confidence, inv_norm_x, inv_norm_y):
    b, h, w, _ = z.shape
    return z.new_empty((b, h, w, 2), dtype=torch.float32), z.new_empty((b, h, w, 4), dtype=torch.float32)


def _channels_first_view(value: Tensor) -> bool:
    """``value`` is ``x.permute(0, 2, 3, 1)`` of an NCHW-contiguous ``x`` and not itself row-major — the case FlashIM's
    quantisers read in place (flashim/backends/triton/quantize.py:237-239)."""
    return value.ndim == 4 and not value.is_contiguous() and value.permute(0, 3, 1, 2).is_contiguous()


# ---- custom ops: tcgen05 convs -----------------------------------------------------------------------------------------

_OUT_DTYPES = {
    _native.OUT_BF16: torch.bfloat16, _native.OUT_F32: torch.float32, _native.OUT_E4M3_STATIC: E4M3,
    _native.OUT_E4M3_DYNAMIC: E4M3, _native.OUT_INT8: torch.int8, _native.OUT_INT32: torch.int32,
}


def _out_size(size: int, k: int, p: int, d: int, s: int = 1) -> int:
    return (size + 2 * p - d * (k - 1) - 1) // s + 1


def _geometry(x: Tensor, cout: int, kh, kw, sh, sw, ph, pw, dh, dw) -> _native.ConvGeometry:
    b, h, w, cin = x.shape
    return _native.ConvGeometry(b, h, w, cin, cout, kh, kw, sh, sw, ph, pw, dh, dw)


def _aligned(t: Tensor | None) -> Tensor | None:
    """``t`` itself when its storage starts on a 16-byte boundary (what TMA and the 128-bit loads need), else a copy:
    alignment is fixed up here, in the wrapper, not tested in ``when`` (flashim/backends/cuda/conv.py:59-60 does the same)."""
    if t is None or t.data_ptr() % 16 == 0:
        return t
    return t.clone()


def _epilogue(bias, residual, act: int, out_mode: int, out_exponent=None, out_scales=None, out_scale=None):
    ep = _native.ConvEpilogue()
    ep.bias = _ptr(bias)
    ep.residual = _ptr(residual)
    if residual is not None:
        for i, s in enumerate(residual.stride()):
            ep.res_stride[i] = s
        ep.res_channels = residual.shape[-1]
    ep.act, ep.out_mode = act, out_mode
    ep.out_exponent, ep.out_scales, ep.out_scale = _ptr(out_exponent), _ptr(out_scales), _ptr(out_scale)
    return ep


@torch.library.custom_op("flashim_b200::mxfp8_conv2d", mutates_args=())
def mxfp8_conv2d_launch(
    x: Tensor, act_exponent: Tensor | None, act_scales: Tensor | None, weight: Tensor, weight_scales: Tensor,
    bias: Tensor | None, residual: Tensor | None, out_exponent: Tensor | None,
    kh: int, kw: int, sh: int, sw: int, ph: int, pw: int, dh: int, dw: int, act: int, out_mode: int,
) -> tuple[Tensor, Tensor]:
    x, weight, weight_scales, bias, act_scales = (_aligned(t) for t in (x, weight, weight_scales, bias, act_scales))
    b, h, w, _ = x.shape
    cout = weight.shape[0]
    ho, wo = _out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw)
    out = torch.empty((b, ho, wo, cout), device=x.device, dtype=_OUT_DTYPES[out_mode])
    if out_mode == _native.OUT_E4M3_DYNAMIC:
        out_scales = _swizzled_scale_buffer(b * ho * wo, cout // BLOCK, x.device)
    else:
        out_scales = torch.empty(0, device=x.device, dtype=torch.uint8)
    geometry = _geometry(x, cout, kh, kw, sh, sw, ph, pw, dh, dw)
    epilogue = _epilogue(bias, residual, act, out_mode, out_exponent, out_scales if out_scales.numel() else None)
    if x.dtype == torch.bfloat16:  # the activation quantiser runs inside the kernel (1x1 layers, Cin % 128 == 0)
        code = _native.library().fim_mxfp8_conv2d_bf16(
            x.data_ptr(), _ptr(act_exponent), weight.data_ptr(), weight_scales.data_ptr(),
            ctypes.byref(geometry), ctypes.byref(epilogue), out.data_ptr(), status_word(x.device).data_ptr(), _stream(x))
    else:
        code = _native.library().fim_mxfp8_conv2d(
            x.data_ptr(), _ptr(act_exponent), _ptr(act_scales), weight.data_ptr(), weight_scales.data_ptr(),
            ctypes.byref(geometry), ctypes.byref(epilogue), out.data_ptr(), status_word(x.device).data_ptr(), _stream(x))
    _finish(code, f"mxfp8_conv2d {tuple(x.shape)} -> {cout} k{kh}x{kw} s{sh}x{sw}", x.device)
    return out, out_scales


@mxfp8_conv2d_launch.register_fake
def _(x, act_exponent, act_scales, weight, weight_scales, bias, residual, out_exponent, kh, kw, sh, sw, ph, pw, dh, dw, act, out_mode):
    b, h, w, _ = x.shape
    cout = weight.shape[0]
    ho, wo = _out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw)
    n = swizzled_scale_bytes(b * ho * wo, cout // BLOCK) if out_mode == _native.OUT_E4M3_DYNAMIC else 0
    return x.new_empty((b, ho, wo, cout), dtype=_OUT_DTYPES[out_mode]), x.new_empty((n,), dtype=torch.uint8)


@torch.library.custom_op("flashim_b200::mxfp8_gelu_mlp_residual", mutates_args=())
def mxfp8_gelu_mlp_residual_launch(x: Tensor, x_scales: Tensor, w1: Tensor, w1_scales: Tensor, b1: Tensor, w2: Tensor,
                                   w2_scales: Tensor, b2: Tensor, residual: Tensor) -> Tensor:
    """E4M3 ``x [..., C]`` with swizzled per-pixel scales -> bf16 ``[..., C]``: up conv, GELU, requantisation, down conv and
    residual add in one kernel (C = 128 or 256)."""
    x, x_scales, w1, w1_scales, b1, w2, w2_scales, b2 = (_aligned(t) for t in (x, x_scales, w1, w1_scales, b1, w2, w2_scales, b2))
    residual = _aligned(residual.contiguous())
    channels = x.shape[-1]
    rows = x.numel() // channels
    out = torch.empty(x.shape, device=x.device, dtype=torch.bfloat16)
    code = _native.library().fim_mxfp8_gelu_mlp_residual(
        x.data_ptr(), x_scales.data_ptr(), w1.data_ptr(), w1_scales.data_ptr(), b1.data_ptr(), w2.data_ptr(), w2_scales.data_ptr(),
        b2.data_ptr(), residual.data_ptr(), out.data_ptr(), rows, channels, status_word(x.device).data_ptr(), _stream(x))
    _finish(code, f"mxfp8_gelu_mlp_residual {tuple(x.shape)}", x.device)
    return out


@mxfp8_gelu_mlp_residual_launch.register_fake
def _(x, x_scales, w1, w1_scales, b1, w2, w2_scales, b2, residual):
    return x.new_empty(x.shape, dtype=torch.bfloat16)


@torch.library.custom_op("flashim_b200::int8_conv2d", mutates_args=())
def int8_conv2d_launch(
    x: Tensor, weight: Tensor, a_scale: Tensor | None, w_scale: Tensor | None, bias: Tensor | None, residual: Tensor | None,
    out_scale: Tensor | None, kh: int, kw: int, sh: int, sw: int, ph: int, pw: int, dh: int, dw: int, act: int, out_mode: int,
) -> Tensor:
    x, weight, w_scale, bias = (_aligned(t) for t in (x, weight, w_scale, bias))
    b, h, w, _ = x.shape
    cout = weight.shape[0]
    ho, wo = _out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw)
    out = torch.empty((b, ho, wo, cout), device=x.device, dtype=_OUT_DTYPES[out_mode])
    geometry = _geometry(x, cout, kh, kw, sh, sw, ph, pw, dh, dw)
    epilogue = _epilogue(bias, residual, act, out_mode, out_scale=out_scale)
    code = _native.library().fim_int8_conv2d(
        x.data_ptr(), weight.data_ptr(), _ptr(a_scale), _ptr(w_scale), ctypes.byref(geometry), ctypes.byref(epilogue),
        out.data_ptr(), status_word(x.device).data_ptr(), _stream(x))
    _finish(code, f"int8_conv2d {tuple(x.shape)} -> {cout} k{kh}x{kw} s{sh}x{sw}", x.device)
    return out


@int8_conv2d_launch.register_fake
def _(x, weight, a_scale, w_scale, bias, residual, out_scale, kh, kw, sh, sw, ph, pw, dh, dw, act, out_mode):
    b, h, w, _ = x.shape
    ho, wo = _out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw)
    return x.new_empty((b, ho, wo, weight.shape[0]), dtype=_OUT_DTYPES[out_mode])


@torch.library.custom_op("flashim_b200::int8_conv2d_maxpool", mutates_args=())
def int8_conv2d_maxpool_launch(
    x: Tensor, weight: Tensor, a_scale: Tensor, w_scale: Tensor, bias: Tensor | None, out_scale: Tensor, kh: int, kw: int,
    sh: int, sw: int, ph: int, pw: int, dh: int, dw: int, act: int,
) -> tuple[Tensor, Tensor]:
    """One launch for both outputs of ``int8_conv2d_maxpool``: the bf16 conv output and, taken from the same tiles before
    they leave shared memory, its 2x2 max pool as INT8 codes."""
    x, weight, w_scale, bias = (_aligned(t) for t in (x, weight, w_scale, bias))
    b, h, w, _ = x.shape
    cout = weight.shape[0]
    ho, wo = _out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw)
    out = torch.empty((b, ho, wo, cout), device=x.device, dtype=torch.bfloat16)
    pooled = torch.empty((b, ho // 2, wo // 2, cout), device=x.device, dtype=torch.int8)
    geometry = _geometry(x, cout, kh, kw, sh, sw, ph, pw, dh, dw)
    epilogue = _epilogue(bias, None, act, _native.OUT_BF16, out_scale=out_scale)
    code = _native.library().fim_int8_conv2d_maxpool(
        x.data_ptr(), weight.data_ptr(), _ptr(a_scale), _ptr(w_scale), ctypes.byref(geometry), ctypes.byref(epilogue),
        out.data_ptr(), pooled.data_ptr(), status_word(x.device).data_ptr(), _stream(x))
    _finish(code, f"int8_conv2d_maxpool {tuple(x.shape)} -> {cout} k{kh}x{kw} s{sh}x{sw}", x.device)
    return out, pooled


@int8_conv2d_maxpool_launch.register_fake
def _(x, weight, a_scale, w_scale, bias, out_scale, kh, kw, sh, sw, ph, pw, dh, dw, act):
    b, h, w, _ = x.shape
    ho, wo = _out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw)
    return (x.new_empty((b, ho, wo, weight.shape[0]), dtype=torch.bfloat16),
            x.new_empty((b, ho // 2, wo // 2, weight.shape[0]), dtype=torch.int8))


@torch.library.custom_op("flashim_b200::bf16_conv2d", mutates_args=())
def bf16_conv2d_launch(x: Tensor, weight: Tensor, bias: Tensor | None, residual: Tensor | None, kh: int, kw: int, sh: int, sw: int,
                       ph: int, pw: int, dh: int, dw: int, act: int) -> Tensor:
    """bf16 NHWC ``x`` and bf16 ``weight [Cout, kh*kw*Cin]`` -> bf16 NHWC (fp32 accumulation on the tensor cores)."""
    x, weight, bias = (_aligned(t) for t in (x, weight, bias))
    b, h, w, _ = x.shape
    cout = weight.shape[0]
    ho, wo = _out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw)
    out = torch.empty((b, ho, wo, cout), device=x.device, dtype=torch.bfloat16)
    geometry = _geometry(x, cout, kh, kw, sh, sw, ph, pw, dh, dw)
    epilogue = _epilogue(bias, residual, act, _native.OUT_BF16)
    code = _native.library().fim_bf16_conv2d(
        x.data_ptr(), weight.data_ptr(), ctypes.byref(geometry), ctypes.byref(epilogue), out.data_ptr(),
        status_word(x.device).data_ptr(), _stream(x))
    _finish(code, f"bf16_conv2d {tuple(x.shape)} -> {cout} k{kh}x{kw}", x.device)
    return out


@bf16_conv2d_launch.register_fake
def _(x, weight, bias, residual, kh, kw, sh, sw, ph, pw, dh, dw, act):
    b, h, w, _ = x.shape
    return x.new_empty((b, _out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw), weight.shape[0]), dtype=torch.bfloat16)


@torch.library.custom_op("flashim_b200::gelu_quantize_mxfp8", mutates_args=())
def gelu_quantize_launch(value: Tensor, input_bias: Tensor | None, exponent: Tensor) -> Tensor:
    """bf16 ``[..., C]`` (C % 32 == 0) -> E4M3: erf GELU of ``value + input_bias`` in fp32, bf16 rounding, static quantiser."""
    value = _aligned(value)
    channels = value.shape[-1]
    out = torch.empty(value.shape, device=value.device, dtype=E4M3)
    code = _native.library().fim_gelu_quantize_mxfp8(
        value.data_ptr(), _ptr(input_bias), exponent.data_ptr(), out.data_ptr(), value.numel() // channels, channels, _stream(value))
    _finish(code, f"gelu_quantize_mxfp8 {tuple(value.shape)}", value.device)
    return out


@gelu_quantize_launch.register_fake
def _(value, input_bias, exponent):
    return value.new_empty(value.shape, dtype=E4M3)


# ---- weight-scale layout cache (ops whose signature carries plain int8 exponents) ----------------------------------------

_SWIZZLED: OrderedDict = OrderedDict()


def swizzled_weight_scales(weight_exponent: Tensor) -> Tensor:
    """The 128x4-swizzled E8M0 bytes of ``weight_exponent`` ``[Cout, K/32]``, computed once per tensor (keyed on its
    storage, shape and version; the source tensor is kept alive by the entry so the key cannot be reused)."""
    key = (weight_exponent.data_ptr(), tuple(weight_exponent.shape), weight_exponent._version, weight_exponent.device)
    hit = _SWIZZLED.get(key)
    if hit is not None:
        _SWIZZLED.move_to_end(key)
        return hit[1]
    packed = swizzle_scales(weight_exponent)
    _SWIZZLED[key] = (weight_exponent, packed)
    if len(_SWIZZLED) > 512:
        _SWIZZLED.popitem(last=False)
    return packed


# ---- eligibility ---------------------------------------------------------------------------------------------------------


def _cuda(*tensors) -> bool:
    return all(t is None or (isinstance(t, Tensor) and t.is_cuda) for t in tensors)


def _conv_geometry_ok(x, cout, k_total, kh, kw, sh, sw, ph, pw, dh, dw) -> bool:
    if x.ndim != 4 or not x.is_contiguous() or not (1 <= sh <= 4 and 1 <= sw <= 4):
        return False
    cin = x.shape[-1]
    return cin % 32 == 0 and cout % 32 == 0 and k_total == kh * kw * cin and min(kh, kw, dh, dw) >= 1 and min(ph, pw) >= 0


def _residual_ok(residual, cout) -> bool:
    return residual is None or (residual.ndim == 4 and residual.dtype == torch.bfloat16 and residual.shape[-1] <= cout)


def _depthwise_ok(value, weight, bias) -> bool:
    return (
        _cuda(value, weight, bias) and value.ndim == 4 and value.shape[1] % 32 == 0
        and value.dtype in (torch.bfloat16, torch.float32, torch.float16)
        and tuple(weight.shape) == (25, value.shape[1]) and weight.dtype == torch.bfloat16 and weight.is_contiguous()
        and tuple(bias.shape) == (value.shape[1],) and bias.dtype == torch.float32 and bias.is_contiguous()
    )


# ---- registration ---------------------------------------------------------------------------------------------------------


def register(ops=None, device_spec=None, feature=None) -> None:
    """Register the sm100 implementations into ``ops`` (default: :mod:`flashim_b200.ops`). ``device_spec`` and ``feature``
    are the registry's ``DeviceSpec`` class and ``Feature`` enum (FlashIM's own when registering into ``flashim.ops``)."""
    own = ops is None
    if own:
        from flashim_b200 import ops
        from flashim_b200.ops._registry import DeviceSpec as device_spec
        from flashim_b200.platforms import Feature as feature

    spec = device_spec("cuda", (10, 0), (10, 0))
    requires = [feature.TCGEN05, feature.TMA]
    if hasattr(feature, "SM100A_KERNELS"):
        requires.append(feature.SM100A_KERNELS)
    have = _native.available
    act_code = _native.ACT

    def mxfp8_when(x, channel_exponent, weight, weight_exponent, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu=False,
                   residual=None, out_exponent=None):
        return (
            have() and _cuda(x, channel_exponent, weight, weight_exponent, bias, residual, out_exponent)
            and x.dtype == E4M3 and weight.dtype == E4M3 and weight.is_contiguous()
            and _conv_geometry_ok(x, weight.shape[0], weight.shape[1], kh, kw, sh, sw, ph, pw, dh, dw)
            and channel_exponent.dtype == torch.int8 and tuple(channel_exponent.shape) == (x.shape[-1] // 32,)
            and weight_exponent.dtype == torch.int8 and tuple(weight_exponent.shape) == (weight.shape[0], weight.shape[1] // 32)
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.numel() == weight.shape[0]))
            and _residual_ok(residual, weight.shape[0])
        )

    @ops.mxfp8_conv2d.register("sm100", device=spec, requires=requires, priority=3, when=mxfp8_when)
    def mxfp8_conv2d(x, channel_exponent, weight, weight_exponent, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu=False,
                     residual=None, out_exponent=None):
        mode = _native.OUT_BF16 if out_exponent is None else _native.OUT_E4M3_STATIC
        exponent = None if out_exponent is None else out_exponent.to(device=x.device, dtype=torch.int8).contiguous()
        out, _ = mxfp8_conv2d_launch(
            x, channel_exponent.contiguous(), None, weight, swizzled_weight_scales(weight_exponent),
            None if bias is None else bias.contiguous(), residual, exponent, kh, kw, sh, sw, ph, pw, dh, dw,
            act_code["relu" if relu else "none"], mode)
        return out

    def fused_when(x, act_scale, weight, weight_scales, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, act="none", residual=None,
                   out_exponent=None, dynamic_out=False, out_fp32=False):
        per_pixel = act_scale.dtype == torch.uint8
        return (
            have() and _cuda(x, act_scale, weight, weight_scales, bias, residual, out_exponent)
            and x.dtype == E4M3 and weight.dtype == E4M3 and weight.is_contiguous() and weight_scales.dtype == torch.uint8
            and _conv_geometry_ok(x, weight.shape[0], weight.shape[1], kh, kw, sh, sw, ph, pw, dh, dw)
            and act in act_code and _residual_ok(residual, weight.shape[0])
            and (not per_pixel or ((kh, kw, sh, sw, ph, pw) == (1, 1, 1, 1, 0, 0) and act_scale.numel() == swizzled_scale_bytes(
                x.numel() // x.shape[-1], x.shape[-1] // BLOCK)))
            and weight_scales.numel() == swizzled_scale_bytes(weight.shape[0], weight.shape[1] // BLOCK)
            and (per_pixel or (act_scale.dtype == torch.int8 and tuple(act_scale.shape) == (x.shape[-1] // 32,)))
            and (out_exponent is None) + (not dynamic_out) + (not out_fp32) >= 2
        )

    if hasattr(ops, "mxfp8_conv2d_fused"):
        @ops.mxfp8_conv2d_fused.register("sm100", device=spec, requires=requires, priority=3, when=fused_when)
        def mxfp8_conv2d_fused(x, act_scale, weight, weight_scales, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, act="none",
                               residual=None, out_exponent=None, dynamic_out=False, out_fp32=False):
            per_pixel = act_scale.dtype == torch.uint8
            if out_fp32:
                mode = _native.OUT_F32
            elif dynamic_out:
                mode = _native.OUT_E4M3_DYNAMIC
            else:
                mode = _native.OUT_BF16 if out_exponent is None else _native.OUT_E4M3_STATIC
            out, scales = mxfp8_conv2d_launch(
                x, None if per_pixel else act_scale, act_scale if per_pixel else None, weight, weight_scales, bias, residual,
                out_exponent, kh, kw, sh, sw, ph, pw, dh, dw, act_code[act], mode)
            return (out, scales) if dynamic_out else out

    if hasattr(ops, "mxfp8_gelu_mlp_residual"):
        def mlp_residual_when(x, x_scales, w1, w1_scales, b1, w2, w2_scales, b2, residual):
            c = x.shape[-1]
            rows = x.numel() // max(c, 1)
            return (
                have() and _cuda(x, x_scales, w1, w1_scales, b1, w2, w2_scales, b2, residual) and c in (128, 256)
                and x.dtype == E4M3 and x.is_contiguous() and w1.dtype == E4M3 and w2.dtype == E4M3
                and w1.is_contiguous() and w2.is_contiguous() and tuple(w1.shape) == (2 * c, c) and tuple(w2.shape) == (c, 2 * c)
                and x_scales.dtype == torch.uint8 and x_scales.numel() == swizzled_scale_bytes(rows, c // BLOCK)
                and w1_scales.dtype == torch.uint8 and w1_scales.numel() == swizzled_scale_bytes(2 * c, c // BLOCK)
                and w2_scales.dtype == torch.uint8 and w2_scales.numel() == swizzled_scale_bytes(c, 2 * c // BLOCK)
                and b1.dtype == torch.bfloat16 and b1.numel() == 2 * c and b2.dtype == torch.bfloat16 and b2.numel() == c
                and residual.dtype == torch.bfloat16 and residual.shape == x.shape
            )

        @ops.mxfp8_gelu_mlp_residual.register("sm100", device=spec, requires=requires, priority=3, when=mlp_residual_when)
        def mxfp8_gelu_mlp_residual(x, x_scales, w1, w1_scales, b1, w2, w2_scales, b2, residual):
            return mxfp8_gelu_mlp_residual_launch(x, x_scales, w1, w1_scales, b1.contiguous(), w2, w2_scales, b2.contiguous(), residual)

    def bf16_in_when(x, act_exponent, weight, weight_scales, bias, *, act="none", residual=None, out_exponent=None,
                     dynamic_out=False, out_fp32=False):
        return (
            have() and _cuda(x, act_exponent, weight, weight_scales, bias, residual, out_exponent)
            and x.dtype == torch.bfloat16 and x.ndim == 4 and x.is_contiguous() and x.shape[-1] % 128 == 0
            and weight.dtype == E4M3 and weight.is_contiguous() and weight.shape[1] == x.shape[-1] and weight.shape[0] % BLOCK == 0
            and weight_scales.dtype == torch.uint8
            and weight_scales.numel() == swizzled_scale_bytes(weight.shape[0], weight.shape[1] // BLOCK)
            and (act_exponent is None or (act_exponent.dtype == torch.int8 and tuple(act_exponent.shape) == (x.shape[-1] // 32,)))
            and act in act_code and _residual_ok(residual, weight.shape[0])
            and (out_exponent is None) + (not dynamic_out) + (not out_fp32) >= 2
        )

    if hasattr(ops, "mxfp8_conv2d_bf16"):
        @ops.mxfp8_conv2d_bf16.register("sm100", device=spec, requires=requires, priority=3, when=bf16_in_when)
        def mxfp8_conv2d_bf16(x, act_exponent, weight, weight_scales, bias, *, act="none", residual=None, out_exponent=None,
                              dynamic_out=False, out_fp32=False):
            if out_fp32:
                mode = _native.OUT_F32
            elif dynamic_out:
                mode = _native.OUT_E4M3_DYNAMIC
            else:
                mode = _native.OUT_BF16 if out_exponent is None else _native.OUT_E4M3_STATIC
            out, scales = mxfp8_conv2d_launch(x, act_exponent, None, weight, weight_scales, bias, residual, out_exponent,
                                              1, 1, 1, 1, 0, 0, 1, 1, act_code[act], mode)
            return (out, scales) if dynamic_out else out

    def int8_when(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu=False, residual=None,
                  out_scale=None):
        return (
            have() and _cuda(x, weight, a_scale, w_scale, bias, residual, out_scale)
            and x.dtype == torch.int8 and weight.dtype == torch.int8 and weight.is_contiguous()
            and _conv_geometry_ok(x, weight.shape[0], weight.shape[1], kh, kw, sh, sw, ph, pw, dh, dw)
            and a_scale.numel() == 1 and w_scale.numel() == weight.shape[0]
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.numel() == weight.shape[0]))
            and _residual_ok(residual, weight.shape[0])
        )

    @ops.int8_conv2d.register("sm100", device=spec, requires=requires, priority=3, when=int8_when)
    def int8_conv2d(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu=False, residual=None,
                    out_scale=None):
        scale = None if out_scale is None else out_scale.to(device=x.device, dtype=torch.float32).reshape(1)
        return int8_conv2d_launch(
            x, weight, a_scale.float().reshape(1), w_scale.float().contiguous(), None if bias is None else bias.contiguous(),
            residual, scale, kh, kw, sh, sw, ph, pw, dh, dw, act_code["relu" if relu else "none"],
            _native.OUT_BF16 if out_scale is None else _native.OUT_INT8)

    if hasattr(ops, "int8_conv2d_maxpool"):
        def pool_when(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu=False, out_scale):
            return (int8_when(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, relu=relu)
                    and _cuda(out_scale) and out_scale.numel() == 1 and weight.shape[0] % 8 == 0)

        @ops.int8_conv2d_maxpool.register("sm100", device=spec, requires=requires, priority=3, when=pool_when)
        def int8_conv2d_maxpool(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu=False, out_scale):
            scale = out_scale.to(device=x.device, dtype=torch.float32).reshape(1)
            b, h, w, _ = x.shape
            if min(_out_size(h, kh, ph, dh, sh), _out_size(w, kw, pw, dw, sw)) >= 2 and x.shape[-1] % 64 == 0:
                # one launch: the epilogue pools each bf16 tile while it lies in shared memory for its own store
                return int8_conv2d_maxpool_launch(
                    x, weight, a_scale.float().reshape(1), w_scale.float().contiguous(), None if bias is None else bias.contiguous(),
                    scale, kh, kw, sh, sw, ph, pw, dh, dw, act_code["relu" if relu else "none"])
            # an output without a whole 2x2 window, or 32 / 96 / ... input channels: the conv, then the pooling pass
            out = int8_conv2d(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, relu=relu)
            return out, maxpool2_quantize_int8(out, scale)

    if hasattr(ops, "int8_conv2d_accumulators"):
        def acc_when(x, weight, kh, kw, sh, sw, ph, pw, dh, dw):
            return (have() and _cuda(x, weight) and x.dtype == torch.int8 and weight.dtype == torch.int8
                    and weight.is_contiguous()
                    and _conv_geometry_ok(x, weight.shape[0], weight.shape[1], kh, kw, sh, sw, ph, pw, dh, dw))

        @ops.int8_conv2d_accumulators.register("sm100", device=spec, requires=requires, priority=3, when=acc_when)
        def int8_conv2d_accumulators(x, weight, kh, kw, sh, sw, ph, pw, dh, dw):
            return int8_conv2d_launch(x, weight, None, None, None, None, None, kh, kw, sh, sw, ph, pw, dh, dw, 0, _native.OUT_INT32)

    # -- GEMMs: a 1x1 conv over a one-row image of M pixels -------------------------------------------------------------
    if hasattr(ops, "mxfp8_scaled_mm"):
        def scaled_mm_when(a, b_t, a_scale, b_scale, bias=None):
            return (
                have() and _cuda(a, b_t, a_scale, b_scale, bias) and a.dim() == 2 and b_t.dim() == 2
                and a.dtype == E4M3 and b_t.dtype == E4M3 and a.is_contiguous() and b_t.t().is_contiguous()
                and a.shape[1] == b_t.shape[0] and a.shape[1] % 32 == 0 and b_t.shape[1] % 32 == 0 and a.shape[0] > 0
                and a_scale.element_size() == 1 and b_scale.element_size() == 1
                and a_scale.numel() == swizzled_scale_bytes(a.shape[0], a.shape[1] // BLOCK)
                and b_scale.numel() == swizzled_scale_bytes(b_t.shape[1], a.shape[1] // BLOCK)
                and (bias is None or (bias.dtype == torch.bfloat16 and bias.numel() == b_t.shape[1]))
            )

        @ops.mxfp8_scaled_mm.register("sm100", device=spec, requires=requires, priority=3, when=scaled_mm_when)
        def mxfp8_scaled_mm(a, b_t, a_scale, b_scale, bias=None):
            m, k = a.shape
            out, _ = mxfp8_conv2d_launch(
                a.view(1, 1, m, k), None, a_scale.view(torch.uint8).reshape(-1), b_t.t(), b_scale.view(torch.uint8).reshape(-1),
                None if bias is None else bias.contiguous(), None, None, 1, 1, 1, 1, 0, 0, 1, 1, act_code["none"], _native.OUT_BF16)
            return out.view(m, -1)

    if hasattr(ops, "int8_linear"):
        def int8_linear_when(a, weight, a_scale, w_scale, bias, *, relu=False, gelu=False, residual=None):
            return (
                have() and _cuda(a, weight, a_scale, w_scale, bias, residual) and a.dim() == 2 and weight.dim() == 2
                and a.dtype == torch.int8 and weight.dtype == torch.int8 and a.is_contiguous() and weight.is_contiguous()
                and a.shape[1] == weight.shape[1] and a.shape[1] % 32 == 0 and weight.shape[0] % 32 == 0 and a.shape[0] > 0
                and a_scale.numel() == 1 and w_scale.numel() == weight.shape[0]
                and not (relu and gelu)  # ReLU then GELU: not an epilogue the kernel has
                and (bias is None or (bias.dtype == torch.bfloat16 and bias.numel() == weight.shape[0]))
                and (residual is None or (residual.dtype == torch.bfloat16 and residual.is_contiguous()
                                          and tuple(residual.shape) == (a.shape[0], weight.shape[0])))
            )

        @ops.int8_linear.register("sm100", device=spec, requires=requires, priority=3, when=int8_linear_when)
        def int8_linear(a, weight, a_scale, w_scale, bias, *, relu=False, gelu=False, residual=None):
            # the linear's order is ReLU -> bf16 -> GELU -> residual (flashim/ops/gemm.py:87-98): its ReLU comes before the
            # residual, the conv's after it, hence the epilogue's own activation code
            m, k = a.shape
            act = "gelu" if gelu else ("relu_early" if relu else "none")
            out = int8_conv2d_launch(
                a.view(1, 1, m, k), weight, a_scale.float().reshape(1), w_scale.float().contiguous(),
                None if bias is None else bias.contiguous(), None if residual is None else residual.view(1, 1, m, -1), None,
                1, 1, 1, 1, 0, 0, 1, 1, act_code[act], _native.OUT_BF16)
            return out.view(m, -1)

    # -- static MXFP8 linear, GELU -> quantise, the GELU MLP (flashim/ops/gemm.py:58-72,146-157, ops/quantize.py:62-74) ------
    def _linear(values, scale_exponent, bias, weight_values, weight_exponent):
        rows, k = values.shape
        out, _ = mxfp8_conv2d_launch(
            values.view(1, 1, rows, k), scale_exponent.contiguous(), None, weight_values, swizzled_weight_scales(weight_exponent),
            None if bias is None else bias.to(torch.bfloat16).contiguous(), None, None, 1, 1, 1, 1, 0, 0, 1, 1,
            act_code["none"], _native.OUT_BF16)
        return out.view(rows, -1)

    def _linear_operands_ok(values, exponent, w, we) -> bool:
        return (
            have() and all(isinstance(t, Tensor) for t in (values, exponent, w, we)) and _cuda(values, exponent, w, we)
            and values.dtype == E4M3 and w.dtype == E4M3 and values.is_contiguous() and w.is_contiguous()
            and values.shape[-1] == w.shape[1] and w.shape[1] % 32 == 0 and w.shape[0] % 32 == 0 and values.numel() > 0
            and exponent.dtype == torch.int8 and tuple(exponent.shape) == (w.shape[1] // 32,)
            and we.dtype == torch.int8 and tuple(we.shape) == (w.shape[0], w.shape[1] // 32)
        )

    def _quantized_ok(activation, weight) -> bool:
        return _linear_operands_ok(getattr(activation, "values", None), getattr(activation, "scale_exponent", None),
                                   getattr(weight, "values", None), getattr(weight, "scale_exponent", None))

    def _bias_exact_in_bf16(bias, n) -> bool:
        """The epilogue adds a bf16 bias (widened to fp32); a bias of another dtype is taken only if bf16 holds it exactly."""
        if bias is None:
            return True
        if not (isinstance(bias, Tensor) and bias.is_cuda and bias.numel() == n):
            return False
        return bias.dtype == torch.bfloat16 or bool((bias.to(torch.bfloat16).to(bias.dtype) == bias).all())

    if hasattr(ops, "mxfp8_linear"):
        def linear_when(activation, bias, weight):
            return _quantized_ok(activation, weight) and _bias_exact_in_bf16(bias, weight.values.shape[0])

        @ops.mxfp8_linear.register("sm100", device=spec, requires=requires, priority=3, when=linear_when)
        def mxfp8_linear(activation, bias, weight):
            values = activation.values.reshape(-1, activation.values.shape[-1])
            return _linear(values, activation.scale_exponent, bias, weight.values, weight.scale_exponent)

    if hasattr(ops, "gelu_quantize"):
        def gelu_quantize_when(value, scale_exponent, approximate="none", *, input_bias=None):
            return (
                have() and approximate == "none" and _cuda(value, scale_exponent, input_bias) and value.dtype == torch.bfloat16
                and value.is_contiguous() and value.ndim >= 2 and value.shape[-1] % 32 == 0 and value.numel() > 0
                and tuple(scale_exponent.shape) == (value.shape[-1] // 32,)
                and (input_bias is None or input_bias.numel() == value.shape[-1])
            )

        @ops.gelu_quantize.register("sm100", device=spec, requires=dw_requires_early(feature), priority=3, when=gelu_quantize_when)
        def gelu_quantize(value, scale_exponent, approximate="none", *, input_bias=None):
            exponent = (scale_exponent if scale_exponent.dtype == torch.int8 else scale_exponent.to(torch.int8)).contiguous()
            bias = None if input_bias is None else input_bias.float().contiguous()
            qt = getattr(ops, "QuantizedTensor", None) or _quantized_tensor_type(ops)
            return qt(gelu_quantize_launch(value, bias, exponent), exponent if scale_exponent.dtype != torch.int8 else scale_exponent,
                      tuple(value.shape))

    if hasattr(ops, "mxfp8_gelu_mlp"):
        def mlp_when(x, w1, b1, hidden_exponent, w2):
            if not (_quantized_ok(x, w1) and isinstance(hidden_exponent, Tensor) and isinstance(b1, Tensor)):
                return False
            hidden = w1.values.shape[0]
            return (
                hidden_exponent.is_cuda and tuple(hidden_exponent.shape) == (hidden // 32,) and b1.is_cuda and b1.numel() == hidden
                and isinstance(getattr(w2, "values", None), Tensor) and w2.values.is_cuda and w2.values.dtype == E4M3
                and w2.values.is_contiguous() and w2.values.shape[1] == hidden and w2.values.shape[0] % 32 == 0
                and tuple(w2.scale_exponent.shape) == (w2.values.shape[0], hidden // 32) and w2.scale_exponent.dtype == torch.int8
            )

        @ops.mxfp8_gelu_mlp.register("sm100", device=spec, requires=requires, priority=3, when=mlp_when)
        def mxfp8_gelu_mlp(x, w1, b1, hidden_exponent, w2):
            # three launches with the reference's rounding points: the first product rounds to bf16 before b1 is added,
            # GELU runs in fp32 on that sum, and the second product has no bias
            values = x.values.reshape(-1, x.values.shape[-1])
            hidden = _linear(values, x.scale_exponent, None, w1.values, w1.scale_exponent)
            exponent = hidden_exponent.to(torch.int8).contiguous()
            activated = gelu_quantize_launch(hidden, b1.float().contiguous(), exponent)
            return _linear(activated, exponent, None, w2.values, w2.scale_exponent)

    # -- depthwise ---------------------------------------------------------------------------------------------------
    dw_requires = [feature.TMA] + ([feature.SM100A_KERNELS] if hasattr(feature, "SM100A_KERNELS") else [])

    def dw_when(value, weight, bias, *rest, **kw):
        return have() and _depthwise_ok(value, weight, bias)

    @ops.depthwise5x5_relu_mxfp8.register("sm100", device=spec, requires=dw_requires, priority=3, when=dw_when)
    def depthwise5x5_relu_mxfp8(value, weight, bias):
        q, scales = dw5x5_mxfp8(_nhwc(value), weight, bias, act_code["relu"], True)
        return q, scales.view(torch.float8_e8m0fnu)

    def dw_int8_when(value, weight, bias, scale):
        return dw_when(value, weight, bias) and _cuda(scale) and scale.numel() == 1

    @ops.depthwise5x5_relu_int8.register("sm100", device=spec, requires=dw_requires, priority=3, when=dw_int8_when)
    def depthwise5x5_relu_int8(value, weight, bias, scale):
        return dw5x5_relu_int8(_nhwc(value), weight, bias, scale.float().reshape(1))

    if hasattr(ops, "depthwise5x5_act"):
        def dw_act_when(value, weight, bias, act="gelu"):
            return dw_when(value, weight, bias) and act in act_code

        @ops.depthwise5x5_act.register("sm100", device=spec, requires=dw_requires, priority=3, when=dw_act_when)
        def depthwise5x5_act(value, weight, bias, act="gelu"):
            return dw5x5_bf16(_nhwc(value), weight, bias, act_code[act])

        @ops.depthwise5x5_act_mxfp8.register("sm100", device=spec, requires=dw_requires, priority=3, when=dw_act_when)
        def depthwise5x5_act_mxfp8(value, weight, bias, act="gelu"):
            return dw5x5_mxfp8(_nhwc(value), weight, bias, act_code[act], True)

    # -- depthwise-separable blocks (flashim/ops/conv.py:67-138) ---------------------------------------------------------
    if hasattr(ops, "depthwise5x5_relu_pointwise"):
        def dwpw_when(value, dw_weight, dw_bias, pw_weight, pw_bias):
            c = value.shape[1] if isinstance(value, Tensor) and value.ndim == 4 else 0
            return (
                have() and _cuda(value, dw_weight, dw_bias, pw_weight, pw_bias) and c % 32 == 0 and c > 0
                and value.dtype in (torch.bfloat16, torch.float32, torch.float16)
                and tuple(dw_weight.shape) == (25, c) and dw_weight.dtype == torch.bfloat16 and dw_weight.is_contiguous()
                and tuple(dw_bias.shape) == (c,) and pw_weight.ndim == 2 and pw_weight.shape[1] == c
                and pw_weight.shape[0] % 32 == 0 and pw_weight.dtype == torch.bfloat16 and pw_weight.is_contiguous()
                and pw_bias.dtype == torch.bfloat16 and pw_bias.numel() == pw_weight.shape[0]
            )

        @ops.depthwise5x5_relu_pointwise.register("sm100", device=spec, requires=requires, priority=3, when=dwpw_when)
        def depthwise5x5_relu_pointwise(value, dw_weight, dw_bias, pw_weight, pw_bias):
            # two launches: the depthwise kernel writes its ReLU output once as bf16 (the rounding point of the reference),
            # the pointwise product is a bf16 tensor-core GEMM over the pixels with the bias in its epilogue
            hidden = dw5x5_bf16(_nhwc(value), dw_weight, dw_bias.float().contiguous(), act_code["relu"])
            out = bf16_conv2d_launch(hidden, pw_weight, pw_bias.contiguous(), None, 1, 1, 1, 1, 0, 0, 1, 1, act_code["none"])
            return out.permute(0, 3, 1, 2)

    if hasattr(ops, "depthwise5x5_relu_pointwise_mxfp8"):
        def dwpw_mx_when(value, dw_weight, dw_bias, pw_weight, pw_scale_swizzled, pw_scale_u8, pw_bias):
            c = value.shape[1] if isinstance(value, Tensor) and value.ndim == 4 else 0
            return (
                dw_when(value, dw_weight, dw_bias) and _cuda(pw_weight, pw_scale_swizzled, pw_bias) and pw_weight.dtype == E4M3
                and pw_weight.ndim == 2 and pw_weight.shape[1] == c and pw_weight.shape[0] % 32 == 0 and pw_weight.is_contiguous()
                and pw_scale_swizzled.element_size() == 1
                and pw_scale_swizzled.numel() == swizzled_scale_bytes(pw_weight.shape[0], c // BLOCK)
                and (pw_bias is None or (pw_bias.dtype == torch.bfloat16 and pw_bias.numel() == pw_weight.shape[0]))
            )

        @ops.depthwise5x5_relu_pointwise_mxfp8.register("sm100", device=spec, requires=requires, priority=3, when=dwpw_mx_when)
        def depthwise5x5_relu_pointwise_mxfp8(value, dw_weight, dw_bias, pw_weight, pw_scale_swizzled, pw_scale_u8, pw_bias):
            # the producer's swizzled E8M0 tiles are what the GEMM's tensor-memory copies read: no re-layout in between
            b, c, h, w = value.shape
            q, scales = dw5x5_mxfp8(_nhwc(value), dw_weight, dw_bias, act_code["relu"], True)
            out, _ = mxfp8_conv2d_launch(
                q.view(1, 1, b * h * w, c), None, scales, pw_weight, pw_scale_swizzled.view(torch.uint8).reshape(-1),
                None if pw_bias is None else pw_bias.contiguous(), None, None, 1, 1, 1, 1, 0, 0, 1, 1, act_code["none"],
                _native.OUT_BF16)
            return out.view(b, h, w, -1).permute(0, 3, 1, 2)

    if hasattr(ops, "depthwise5x5_relu_pointwise_int8"):
        def dwpw_i8_when(value, dw_weight, dw_bias, pw_weight, pw_wscale, pw_bias, scale):
            c = value.shape[1] if isinstance(value, Tensor) and value.ndim == 4 else 0
            return (
                dw_when(value, dw_weight, dw_bias) and _cuda(pw_weight, pw_wscale, pw_bias, scale) and scale.numel() == 1
                and pw_weight.dtype == torch.int8 and pw_weight.ndim == 2 and pw_weight.shape[1] == c
                and pw_weight.shape[0] % 32 == 0 and pw_weight.is_contiguous() and pw_wscale.numel() == pw_weight.shape[0]
                and (pw_bias is None or (pw_bias.dtype == torch.bfloat16 and pw_bias.numel() == pw_weight.shape[0]))
            )

        @ops.depthwise5x5_relu_pointwise_int8.register("sm100", device=spec, requires=requires, priority=3, when=dwpw_i8_when)
        def depthwise5x5_relu_pointwise_int8(value, dw_weight, dw_bias, pw_weight, pw_wscale, pw_bias, scale):
            b, c, h, w = value.shape
            scale32 = scale.float().reshape(1)
            q = dw5x5_relu_int8(_nhwc(value), dw_weight, dw_bias, scale32)
            out = int8_conv2d_launch(
                q.view(1, 1, b * h * w, c), pw_weight, scale32, pw_wscale.float().contiguous(),
                None if pw_bias is None else pw_bias.contiguous(), None, None, 1, 1, 1, 1, 0, 0, 1, 1, act_code["none"],
                _native.OUT_BF16)
            return out.view(b, h, w, -1).permute(0, 3, 1, 2)

    if hasattr(ops, "romav2_refiner_input"):
        def input_when(f_a, f_b, warp, emb_weight, emb_bias, scale_factor, radius, pair=0):
            # the conditions of FlashIM's own fused implementation (flashim/backends/triton/romav2.py:292-303)
            return (
                have() and _cuda(f_a, f_b, warp, emb_weight, emb_bias) and f_a.ndim == 4
                and f_a.dtype == f_b.dtype == warp.dtype == torch.float32 and f_a.is_contiguous() and f_b.is_contiguous()
                and warp.is_contiguous() and f_a.shape == f_b.shape and f_a.shape[-1] % 4 == 0 and f_a.shape[-1] <= 256
                and emb_weight.numel() == 2 * emb_weight.shape[0] and radius <= 3 and f_a.numel() > 0
                and (pair == 0 or f_a.shape[0] == 2 * pair)
            )

        @ops.romav2_refiner_input.register("sm100", device=spec, requires=dw_requires, priority=3, when=input_when)
        def romav2_refiner_input(f_a, f_b, warp, emb_weight, emb_bias, scale_factor, radius, pair=0):
            scale = scale_factor.detach().float().cpu().tolist() if isinstance(scale_factor, Tensor) else list(scale_factor)
            rows = romav2_refiner_input_launch(
                f_a, f_b, warp, emb_weight.reshape(emb_weight.shape[0], 2).float().contiguous(), emb_bias.float().contiguous(),
                float(scale[0]), float(scale[1]), int(radius), int(pair))
            return rows.permute(0, 3, 1, 2)

    if hasattr(ops, "romav2_refiner_heads"):
        def heads_when(z, weight, bias, prev_warp, prev_confidence, refine_init):
            # the conditions of FlashIM's own fused implementation (flashim/backends/triton/romav2.py:313-322)
            return (
                have() and _cuda(z, weight, bias, prev_warp, prev_confidence) and z.ndim == 4 and z.dtype == torch.bfloat16
                and z.is_contiguous(memory_format=torch.channels_last) and z.shape[1] % 8 == 0 and z.shape[1] <= 512
                and tuple(weight.shape[:2]) == (6, z.shape[1]) and weight.numel() == 6 * z.shape[1] and bias.numel() == 6
                and prev_confidence.shape[-1] in (1, 4) and prev_warp.shape[-1] == 2
                and prev_warp.dtype == torch.float32 and prev_confidence.dtype == torch.float32 and z.numel() > 0
            )

        @ops.romav2_refiner_heads.register("sm100", device=spec, requires=dw_requires, priority=3, when=heads_when)
        def romav2_refiner_heads(z, weight, bias, prev_warp, prev_confidence, refine_init):
            _, _, h, w = z.shape
            return romav2_refiner_heads_launch(
                z.permute(0, 2, 3, 1), weight.reshape(6, -1).float().contiguous(), bias.float().contiguous(),
                prev_warp.contiguous(), prev_confidence.contiguous(), 1.0 / (refine_init * w), 1.0 / (refine_init * h))

    # -- quantisers ---------------------------------------------------------------------------------------------------
    def quantize_when(value, scale_exponent):
        return (
            have() and _cuda(value, scale_exponent) and value.ndim >= 2 and value.dtype in _IN_DTYPES
            and (value.is_contiguous() or (_channels_first_view(value) and value.numel() > 0))
            and tuple(scale_exponent.shape) == (padded_channels(value.shape[-1]) // 32,)
        )

    @ops.quantize_mxfp8.register("sm100", device=spec, requires=dw_requires, priority=3, when=quantize_when)
    def quantize_mxfp8(value, scale_exponent):
        exponent = (scale_exponent if scale_exponent.dtype == torch.int8 else scale_exponent.to(torch.int8)).contiguous()
        if _channels_first_view(value):
            return _make_quantized(quantize_mxfp8_static_nchw(value.permute(0, 3, 1, 2), exponent), scale_exponent, value)
        return _make_quantized(quantize_mxfp8_static(value, exponent), scale_exponent, value)

    def _make_quantized(values, scale_exponent, value):
        qt = getattr(ops, "QuantizedTensor", None) or _quantized_tensor_type(ops)
        exponent = scale_exponent if scale_exponent.dtype == torch.int8 else scale_exponent.to(torch.int8)
        return qt(values, exponent, tuple(value.shape))

    def quantize_int8_when(value, scale, *, channel_scale=None):
        row_major = value.is_contiguous()
        channels_first = _channels_first_view(value) and value.numel() > 0 and value.shape[-1] % 16 == 0
        return (have() and channel_scale is None and _cuda(value, scale) and value.dtype in _IN_DTYPES
                and (row_major or channels_first) and scale.numel() == 1)

    @ops.quantize_int8.register("sm100", device=spec, requires=dw_requires, priority=3, when=quantize_int8_when)
    def quantize_int8(value, scale, *, channel_scale=None):
        scale32 = scale.to(device=value.device, dtype=torch.float32).reshape(())
        if _channels_first_view(value):
            return _int8_tensor_type(ops)(quantize_int8_static_nchw(value.permute(0, 3, 1, 2), scale32.reshape(1)), scale32)
        return _int8_tensor_type(ops)(quantize_int8_static(value, scale32.reshape(1)), scale32)

    if hasattr(ops, "quantize_mxfp8_dynamic"):
        def dynamic_when(value):
            return (have() and _cuda(value) and value.dtype in _IN_DTYPES and value.is_contiguous()
                    and value.shape[-1] % 32 == 0)

        @ops.quantize_mxfp8_dynamic.register("sm100", device=spec, requires=dw_requires, priority=3, when=dynamic_when)
        def quantize_mxfp8_dynamic_impl(value):
            return quantize_mxfp8_dynamic(value, True)


def dw_requires_early(feature):
    """Features of the kernels that use no tensor-core instruction."""
    return [feature.TMA] + ([feature.SM100A_KERNELS] if hasattr(feature, "SM100A_KERNELS") else [])


def _quantized_tensor_type(ops):
    """The ``QuantizedTensor`` class of the registry's own package (FlashIM's when registered into ``flashim.ops``)."""
    if ops.__name__.startswith("flashim."):
        from flashim.quant.tensor import QuantizedTensor as theirs
        return theirs
    return QuantizedTensor


def _int8_tensor_type(ops):
    if ops.__name__.startswith("flashim."):
        from flashim.quant.tensor import Int8Tensor as theirs
        return theirs
    return Int8Tensor
