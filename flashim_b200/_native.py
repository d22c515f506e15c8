"""ctypes binding of ``libflashim_sm100.so`` (the C ABI declared in ``include/flashim_sm100.h``).

The library is built in-tree by :mod:`flashim_b200.build_native` (``nvcc`` for sm_100a) and loaded from
``flashim_b200/_lib``. There is no fallback: a missing library is an error, not a slower path.
"""

from __future__ import annotations

import ctypes
import functools
import os
from pathlib import Path

LIBRARY_NAME = "libflashim_sm100.so"
#: the in-tree build; ``FLASHIM_B200_LIBRARY`` names another build of the same sources (e.g. one with measurement probes)
LIBRARY_PATH = Path(os.environ.get("FLASHIM_B200_LIBRARY") or Path(__file__).resolve().parent / "_lib" / LIBRARY_NAME)

DTYPE_F32, DTYPE_BF16 = 0, 1
ACT = {"none": 0, "relu": 1, "gelu": 2, "relu_early": 3}
OUT_BF16, OUT_F32, OUT_E4M3_STATIC, OUT_E4M3_DYNAMIC, OUT_INT8, OUT_INT32 = range(6)

ERRORS = {
    -1: "unsupported pointer alignment or layout",
    -2: "invalid argument",
    -3: "the CUDA driver could not encode a tensor map",
    99: "no kernel compiled for this geometry",
}
STATUS = {
    0x101: "a TMA load never arrived (full barrier)",
    0x102: "the MMA warp never released a stage (empty barrier)",
    0x103: "the accumulator never completed (tensor-memory full barrier)",
    0x104: "the epilogue never released the accumulator (tensor-memory empty barrier)",
    0x105: "a depthwise row never arrived (row ring barrier)",
}


class NativeLibraryMissing(RuntimeError):
    pass


class ConvGeometry(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int) for name in (
        "batch", "height", "width", "cin", "cout", "kh", "kw", "stride_h", "stride_w", "pad_h", "pad_w", "dil_h", "dil_w")]


class ConvEpilogue(ctypes.Structure):
    _fields_ = [
        ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p),
        ("res_stride", ctypes.c_longlong * 4),
        ("res_channels", ctypes.c_int),
        ("act", ctypes.c_int),
        ("out_mode", ctypes.c_int),
        ("out_exponent", ctypes.c_void_p),
        ("out_scales", ctypes.c_void_p),
        ("out_scale", ctypes.c_void_p),
    ]


_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong

#: every symbol ``include/flashim_sm100.h`` declares -> (restype, argtypes)
SIGNATURES: dict[str, tuple] = {
    "fim_abi_version": (_I, []),
    "fim_quantize_mxfp8_static": (_I, [_P, _I, _P, _P, _L, _I, _P]),
    "fim_quantize_mxfp8_dynamic": (_I, [_P, _I, _P, _P, _I, _L, _I, _P]),
    "fim_quantize_int8_static": (_I, [_P, _I, _P, _P, _L, _P]),
    "fim_quantize_mxfp8_static_nchw": (_I, [_P, _I, _P, _P, _I, _I, _L, _P]),
    "fim_quantize_int8_static_nchw": (_I, [_P, _I, _P, _P, _I, _I, _L, _P]),
    "fim_maxpool2_quantize_int8": (_I, [_P, _P, _P, _I, _I, _I, _I, _P]),
    "fim_romav2_refiner_input": (_I, [_P, _P, _P, _P, _P, ctypes.c_float, ctypes.c_float, _P, _I, _I, _I, _I, _I, _I, _I, _P]),
    "fim_romav2_refiner_heads": (_I, [_P, _P, _P, _P, _P, _I, _P, _P, _L, _I, ctypes.c_float, ctypes.c_float, _P]),
    "fim_dw5x5_bf16": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "fim_dw5x5_mxfp8": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P]),
    "fim_dw5x5_relu_int8": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "fim_mxfp8_conv2d": (_I, [_P, _P, _P, _P, _P, ctypes.POINTER(ConvGeometry), ctypes.POINTER(ConvEpilogue), _P, _P, _P]),
    "fim_mxfp8_conv2d_bf16": (_I, [_P, _P, _P, _P, ctypes.POINTER(ConvGeometry), ctypes.POINTER(ConvEpilogue), _P, _P, _P]),
    "fim_int8_conv2d": (_I, [_P, _P, _P, _P, ctypes.POINTER(ConvGeometry), ctypes.POINTER(ConvEpilogue), _P, _P, _P]),
    "fim_mxfp8_gelu_mlp_residual": (_I, [_P] * 10 + [ctypes.c_longlong, _I, _P, _P]),
    "fim_int8_conv2d_maxpool": (_I, [_P, _P, _P, _P, ctypes.POINTER(ConvGeometry), ctypes.POINTER(ConvEpilogue), _P, _P, _P, _P]),
    "fim_bf16_conv2d": (_I, [_P, _P, ctypes.POINTER(ConvGeometry), ctypes.POINTER(ConvEpilogue), _P, _P, _P]),
    "fim_gelu_quantize_mxfp8": (_I, [_P, _P, _P, _P, _L, _I, _P]),
    "fim_conv_plan": (_I, [ctypes.POINTER(ConvGeometry), _I, _I, ctypes.POINTER(ctypes.c_int * 6)]),
    "fim_conv_schedule": (_I, [ctypes.POINTER(ConvGeometry), _I, _I, ctypes.POINTER(ctypes.c_int * 8)]),
}

#: the schedule overrides of ``include/flashim_sm100_tune.h`` (tests and measurements only)
TUNE_SIGNATURES: dict[str, tuple] = {
    "fim_conv_tune": (None, [_I, _I, _I]),
    "fim_dw_tune": (None, [_I, _I]),
}


@functools.cache
def library() -> ctypes.CDLL:
    """The loaded library with every entry point typed. Raises :class:`NativeLibraryMissing` if it was not built."""
    if not LIBRARY_PATH.is_file():
        raise NativeLibraryMissing(
            f"{LIBRARY_PATH} is missing: build it with `python -m flashim_b200.build_native` (needs nvcc with sm_100a "
            "support). flashim_b200 has no fallback implementation."
        )
    lib = ctypes.CDLL(str(LIBRARY_PATH))
    for name, (restype, argtypes) in {**SIGNATURES, **TUNE_SIGNATURES}.items():
        fn = getattr(lib, name)  # AttributeError if the library and the header disagree
        fn.restype, fn.argtypes = restype, argtypes
    return lib


def available() -> bool:
    return LIBRARY_PATH.is_file()


def check(code: int, what: str) -> None:
    """Raise for a non-zero return code of an entry point (as flashim/backends/cuda/conv.py:69-70 does)."""
    if code == 0:
        return
    reason = ERRORS.get(code, f"CUDA error {code}" if code > 0 else f"error {code}")
    raise RuntimeError(f"{what} failed: {reason} (code {code})")
