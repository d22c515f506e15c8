"""The C ABI on a machine without a GPU: the library loads, exports every symbol the header declares, and its argument
checks answer before any launch. No compute call is made here."""

import ctypes
import re
from pathlib import Path

import pytest

from flashim_b200 import _native

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "flashim_sm100.h").read_text()
TUNE_HEADER = (ROOT / "include" / "flashim_sm100_tune.h").read_text()


def _declared(text: str = HEADER) -> list[str]:
    return sorted(set(re.findall(r"^\s*(?:int|void)\s+(fim_\w+)\s*\(", text, flags=re.M)))


def test_library_is_built_and_exports_the_header():
    lib = _native.library()
    names = _declared()
    assert len(names) >= 11
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/flashim_sm100.h but not exported"
    assert sorted(_native.SIGNATURES) == names  # the ctypes table covers exactly the header
    tune = _declared(TUNE_HEADER)
    assert sorted(_native.TUNE_SIGNATURES) == tune and all(hasattr(lib, name) for name in tune)
    assert not set(tune) & set(names)  # the schedule overrides are not part of the product header
    assert lib.fim_abi_version() == int(re.search(r"#define FIM_ABI_VERSION (\d+)", HEADER).group(1))


def test_header_cites_the_reference_interface_of_every_entry_point():
    blocks = re.split(r"\n(?=/\*)", HEADER)
    for name in _declared():
        if name in ("fim_abi_version", "fim_conv_plan", "fim_conv_schedule"):
            continue
        block = next(b for b in blocks if re.search(rf"\b{name}\s*\(", b))
        assert "flashim/" in block, f"{name}: the comment must cite the reference interface it replaces"


def test_argument_errors_are_reported_before_any_launch():
    lib = _native.library()
    assert lib.fim_quantize_mxfp8_static(None, 1, None, None, 4, 32, None) == -2
    assert lib.fim_quantize_mxfp8_static(None, 1, None, None, 0, 32, None) == 0  # empty input: nothing to do
    assert lib.fim_quantize_int8_static(None, 1, None, None, 0, None) == 0
    assert lib.fim_dw5x5_bf16(None, None, None, None, 1, 8, 8, 48, 0, None, None) == 99  # channels % 32
    assert lib.fim_dw5x5_bf16(None, None, None, None, 0, 8, 8, 64, 0, None, None) == 0
    assert lib.fim_dw5x5_bf16(None, None, None, None, 1, 8, 8, 64, 0, None, None) == -2
    geometry = _native.ConvGeometry(1, 8, 8, 64, 64, 3, 3, 5, 5, 1, 1, 1, 1)
    plan = (ctypes.c_int * 6)()
    assert lib.fim_conv_plan(ctypes.byref(geometry), 0, 0, ctypes.byref(plan)) == 99  # stride 5: no kernel
    geometry = _native.ConvGeometry(1, 8, 8, 64, 64, 3, 3, 2, 2, 1, 1, 1, 1)
    assert lib.fim_conv_plan(ctypes.byref(geometry), 0, 0, ctypes.byref(plan)) == 0
    geometry = _native.ConvGeometry(4, 100, 100, 512, 512, 3, 3, 1, 1, 1, 1, 1, 1)
    assert lib.fim_conv_plan(ctypes.byref(geometry), 0, 0, ctypes.byref(plan)) == 0
    tile_h, tile_w, block_n, block_k, stages, ctas = list(plan)
    assert tile_h * tile_w <= 128 and (tile_h, tile_w) == (5, 25) and block_k == 128 and stages >= 3 and ctas == 148
    geometry = _native.ConvGeometry(2, 33, 47, 64, 96, 1, 1, 1, 1, 0, 0, 1, 1)
    assert lib.fim_conv_plan(ctypes.byref(geometry), 0, 1, ctypes.byref(plan)) == 0 and list(plan)[:2] == [1, 128]
    with pytest.raises(RuntimeError, match="code 99"):
        _native.check(99, "probe")
