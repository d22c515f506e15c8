"""Registering the backend into a real FlashIM checkout (skipped where FlashIM is not importable, e.g. on the GPU box).
Set FLASHIM_REFERENCE to the checkout, or install FlashIM."""

import os
import sys

import pytest
import torch

# a FlashIM checkout: $FLASHIM_REFERENCE, else a directory "reference" beside this repository
reference = os.environ.get("FLASHIM_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
if os.path.isdir(os.path.join(reference, "flashim")) and reference not in sys.path:
    sys.path.append(reference)  # behind this repository, whose `tests` package must keep winning
flashim = pytest.importorskip("flashim")


def test_registers_behind_flashims_own_registry():
    from flashim import ops
    from flashim.platforms import Feature, Platform

    from flashim_b200.integration import register_into_flashim

    gained = register_into_flashim()
    assert set(gained) == {"mxfp8_conv2d", "int8_conv2d", "depthwise5x5_relu_mxfp8", "depthwise5x5_relu_int8",
                           "quantize_mxfp8", "quantize_int8", "mxfp8_scaled_mm", "int8_linear", "int8_conv2d_maxpool", "romav2_refiner_heads", "romav2_refiner_input",
                           "mxfp8_linear", "mxfp8_gelu_mlp", "gelu_quantize", "depthwise5x5_relu_pointwise",
                           "depthwise5x5_relu_pointwise_mxfp8", "depthwise5x5_relu_pointwise_int8"}
    assert register_into_flashim() == gained  # idempotent
    b200 = Platform("cuda", 0, name="B200", capability=(10, 0),
                    features=frozenset({Feature.TCGEN05, Feature.TMA, Feature.NVCC, Feature.TRITON, Feature.FP8_E4M3,
                                        Feature.MXFP8_SCALED_MM}))
    # on a B200 the sm100 implementation outranks every other candidate of these ops
    for name in gained:
        candidates = getattr(ops, name).candidates(b200)
        assert candidates and candidates[0].name == "sm100", (name, [c.name for c in candidates])
    # and it is absent elsewhere: consumer Blackwell and Hopper keep FlashIM's own kernels
    rtx = Platform("cuda", 0, capability=(12, 0), features=frozenset({Feature.TMA, Feature.TRITON, Feature.MXFP8_SCALED_MM}))
    assert all("sm100" not in [c.name for c in getattr(ops, n).candidates(rtx)] for n in gained)
    # CPU calls still reach FlashIM's torch reference, untouched
    x = (torch.randn(1, 5, 6, 32) * 3).to(torch.float8_e4m3fn)
    args = (x, torch.zeros(1, dtype=torch.int8), (torch.randn(32, 32)).to(torch.float8_e4m3fn),
            torch.zeros(32, 1, dtype=torch.int8), None, 1, 1, 1, 1, 0, 0, 1, 1)
    report = ops.mxfp8_conv2d.explain(*args)
    assert "does not match cpu" in report["sm100"] and report["reference"] == "selected"
    assert ops.mxfp8_conv2d(*args).shape == (1, 5, 6, 32)
