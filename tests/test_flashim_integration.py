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


def test_conv_modules_are_routed_to_the_fused_op_on_capability_10():
    """FlashIM's own gate keeps a wide MXFP8 conv on the im2col path unless the platform is one it was measured on; the
    pass shipped here flips such modules to the fused op (and epilogue chaining) for compute capability 10.0 only."""
    from flashim.quant.formats import mx
    from flashim.quant.methods.conv2d import StaticInt8Conv2d, StaticMXFP8Conv2d

    from flashim_b200 import integration

    torch.manual_seed(0)
    wide = torch.nn.Conv2d(256, 256, 3, padding=1)
    strided = torch.nn.Conv2d(64, 64, 3, stride=2, padding=1)
    x = torch.randn(1, 6, 6, 256)
    model = torch.nn.Sequential(
        StaticMXFP8Conv2d.from_conv(wide, mx.calibrate_block32_exponent(x)),
        StaticMXFP8Conv2d.from_conv(strided, mx.calibrate_block32_exponent(x[..., :64])),
        StaticInt8Conv2d.from_conv(strided, torch.tensor(0.05)),
    )
    assert not model[0].use_fused and not model[0].chain_output  # 72 (tap, block) products on an unlisted platform
    assert integration.enable_sm100_conv_paths(model, capability=(9, 0)) == []
    assert integration.enable_sm100_conv_paths(model) == []  # CPU tensors: no capability
    changed = integration.enable_sm100_conv_paths(model, capability=(10, 0))
    assert changed == ["0", "1", "2"]
    assert all(m.use_fused and m.chain_output for m in model[:2]) and model[2].chain_output
    assert model[0].feeds(model[0])
    conv_pass = integration.SM100_CONV_PASS
    assert conv_pass.stage == "post_quant" and conv_pass.apply(model, None) == []
