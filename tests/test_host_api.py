"""Host-side surface on the CPU: op registry semantics, platform features, config layering and the builder."""

import dataclasses
import json

import pytest
import torch

import flashim_b200
from flashim_b200 import ops
from flashim_b200.build import EAGER, ModelSpec, Pass, get_spec, register_spec, resolve, spec_names
from flashim_b200.config import RunConfig, merge, parse_overrides
from flashim_b200.ops._registry import OPS, DeviceSpec, NoImplementation, Op
from flashim_b200.platforms import Feature, Platform, isa_features, platform_for


def _op(name, reference=lambda x: "reference"):
    OPS.pop(name, None)
    return Op(name, reference)


def test_priority_then_narrowest_range():  # flashim tests/unit/test_registry.py:14-24
    op = _op("t_order")
    op.register("wide", device=DeviceSpec("cuda", (8, 0)))(lambda x: "wide")
    op.register("narrow", device=DeviceSpec("cuda", (10, 0), (10, 0)))(lambda x: "narrow")
    op.register("low", device=DeviceSpec("cuda"), priority=-1)(lambda x: "low")
    assert [i.name for i in op.candidates(Platform("cuda", 0, capability=(10, 0)))] == ["narrow", "wide", "low"]
    assert [i.name for i in op.candidates(Platform("cuda", 0, capability=(9, 0)))] == ["wide", "low"]
    assert op.candidates(Platform("cpu")) == []


def test_opt_in_overrides_and_pinning():  # flashim tests/unit/test_registry.py:27-67
    op = _op("t_cpu")
    op.register("any", device=DeviceSpec("*"), when=lambda x: x.numel() > 1)(lambda x: "any")
    op.register("extra", device=DeviceSpec("*"), priority=-1)(lambda x: "extra")
    assert op(torch.zeros(2)) == "any" and op(torch.zeros(1)) == "reference"
    assert op.explain(torch.zeros(1))["extra"].startswith("opt-in") and op.get("extra")(torch.zeros(1)) == "extra"
    ops.configure("-t_cpu")
    assert op(torch.zeros(2)) == "reference" and not op.supports(torch.zeros(2))
    ops.configure("t_cpu:any")
    assert op(torch.zeros(1)) == "any"
    ops.configure(None)
    assert op.get("reference")(torch.zeros(2)) == "reference"
    assert op.get("any")(torch.zeros(1)) == "reference"  # a pinned impl whose predicate rejects falls to the reference
    with pytest.raises(ValueError):
        op.get("missing")
    with pytest.raises(ValueError):
        ops.configure("bogus")
    assert op.supports(torch.zeros(2)) and not op.supports(torch.zeros(1))
    assert ops.call_counts()["t_cpu"]["any"] >= 2


def test_required_features_filter():
    op = _op("t_features")
    op.register("tc", device=DeviceSpec("cuda"), requires=[Feature.TCGEN05])(lambda x: "tc")
    assert op.candidates(Platform("cuda", 0, capability=(9, 0))) == []
    assert op.candidates(Platform("cuda", 0, capability=(10, 0), features=frozenset({Feature.TCGEN05})))


def test_ops_without_a_reference_raise_instead_of_falling_back():
    x = torch.zeros(4, 32, dtype=torch.bfloat16)
    with pytest.raises(NoImplementation, match="ships no fallback"):
        ops.quantize_mxfp8(x, torch.zeros(1, dtype=torch.int8))
    with pytest.raises(NoImplementation):
        ops.depthwise5x5_relu_mxfp8(torch.zeros(1, 64, 8, 8), torch.zeros(25, 64, dtype=torch.bfloat16), torch.zeros(64))
    report = ops.mxfp8_conv2d.explain(
        torch.zeros(1, 4, 4, 32, dtype=torch.float8_e4m3fn), torch.zeros(1, dtype=torch.int8),
        torch.zeros(32, 32, dtype=torch.float8_e4m3fn), torch.zeros(32, 1, dtype=torch.int8), None, 1, 1, 1, 1, 0, 0, 1, 1)
    assert "the call is on cpu" in report["sm100"] and report["reference"].startswith("none shipped")


def test_widened_ops_decline_cpu_calls_and_say_why():
    z = torch.zeros(1, 64, 4, 4, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    heads = (z, torch.zeros(6, 64), torch.zeros(6), torch.zeros(1, 4, 4, 2), torch.zeros(1, 4, 4, 1), 4.0)
    with pytest.raises(NoImplementation, match="ships no fallback"):
        ops.romav2_refiner_heads(*heads)
    assert "the call is on cpu" in ops.romav2_refiner_heads.explain(*heads)["sm100"]
    features = torch.zeros(1, 4, 4, 16)
    with pytest.raises(NoImplementation):
        ops.romav2_refiner_input(features, features, torch.zeros(1, 4, 4, 2), torch.zeros(8, 2), torch.zeros(8), torch.ones(2), 1)
    with pytest.raises(NoImplementation):
        ops.int8_conv2d_maxpool(torch.zeros(1, 4, 4, 32, dtype=torch.int8), torch.zeros(32, 32, dtype=torch.int8), torch.ones(()),
                                torch.ones(32), None, 1, 1, 1, 1, 0, 0, 1, 1, relu=True, out_scale=torch.ones(()))
    from flashim_b200.backends.sm100.kernels import _channels_first_view

    nchw = torch.zeros(2, 8, 3, 5)
    assert _channels_first_view(nchw.permute(0, 2, 3, 1)) and not _channels_first_view(nchw.permute(0, 2, 3, 1).contiguous())
    assert not _channels_first_view(nchw) and not _channels_first_view(torch.zeros(4, 8))


def test_the_sm100_backend_registers_for_capability_10_only():
    b200 = Platform("cuda", 0, "B200", (10, 0), frozenset({Feature.TCGEN05, Feature.TMA, Feature.SM100A_KERNELS}), "sm_100")
    rtx = Platform("cuda", 0, "RTX", (12, 0), frozenset({Feature.TMA}), "sm_120")
    h100 = Platform("cuda", 0, "H100", (9, 0), frozenset({Feature.TMA, Feature.WGMMA}), "sm_90")
    for name in ("mxfp8_conv2d", "int8_conv2d", "depthwise5x5_relu_mxfp8", "depthwise5x5_relu_int8", "quantize_mxfp8",
                 "quantize_int8", "mxfp8_conv2d_fused", "depthwise5x5_act", "int8_conv2d_maxpool", "mxfp8_scaled_mm",
                 "int8_linear", "romav2_refiner_input", "romav2_refiner_heads"):
        op = OPS[name]
        assert [i.name for i in op.candidates(b200)] == ["sm100"], name
        assert op.candidates(rtx) == [] and op.candidates(h100) == [], name
    no_library = Platform("cuda", 0, "B200", (10, 0), frozenset({Feature.TCGEN05, Feature.TMA}), "sm_100")
    assert OPS["mxfp8_conv2d"].candidates(no_library) == []  # kernels not built: nothing to dispatch to


def test_isa_features_and_cpu_platform():
    assert Feature.TCGEN05 in isa_features((10, 0)) and Feature.TCGEN05 not in isa_features((12, 0))
    assert Feature.WGMMA in isa_features((9, 0)) and Feature.TMA in isa_features((12, 0))
    assert platform_for("cpu").device_type == "cpu" and not platform_for("cpu").supports(Feature.TMA)


def test_merge_and_overrides():  # flashim tests/unit/test_config.py:32-49
    base = {"optimize": {"passes": ["a"], "strict": False}}
    assert merge(base, {"optimize": {"passes": ["b"]}})["optimize"] == {"passes": ["b"], "strict": False}
    assert merge(base, {"optimize": {"passes+": ["b"]}})["optimize"]["passes"] == ["a", "b"]
    assert base == {"optimize": {"passes": ["a"], "strict": False}}
    overlay = parse_overrides(["engine.kind=cuda-graph", "optimize.passes+=x", "arch.blocks=2", "optimize.strict=true"])
    assert overlay == {"engine": {"kind": "cuda-graph"}, "optimize": {"passes+": "x", "strict": True}, "arch": {"blocks": 2}}
    with pytest.raises(ValueError):
        parse_overrides(["nonsense"])


def test_resolve_roundtrip_digest_and_errors():  # flashim tests/unit/test_config.py:52-64
    config = resolve("refiner-stack", "fp8")
    again = RunConfig.from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config and again.digest() == config.digest()
    assert resolve("refiner-stack", "fp8", overrides=["arch.blocks=2"]).digest() != config.digest()
    assert config.preset == "fp8" and config.precision.quant == "mxfp8-dynamic"
    with pytest.raises(ValueError, match="no such configuration key"):
        RunConfig.from_dict({"model": "refiner-stack", "optimise": {}})
    with pytest.raises(ValueError, match="unknown pass"):
        resolve("refiner-stack", "fp8", overrides=["optimize.passes+=nope"])
    with pytest.raises(ValueError, match="unknown engine"):
        resolve("refiner-stack", "fp8", overrides=["engine.kind=compile"])
    with pytest.raises(ValueError, match="compute_dtype"):
        resolve("refiner-stack", "fp8", overrides=["precision.compute_dtype=fp64"])
    with pytest.raises(ValueError, match="is not a preset"):
        resolve("refiner-stack", "fp8-p8")
    with pytest.raises(ValueError, match="no model named"):
        resolve("romav3")


def test_nearest_preset_and_fp8_fallback():
    spec = dataclasses.replace(get_spec("refiner-stack"), name="toy", presets={"bf16": {}, "fp8": {}}, default_preset="bf16")
    register_spec("toy", spec)
    assert "toy" in spec_names()
    fallbacks = {}
    assert resolve("toy", "int8", fallbacks=fallbacks).preset == "bf16" and "toy has no int8" in fallbacks["toy"]
    with pytest.raises(ValueError, match="no 'int8' preset"):
        resolve("toy", "int8", overrides=["optimize.strict=true"])
    ampere = Platform("cuda", 0, "A100", (8, 0), frozenset(), "sm_80")
    assert resolve("toy", "fp8", platform=ampere).preset == "bf16"  # no FP8 on the device: nearest preset
    assert resolve("toy", "fp8", platform=Platform("cpu")).preset == "fp8"
    with pytest.raises(ValueError, match="preset names are precisions"):
        dataclasses.replace(spec, presets={"int8-full": {}}, default_preset="int8-full")


def test_passes_run_in_order_and_skip_when_unsupported():
    from flashim_b200.build import build_config
    from torch import nn

    log = []
    spec = ModelSpec(
        name="toy2", role="dense", description="", load=lambda config: nn.Linear(2, 2), presets={"bf16": {}},
        default_preset="bf16",
        passes={
            "a": Pass(lambda m, ctx: log.append("a") or "ran", stage="pre_quant"),
            "b": Pass(lambda m, ctx: log.append("b"), requires=lambda platform: False),
            "c": Pass(lambda m, ctx: log.append("c")),
        },
        engines={"eager": EAGER},
    )
    register_spec("toy2", spec)
    model = build_config(resolve("toy2", overrides=['optimize.passes=["c", "b", "a"]']))
    assert log == ["a", "c"] and model.build_report.passes["a"] == "ran" and "b" in model.build_report.skipped
    with pytest.raises(RuntimeError, match="pass 'b'"):
        build_config(resolve("toy2", overrides=["optimize.passes+=b", "optimize.strict=true"]))
    assert model.preset == "bf16" and model.engine == "eager" and model.run_config.model == "toy2"


def test_quant_containers_validate():
    from flashim_b200.quant import Int8Tensor, QuantizedTensor, QuantizedWeight, swizzle_scales

    w = QuantizedWeight.from_float(torch.randn(100, 70))
    assert w.values.shape == (128, 96) and w.scale_exponent.shape == (128, 3) and w.logical_shape == (100, 70)
    assert swizzle_scales(w.scale_exponent).numel() == 512
    conv = QuantizedWeight.from_conv(torch.randn(40, 48, 3, 3))
    assert conv.values.shape == (64, 9 * 64)
    with pytest.raises(ValueError):
        QuantizedTensor(torch.zeros(2, 32), torch.zeros(1, dtype=torch.int8), (2, 32))
    with pytest.raises(ValueError):
        Int8Tensor(torch.zeros(2, dtype=torch.int8), torch.zeros(2))
    assert flashim_b200.__version__
