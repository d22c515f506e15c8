"""Model builder with FlashIM's public surface (flashim/build.py:50-148,212-232,344-430): ``ModelSpec`` +
``RunConfig`` -> a ready-to-run module; ``register_spec`` / ``get_spec``; ``resolve`` (preset + config + overrides ->
validated ``RunConfig``, FP8 replaced by the nearest preset on a GPU without FP8); ``build_config`` (stages: load ->
pre-quant passes -> post-quant passes -> engine); ``load(name, preset, *, device, engine, strict, config, overrides)``.

The models this package registers are synthetic stacks built from the conv-path ops (see ``flashim_b200.refiner``); the
stages that need checkpoints or calibration tables in FlashIM have no counterpart here.
"""

from __future__ import annotations

import importlib
import logging
from collections.abc import Callable, Iterable, Mapping, Sequence
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Literal

import torch
from torch import nn

from flashim_b200.config import RunConfig, load_file, merge, parse_overrides, resolve_preset
from flashim_b200.platforms import Feature, Platform, default_device, platform_for

logger = logging.getLogger("flashim_b200.build")

PRECISIONS = ("fp32", "bf16", "int8", "fp8")
NEAREST = {"fp8": ("int8", "bf16", "fp32"), "int8": ("bf16", "fp32"), "bf16": ("fp32",), "fp32": ("bf16",)}


@dataclass(frozen=True)
class Pass:
    apply: Callable[[nn.Module, "BuildContext"], Any]
    stage: Literal["pre_quant", "post_quant"] = "post_quant"
    requires: Callable[[Platform], bool] | None = None
    description: str = ""
    exact: bool = True


@dataclass(frozen=True)
class EngineSpec:
    """``setup(model, ctx)`` prepares the engine (for ``cuda-graph``: wraps the forward in a graph runner)."""

    regions: Sequence[str] = ()
    setup: Callable[[nn.Module, "BuildContext"], None] | None = None


EAGER = EngineSpec()


@dataclass(frozen=True)
class ModelSpec:
    name: str
    role: str
    description: str
    load: Callable[[RunConfig], nn.Module]
    presets: Mapping[str, Mapping[str, Any]]
    default_preset: str
    passes: Mapping[str, Pass] = field(default_factory=dict)
    engines: Mapping[str, EngineSpec] = field(default_factory=lambda: {"eager": EAGER})
    validate: Callable[[RunConfig], None] | None = None

    def __post_init__(self) -> None:
        unknown = sorted(set(self.presets) - set(PRECISIONS))
        if unknown or self.default_preset not in self.presets:
            raise ValueError(f"{self.name}: presets must be among {PRECISIONS} and include the default, got "
                             f"{sorted(self.presets)} (default {self.default_preset!r})")

    def check(self, config: RunConfig) -> None:
        unknown = [p for p in config.optimize.passes if p not in self.passes]
        if unknown:
            raise ValueError(f"{self.name}: unknown pass(es) {unknown}; available: {sorted(self.passes)}")
        if config.engine.kind not in self.engines:
            raise ValueError(f"{self.name}: unknown engine {config.engine.kind!r}; choose from {sorted(self.engines)}")
        if self.validate is not None:
            self.validate(config)


@dataclass
class BuildReport:
    config_digest: str
    platform: str
    passes: dict[str, Any] = field(default_factory=dict)
    skipped: dict[str, str] = field(default_factory=dict)
    fallbacks: dict[str, str] = field(default_factory=dict)
    engine: str = "eager"


@dataclass
class BuildContext:
    config: RunConfig
    spec: ModelSpec
    platform: Platform
    report: BuildReport

    def option(self, name: str, default: Any = None) -> Any:
        return self.config.optimize.options.get(name, default)


_SPEC_PATHS: dict[str, str] = {"refiner-stack": "flashim_b200.refiner:SPEC"}
_SPECS: dict[str, ModelSpec] = {}


def register_spec(name: str, target: str | ModelSpec) -> None:
    if isinstance(target, ModelSpec):
        _SPECS[name] = target
    else:
        _SPEC_PATHS[name] = target


def get_spec(name: str) -> ModelSpec:
    spec = _SPECS.get(name)
    if spec is None:
        if name not in _SPEC_PATHS:
            raise ValueError(f"Unknown model {name!r}; available: {sorted({*_SPECS, *_SPEC_PATHS})}")
        module, attr = _SPEC_PATHS[name].split(":")
        spec = _SPECS[name] = getattr(importlib.import_module(module), attr)
    return spec


def spec_names() -> list[str]:
    return sorted({*_SPECS, *_SPEC_PATHS})


def _nearest(spec: ModelSpec, preset: str, skip: str | None = None) -> str:
    return next(p for p in (preset, *NEAREST[preset]) if p in spec.presets and p != skip)


def _user_overlay(config) -> dict[str, Any]:
    if isinstance(config, RunConfig):
        return config.to_dict()
    if isinstance(config, (str, Path)):
        return load_file(config)
    return dict(config) if config is not None else {}


def resolve(name: str, preset: str | None = None, config=None, overrides: Iterable[str] | Mapping[str, Any] = (), *,
            platform: Platform | None = None, fallbacks: dict[str, str] | None = None) -> RunConfig:
    spec = get_spec(name)
    user = merge(_user_overlay(config), parse_overrides(overrides))
    user.pop("model", None)
    preset = preset or user.pop("preset", None) or spec.default_preset
    user.pop("preset", None)
    if preset not in PRECISIONS:
        raise ValueError(f"{spec.name}: unknown preset {preset!r}; choose from {PRECISIONS}")
    strict = bool((user.get("optimize") or {}).get("strict", False))
    built, reason = _nearest(spec, preset), None
    if built != preset:
        if strict:
            raise ValueError(f"{spec.name}: no {preset!r} preset (optimize.strict); available: {sorted(spec.presets)}")
        reason = f"{spec.name} has no {preset}"
    if built == "fp8" and platform is not None and platform.device_type != "cpu" and not platform.supports(Feature.FP8_E4M3):
        if strict:
            logger.warning("%s: no FP8 on %s, preset 'fp8' kept (optimize.strict)", spec.name, platform.describe())
        else:
            built, reason = _nearest(spec, "fp8", skip="fp8"), f"no FP8 on {platform.describe()}"
    if reason is not None:
        logger.warning("%s: preset %r replaced by %r (%s)", spec.name, preset, built, reason)
        if fallbacks is not None:
            fallbacks[spec.name] = f"{preset} -> {built} ({reason})"
    data = merge(resolve_preset(spec.presets, built), user)
    data.update(model=spec.name, preset=built)
    resolved = RunConfig.from_dict(data)
    spec.check(resolved)
    return resolved


def _run_passes(model: nn.Module, ctx: BuildContext, stage: str) -> None:
    for name in ctx.config.optimize.passes:
        p = ctx.spec.passes[name]
        if p.stage != stage:
            continue
        if p.requires is not None and not p.requires(ctx.platform):
            reason = f"not supported on {ctx.platform.describe()}"
            if ctx.config.optimize.strict:
                raise RuntimeError(f"{ctx.spec.name}: pass {name!r} {reason}")
            logger.warning("%s: skipping pass %r (%s)", ctx.spec.name, name, reason)
            ctx.report.skipped[name] = reason
            continue
        ctx.report.passes[name] = p.apply(model, ctx)


def build_config(config: RunConfig) -> nn.Module:
    spec = get_spec(config.model)
    spec.check(config)
    if config.optimize.ops:
        from flashim_b200 import ops

        ops.configure(config.optimize.ops)
    model = spec.load(config)
    device = next((b.device for b in model.buffers()), torch.device(config.device or "cpu"))
    platform = platform_for(device)
    report = BuildReport(config.digest(), platform.describe(), engine=config.engine.kind)
    ctx = BuildContext(config, spec, platform, report)
    _run_passes(model, ctx, "pre_quant")
    _run_passes(model, ctx, "post_quant")
    engine = spec.engines[config.engine.kind]
    if engine.setup is not None:
        engine.setup(model, ctx)
    model.run_config, model.build_report = config, report
    model.preset, model.engine = config.preset, config.engine.kind
    return model


def load(name: str, preset: str | None = None, *, device: torch.device | str | None = None, engine: str | None = None,
         strict: bool | None = None, config=None, overrides: Iterable[str] | Mapping[str, Any] = ()) -> nn.Module:
    """Load a registered model: ``preset`` + ``config`` (RunConfig / dict / file) + dotted ``overrides`` + the keyword
    arguments (later layers win), resolved for the target device's platform and built."""
    overlay: dict[str, Any] = {}
    if device is not None:
        overlay["device"] = str(device)
    if engine is not None:
        overlay["engine"] = {"kind": engine}
    if strict is not None:
        overlay["optimize"] = {"strict": strict}
    user = merge(merge(_user_overlay(config), parse_overrides(overrides)), overlay)
    fallbacks: dict[str, str] = {}
    platform = platform_for(user.get("device") or default_device())
    model = build_config(resolve(name, preset, user, platform=platform, fallbacks=fallbacks))
    model.build_report.fallbacks = fallbacks
    return model
