"""From a model name and a preset to a module that runs: the ``load(name, preset)`` surface of this backend.

The public names and their meaning follow FlashIM's builder (flashim/build.py:50-148,212-232,344-430) so that code
written against ``flashim.load`` ports by changing the import: a model is described by a ``ModelSpec`` (how to
construct it, its precision presets, its optional graph passes and its engines); ``resolve`` turns *preset + user
config + overrides* into a validated ``RunConfig`` (substituting the nearest available precision when the asked one is
missing, or FP8 is asked on a GPU without it); ``build_config`` constructs the module, applies the requested passes in
two stages and installs the engine; ``load`` is the one-call form.

The models registered here are synthetic stacks assembled from the conv-path ops (``flashim_b200.refiner``): there are
no checkpoints or calibration tables, so the stages FlashIM has for those do not exist in this builder.
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

from flashim_b200 import config as cfg
from flashim_b200.config import RunConfig
from flashim_b200.platforms import Feature, Platform, default_device, platform_for

log = logging.getLogger("flashim_b200.build")

PRECISIONS = ("fp32", "bf16", "int8", "fp8")
# which presets stand in for a missing one, best first
_SUBSTITUTES = {"fp8": ("int8", "bf16", "fp32"), "int8": ("bf16", "fp32"), "bf16": ("fp32",), "fp32": ("bf16",)}
_STAGES = ("pre_quant", "post_quant")


# ---- what a model declares -------------------------------------------------------------------------------------------


@dataclass(frozen=True)
class Pass:
    """A named, optional transformation of the built module. ``apply(model, ctx)`` may return a summary that lands in the
    build report; ``requires(platform)`` gates it; ``exact`` says whether outputs stay bit-identical."""

    apply: Callable[[nn.Module, "BuildContext"], Any]
    stage: Literal["pre_quant", "post_quant"] = "post_quant"
    requires: Callable[[Platform], bool] | None = None
    description: str = ""
    exact: bool = True


@dataclass(frozen=True)
class EngineSpec:
    """An execution engine: ``setup(model, ctx)`` installs it on the built module (``None``: plain eager calls)."""

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
        foreign = [p for p in self.presets if p not in PRECISIONS]
        if foreign:
            raise ValueError(f"{self.name}: preset names are precisions ({', '.join(PRECISIONS)}); got {foreign}")
        if self.default_preset not in self.presets:
            raise ValueError(f"{self.name}: the default preset {self.default_preset!r} is not among its presets")

    def check(self, config: RunConfig) -> None:
        """Raise if ``config`` names a pass or an engine this model does not have, then run the model's own validation."""
        for name in config.optimize.passes:
            if name not in self.passes:
                raise ValueError(f"{self.name}: unknown pass {name!r} (it has: {', '.join(sorted(self.passes)) or 'none'})")
        if config.engine.kind not in self.engines:
            raise ValueError(f"{self.name}: unknown engine {config.engine.kind!r} (it has: {', '.join(sorted(self.engines))})")
        if self.validate is not None:
            self.validate(config)

    def closest_preset(self, wanted: str, *, excluding: str | None = None) -> str:
        for candidate in (wanted, *_SUBSTITUTES[wanted]):
            if candidate in self.presets and candidate != excluding:
                return candidate
        raise ValueError(f"{self.name}: nothing can stand in for preset {wanted!r}")


@dataclass
class BuildReport:
    """What happened while building: which passes ran (and what they returned), which were skipped and why, which
    precision substitutions were made."""

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


# ---- the model table -------------------------------------------------------------------------------------------------


class _SpecTable:
    """Specs by name; an entry may be a ``"module:attribute"`` path that is imported on first use."""

    def __init__(self) -> None:
        self._entries: dict[str, str | ModelSpec] = {"refiner-stack": "flashim_b200.refiner:SPEC"}

    def add(self, name: str, target: str | ModelSpec) -> None:
        self._entries[name] = target

    def names(self) -> list[str]:
        return sorted(self._entries)

    def get(self, name: str) -> ModelSpec:
        try:
            entry = self._entries[name]
        except KeyError:
            raise ValueError(f"no model named {name!r}; registered: {', '.join(self.names())}") from None
        if isinstance(entry, str):
            module, _, attribute = entry.partition(":")
            entry = self._entries[name] = getattr(importlib.import_module(module), attribute)
        return entry


_TABLE = _SpecTable()


def register_spec(name: str, target: str | ModelSpec) -> None:
    _TABLE.add(name, target)


def get_spec(name: str) -> ModelSpec:
    return _TABLE.get(name)


def spec_names() -> list[str]:
    return _TABLE.names()


# ---- resolve ---------------------------------------------------------------------------------------------------------


def _as_table(config) -> dict[str, Any]:
    """The user's layer as a plain table, from a RunConfig, a path, a mapping or nothing."""
    if config is None:
        return {}
    if isinstance(config, RunConfig):
        return config.to_dict()
    if isinstance(config, (str, Path)):
        return cfg.load_file(config)
    return dict(config)


def resolve(name: str, preset: str | None = None, config=None, overrides: Iterable[str] | Mapping[str, Any] = (), *,
            platform: Platform | None = None, fallbacks: dict[str, str] | None = None) -> RunConfig:
    """Preset + user config + overrides -> a validated ``RunConfig``. A preset the model lacks, or FP8 on a GPU without
    FP8, is replaced by the closest one the model has (recorded in ``fallbacks``; an error under ``optimize.strict``)."""
    spec = get_spec(name)
    user = cfg.merge(_as_table(config), cfg.parse_overrides(overrides))
    user.pop("model", None)
    from_user = user.pop("preset", None)
    wanted = preset or from_user or spec.default_preset
    if wanted not in PRECISIONS:
        raise ValueError(f"{spec.name}: {wanted!r} is not a preset; presets are {', '.join(PRECISIONS)}")
    strict = bool((user.get("optimize") or {}).get("strict"))

    chosen, why = spec.closest_preset(wanted), None
    if chosen != wanted:
        if strict:
            raise ValueError(f"{spec.name} has no {wanted!r} preset and optimize.strict forbids a substitute "
                             f"(it has: {', '.join(sorted(spec.presets))})")
        why = f"{spec.name} has no {wanted} preset"
    on_gpu_without_fp8 = (platform is not None and platform.device_type != "cpu" and not platform.supports(Feature.FP8_E4M3))
    if chosen == "fp8" and on_gpu_without_fp8:
        if strict:
            log.warning("%s: %s has no FP8; keeping preset 'fp8' because optimize.strict is set", spec.name, platform.describe())
        else:
            chosen, why = spec.closest_preset("fp8", excluding="fp8"), f"{platform.describe()} has no FP8"
    if why is not None:
        log.warning("%s: building preset %r instead of %r: %s", spec.name, chosen, wanted, why)
        if fallbacks is not None:
            fallbacks[spec.name] = f"{wanted} -> {chosen} ({why})"

    table = cfg.merge(cfg.resolve_preset(spec.presets, chosen), user)
    table["model"], table["preset"] = spec.name, chosen
    resolved = RunConfig.from_dict(table)
    spec.check(resolved)
    return resolved


# ---- build -----------------------------------------------------------------------------------------------------------


def _apply_stage(model: nn.Module, ctx: BuildContext, stage: str) -> None:
    wanted = [(name, ctx.spec.passes[name]) for name in ctx.config.optimize.passes if ctx.spec.passes[name].stage == stage]
    for name, step in wanted:
        if step.requires is not None and not step.requires(ctx.platform):
            reason = f"needs a capability {ctx.platform.describe()} lacks"
            if ctx.config.optimize.strict:
                raise RuntimeError(f"{ctx.spec.name}: pass {name!r} {reason} (optimize.strict)")
            log.warning("%s: pass %r left out: %s", ctx.spec.name, name, reason)
            ctx.report.skipped[name] = reason
        else:
            ctx.report.passes[name] = step.apply(model, ctx)


def build_config(config: RunConfig) -> nn.Module:
    """Construct the model of a resolved configuration: load, passes (pre-quant, then post-quant), engine. The module
    gets ``run_config``, ``build_report``, ``preset`` and ``engine`` attributes."""
    spec = get_spec(config.model)
    spec.check(config)
    if config.optimize.ops:
        from flashim_b200 import ops

        ops.configure(config.optimize.ops)
    model = spec.load(config)
    where = next((buffer.device for buffer in model.buffers()), None) or torch.device(config.device or "cpu")
    platform = platform_for(where)
    ctx = BuildContext(config, spec, platform, BuildReport(config.digest(), platform.describe(), engine=config.engine.kind))
    for stage in _STAGES:
        _apply_stage(model, ctx, stage)
    setup = spec.engines[config.engine.kind].setup
    if setup is not None:
        setup(model, ctx)
    model.run_config, model.build_report = config, ctx.report
    model.preset, model.engine = config.preset, config.engine.kind
    return model


def load(name: str, preset: str | None = None, *, device: torch.device | str | None = None, engine: str | None = None,
         strict: bool | None = None, config=None, overrides: Iterable[str] | Mapping[str, Any] = ()) -> nn.Module:
    """``load("refiner-stack", "fp8", device="cuda", engine="cuda-graph")``: resolve for the platform of the target
    device and build. Layers, weakest first: preset, ``config`` (RunConfig / table / file), ``overrides``, keywords."""
    keywords: dict[str, Any] = {}
    if device is not None:
        keywords["device"] = str(device)
    if engine is not None:
        keywords["engine"] = {"kind": engine}
    if strict is not None:
        keywords["optimize"] = {"strict": strict}
    user = cfg.merge(cfg.merge(_as_table(config), cfg.parse_overrides(overrides)), keywords)
    substitutions: dict[str, str] = {}
    platform = platform_for(user.get("device") or default_device())
    model = build_config(resolve(name, preset, user, platform=platform, fallbacks=substitutions))
    model.build_report.fallbacks = substitutions
    return model
