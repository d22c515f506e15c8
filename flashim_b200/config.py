"""Run configuration with FlashIM's layering rules (flashim/config.py:38-216): frozen dataclasses, resolution
``defaults < preset (extends chain) < config dict / file < dotted overrides < keyword arguments``, ``"key+"`` appends to
a list, unknown keys are errors, and a stable ``digest()`` of the resolved config."""

from __future__ import annotations

import copy
import dataclasses
import hashlib
import json
from collections.abc import Iterable, Mapping
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any

DTYPES = ("fp32", "bf16", "fp16")


@dataclass(frozen=True)
class Precision:
    compute_dtype: str = "bf16"
    quant: str | None = None
    calibration: str | None = None
    overrides: dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class Optimize:
    passes: tuple[str, ...] = ()
    attention: str = "sdpa"
    ops: str = ""
    strict: bool = False
    options: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class Engine:
    kind: str = "eager"
    mode: str | None = None
    dynamic: bool = False


@dataclass(frozen=True)
class RunConfig:
    model: str
    preset: str | None = None
    variant: str | None = None
    checkpoint: str | None = None
    device: str | None = None
    arch: dict[str, Any] = field(default_factory=dict)
    precision: Precision = field(default_factory=Precision)
    optimize: Optimize = field(default_factory=Optimize)
    engine: Engine = field(default_factory=Engine)
    inference: dict[str, Any] = field(default_factory=dict)
    components: dict[str, "RunConfig"] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return _plain(self)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RunConfig":
        return _typed(cls, data, "")

    def digest(self) -> str:
        text = json.dumps(self.to_dict(), sort_keys=True, separators=(",", ":"), default=str)
        return hashlib.sha256(text.encode()).hexdigest()[:12]

    def replace(self, **changes) -> "RunConfig":
        return dataclasses.replace(self, **changes)


_SECTIONS = {"precision": Precision, "optimize": Optimize, "engine": Engine}


def _plain(value: Any) -> Any:
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        return {f.name: _plain(getattr(value, f.name)) for f in fields(value)}
    if isinstance(value, tuple):
        return [_plain(v) for v in value]
    if isinstance(value, dict):
        return {k: _plain(v) for k, v in value.items()}
    return value


def _typed(cls: type, data: Mapping[str, Any], where: str) -> Any:
    known = {f.name for f in fields(cls)}
    unknown = sorted(set(data) - known)
    if unknown:
        raise ValueError(f"Unknown config key(s) {[where + k for k in unknown]}; valid: {sorted(known)}")
    kwargs = {}
    for name, value in data.items():
        section = _SECTIONS.get(name)
        if section is not None and value is not None and not isinstance(value, section):
            if not isinstance(value, Mapping):
                raise TypeError(f"{where}{name} must be a mapping, got {type(value).__name__}")
            value = _typed(section, value, f"{where}{name}.")
        elif name == "passes":
            value = tuple(value)
        elif name == "components":
            value = {k: v if isinstance(v, RunConfig) else _typed(RunConfig, v, f"{where}components.{k}.") for k, v in value.items()}
        kwargs[name] = value
    config = cls(**kwargs)
    if isinstance(config, Precision) and config.compute_dtype not in DTYPES:
        raise ValueError(f"{where}compute_dtype must be one of {DTYPES}, got {config.compute_dtype!r}")
    return config


def merge(base: Mapping[str, Any], overlay: Mapping[str, Any]) -> dict[str, Any]:
    """Deep merge into a new dict: mappings recurse, other values are replaced, ``"key+"`` appends to the list at ``key``."""
    out = dict(base)
    for key, value in overlay.items():
        if key.endswith("+"):
            key = key[:-1]
            out[key] = [*(out.get(key) or ()), *(value if isinstance(value, (list, tuple)) else [value])]
        elif isinstance(value, Mapping):  # also normalises "key+" entries of a section the base does not have yet
            out[key] = merge(out[key] if isinstance(out.get(key), Mapping) else {}, value)
        else:
            out[key] = value
    return out


def _parse_value(text: str) -> Any:
    try:
        return json.loads(text)
    except json.JSONDecodeError:
        low = text.lower()
        if low in ("true", "false"):
            return low == "true"
        if low in ("none", "null"):
            return None
        return text


def parse_overrides(overrides: Iterable[str] | Mapping[str, Any]) -> dict[str, Any]:
    """``["engine.kind=cuda-graph", "optimize.passes+=x"]`` or ``{"engine.kind": ...}`` -> nested overlay dict."""
    pairs = overrides.items() if isinstance(overrides, Mapping) else (_split(o) for o in overrides)
    overlay: dict[str, Any] = {}
    for dotted, value in pairs:
        if isinstance(value, str) and not isinstance(overrides, Mapping):
            value = _parse_value(value)
        *parents, leaf = dotted.split(".")
        node = overlay
        for part in parents:
            node = node.setdefault(part, {})
        node[leaf] = value
    return overlay


def _split(override: str) -> tuple[str, str]:
    if "+=" in override:
        key, value = override.split("+=", 1)
        return key.strip() + "+", value.strip()
    if "=" not in override:
        raise ValueError(f"Override {override!r} is not key=value")
    key, value = override.split("=", 1)
    return key.strip(), value.strip()


def load_file(path: str | Path) -> dict[str, Any]:
    path = Path(path)
    text = path.read_text()
    if path.suffix == ".toml":
        import tomllib

        return tomllib.loads(text)
    if path.suffix == ".json":
        return json.loads(text)
    if path.suffix in (".yaml", ".yml"):
        import yaml

        return yaml.safe_load(text) or {}
    raise ValueError(f"Unsupported config file type {path.suffix!r} (use .toml, .json or .yaml)")


def resolve_preset(presets: Mapping[str, Mapping[str, Any]], name: str) -> dict[str, Any]:
    if name not in presets:
        raise ValueError(f"Unknown preset {name!r}; choose from {sorted(presets)}")
    overlay = copy.deepcopy(dict(presets[name]))
    parent = overlay.pop("extends", None)
    return merge(resolve_preset(presets, parent), overlay) if parent else overlay
