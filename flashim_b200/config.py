"""Run configuration for ``load(name, preset)``: what FlashIM's ``RunConfig`` surface means for this backend.

A configuration is resolved from layers, later layers winning: section defaults, the model's preset (presets may name a
parent with ``extends``), a user dict / file, dotted ``key=value`` overrides, keyword arguments. A trailing ``+`` on a key
(``"optimize.passes+=x"``) appends to the list below it instead of replacing it; a key no section declares is an error
rather than a silent no-op; ``digest()`` names a resolved configuration by twelve hex digits of the SHA-256 of its
canonical JSON. The layering rules and field names follow flashim/config.py:38-216 so that a FlashIM user's configs and
overrides carry over; the implementation here is schema-driven: each section is a frozen dataclass and
``RunConfig.from_dict`` walks the declared fields.
"""

from __future__ import annotations

import dataclasses
import hashlib
import json
from collections.abc import Iterable, Mapping
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

DTYPES = ("fp32", "bf16", "fp16")


@dataclass(frozen=True)
class Precision:
    """Arithmetic of the model outside the quantised ops, and which quantisation recipe applies."""

    compute_dtype: str = "bf16"
    quant: str | None = None
    calibration: str | None = None
    overrides: dict[str, str] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.compute_dtype not in DTYPES:
            raise ValueError(f"precision.compute_dtype is {self.compute_dtype!r}; allowed values: {', '.join(DTYPES)}")


@dataclass(frozen=True)
class Optimize:
    """Graph passes by name, op-registry overrides (``ops``: a ``configure`` string) and pass options."""

    passes: tuple[str, ...] = ()
    attention: str = "sdpa"
    ops: str = ""
    strict: bool = False
    options: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "passes", tuple(self.passes))  # lists from JSON / TOML become the hashable form


@dataclass(frozen=True)
class Engine:
    """How the built module is executed: ``kind`` names one of the model spec's engines."""

    kind: str = "eager"
    mode: str | None = None
    dynamic: bool = False


def _section_types() -> dict[str, type]:
    return {"precision": Precision, "optimize": Optimize, "engine": Engine}


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

    # -- conversion ------------------------------------------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        """Plain containers only (tuples as lists): what ``json`` / ``toml`` can carry and ``from_dict`` reads back."""
        return _to_plain(self)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RunConfig":
        return _build(cls, data, prefix="")

    def replace(self, **changes) -> "RunConfig":
        return dataclasses.replace(self, **changes)

    def digest(self) -> str:
        canonical = json.dumps(self.to_dict(), sort_keys=True, separators=(",", ":"), default=str)
        return hashlib.sha256(canonical.encode("utf-8")).hexdigest()[:12]


# ---- dict <-> dataclasses ------------------------------------------------------------------------------------------


def _to_plain(node: Any) -> Any:
    if dataclasses.is_dataclass(node) and not isinstance(node, type):
        return {f.name: _to_plain(getattr(node, f.name)) for f in dataclasses.fields(node)}
    if isinstance(node, Mapping):
        return {key: _to_plain(item) for key, item in node.items()}
    if isinstance(node, (tuple, list)):
        return [_to_plain(item) for item in node]
    return node


def _build(schema: type, data: Mapping[str, Any], prefix: str) -> Any:
    """Instantiate the dataclass ``schema`` from ``data``, recursing into sections and sub-model components."""
    declared = [f.name for f in dataclasses.fields(schema)]
    strangers = [key for key in data if key not in declared]
    if strangers:
        named = ", ".join(prefix + key for key in sorted(strangers))
        raise ValueError(f"no such configuration key: {named} (this level has: {', '.join(declared)})")
    sections = _section_types()
    values: dict[str, Any] = {}
    for key, item in data.items():
        if schema is RunConfig and key in sections and item is not None and not isinstance(item, sections[key]):
            if not isinstance(item, Mapping):
                raise TypeError(f"{prefix}{key} takes a table of settings, not {type(item).__name__}")
            item = _build(sections[key], item, f"{prefix}{key}.")
        elif schema is RunConfig and key == "components":
            item = {name: sub if isinstance(sub, RunConfig) else _build(RunConfig, sub, f"{prefix}components.{name}.")
                    for name, sub in item.items()}
        values[key] = item
    return schema(**values)


# ---- layering --------------------------------------------------------------------------------------------------------


def merge(base: Mapping[str, Any], overlay: Mapping[str, Any]) -> dict[str, Any]:
    """A new dict: ``overlay`` laid over ``base``. Tables merge key by key; anything else replaces; ``"key+"`` extends the
    list at ``key`` (a missing list counts as empty, a scalar as a one-element list)."""
    result = dict(base)
    for key, item in overlay.items():
        if key.endswith("+"):
            target = key[:-1]
            addition = list(item) if isinstance(item, (list, tuple)) else [item]
            result[target] = list(result.get(target) or []) + addition
        elif isinstance(item, Mapping):
            below = result.get(key)
            result[key] = merge(below if isinstance(below, Mapping) else {}, item)
        else:
            result[key] = item
    return result


def _literal(text: str) -> Any:
    """An override's right-hand side: JSON where it parses (numbers, lists, quoted strings), a few bare words, else text."""
    try:
        return json.loads(text)
    except ValueError:
        pass
    bare = {"true": True, "false": False, "none": None, "null": None}
    return bare.get(text.lower(), text)


def _assignment(text: str) -> tuple[str, Any]:
    """``"a.b=1"`` -> ``("a.b", 1)``; ``"a.b+=x"`` -> ``("a.b+", "x")``."""
    head, sep, tail = text.partition("=")
    if not sep:
        raise ValueError(f"an override reads key=value (or key+=value); got {text!r}")
    head = head.strip()
    return head, _literal(tail.strip())


def parse_overrides(overrides: Iterable[str] | Mapping[str, Any] | None) -> dict[str, Any]:
    """Dotted assignments -> the nested overlay ``merge`` takes. Strings are ``key=value`` with the value parsed as in
    ``_literal``; a mapping gives the values as they are."""
    if not overrides:
        return {}
    if isinstance(overrides, Mapping):
        assignments = list(overrides.items())
    else:
        assignments = [_assignment(text) for text in overrides]
    overlay: dict[str, Any] = {}
    for dotted, item in assignments:
        path = dotted.split(".")
        table = overlay
        for step in path[:-1]:
            table = table.setdefault(step, {})
        table[path[-1]] = item
    return overlay


def load_file(path: str | Path) -> dict[str, Any]:
    """A configuration table from a ``.toml``, ``.json`` or ``.yaml`` file."""
    path = Path(path)
    kind = path.suffix.lower()
    if kind == ".json":
        return json.loads(path.read_text())
    if kind == ".toml":
        import tomllib

        return tomllib.loads(path.read_text())
    if kind in (".yaml", ".yml"):
        import yaml

        return yaml.safe_load(path.read_text()) or {}
    raise ValueError(f"{path.name}: configuration files are .toml, .json or .yaml")


def resolve_preset(presets: Mapping[str, Mapping[str, Any]], name: str) -> dict[str, Any]:
    """The overlay of preset ``name`` with its ``extends`` ancestry folded in (ancestors first)."""
    chain: list[Mapping[str, Any]] = []
    seen: set[str] = set()
    while name is not None:
        if name not in presets:
            raise ValueError(f"preset {name!r} is not defined; this model has: {', '.join(sorted(presets))}")
        if name in seen:
            raise ValueError(f"preset {name!r} extends itself")
        seen.add(name)
        chain.append(presets[name])
        name = presets[name].get("extends")
    resolved: dict[str, Any] = {}
    for layer in reversed(chain):
        resolved = merge(resolved, {key: item for key, item in layer.items() if key != "extends"})
    return json.loads(json.dumps(resolved))  # detached from the spec's own tables
