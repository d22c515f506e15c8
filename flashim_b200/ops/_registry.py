"""Op declaration and dispatch with the semantics of FlashIM's registry (flashim/ops/_registry.py:44-428): an op is
declared once, implementations register for a device spec + required features + priority + a per-call ``when``
predicate; selection is highest priority, then narrowest capability range, then registration order; ``get(name)`` pins
an implementation, ``explain`` reports why each one was (not) chosen, ``configure`` applies ``FLASHIM_OPS`` overrides
and strict mode forbids falling back.

One deliberate difference: FlashIM's fallback is a torch reference implementation. This package ships none. An op
declared without a reference raises :class:`NoImplementation` where FlashIM would have fallen back, so a call can never
silently leave the CUDA path.
"""

from __future__ import annotations

import os
from collections import Counter
from collections.abc import Callable, Iterable
from dataclasses import dataclass, fields, is_dataclass

import torch

from flashim_b200.platforms import Feature, Platform, platform_for

REFERENCE = "reference"


class NoImplementation(RuntimeError):
    """No registered implementation applies to the call and the op has no reference to fall back to."""


@dataclass(frozen=True)
class DeviceSpec:
    type: str
    min_capability: tuple[int, int] | None = None
    max_capability: tuple[int, int] | None = None

    def matches(self, platform: Platform) -> bool:
        if self.type not in ("*", platform.device_type):
            return False
        if self.min_capability is None and self.max_capability is None:
            return True
        cap = platform.capability
        if cap is None or (self.min_capability is not None and cap < self.min_capability):
            return False
        return self.max_capability is None or cap <= self.max_capability

    @property
    def span(self) -> float:
        if self.type == "*":
            return float("inf")
        lo, hi = self.min_capability or (0, 0), self.max_capability or (99, 99)
        return (hi[0] * 100 + hi[1]) - (lo[0] * 100 + lo[1])


@dataclass
class Impl:
    name: str
    fn: Callable
    device: DeviceSpec
    requires: frozenset = frozenset()
    priority: int = 0
    when: Callable[..., bool] | None = None
    order: int = 0

    @property
    def opt_in(self) -> bool:
        return self.priority < 0

    def available(self, platform: Platform) -> bool:
        return self.device.matches(platform) and platform.supports(*self.requires)

    def rejection(self, platform: Platform, args: tuple, kwargs: dict) -> str | None:
        if not self.device.matches(platform):
            return f"device {self.device} does not match {platform.device_type} {platform.arch}".rstrip()
        missing = sorted(f.value for f in self.requires if not platform.supports(f))
        if missing:
            return "missing features " + ",".join(missing)
        if self.when is not None and not self.when(*args, **kwargs):
            return "when() rejected the arguments"
        return None


class _Config:
    def __init__(self) -> None:
        self.disabled: set[str] = set()
        self.forced: dict[str, str] = {}
        self.strict = False


_CONFIG = _Config()
OPS: dict[str, "Op"] = {}


def configure(spec: str | None) -> None:
    """Apply a ``FLASHIM_OPS``-style string: ``-op`` disables an op's implementations, ``op:impl`` forces one."""
    _CONFIG.disabled.clear()
    _CONFIG.forced.clear()
    for token in (spec or "").split(","):
        token = token.strip()
        if not token or token.startswith("+"):
            continue
        if token.startswith("-"):
            _CONFIG.disabled.add(token[1:])
        elif ":" in token:
            op, impl = token.split(":", 1)
            _CONFIG.forced[op] = impl
        else:
            raise ValueError(f"Invalid FLASHIM_OPS token {token!r}")


def set_strict(strict: bool) -> None:
    _CONFIG.strict = strict


configure(os.environ.get("FLASHIM_OPS"))
set_strict(os.environ.get("FLASHIM_STRICT_OPS", "0") == "1")


def _first_device(values: Iterable) -> torch.device | None:
    for value in values:
        if isinstance(value, torch.Tensor):
            return value.device
        if is_dataclass(value) and not isinstance(value, type):
            value = [getattr(value, f.name) for f in fields(value)]
        if isinstance(value, (list, tuple)):
            found = _first_device(value)
            if found is not None:
                return found
    return None


class Op:
    def __init__(self, name: str, reference: Callable | None = None, *, doc: str = "") -> None:
        if name in OPS:
            raise ValueError(f"Duplicate op {name!r}")
        self.name = name
        self.reference = reference
        self.impls: list[Impl] = []
        self.calls: Counter = Counter()
        self.__doc__ = doc or (reference.__doc__ if reference is not None else None)
        OPS[name] = self

    def register(self, name: str, *, device: DeviceSpec, requires: Iterable[Feature] = (), priority: int = 0,
                 when: Callable[..., bool] | None = None) -> Callable[[Callable], Callable]:
        if name == REFERENCE or any(i.name == name for i in self.impls):
            raise ValueError(f"Duplicate impl {name!r} for op {self.name!r}")

        def decorator(fn: Callable) -> Callable:
            self.impls.append(Impl(name, fn, device, frozenset(requires), priority, when, len(self.impls)))
            return fn

        return decorator

    def candidates(self, platform: Platform) -> list[Impl]:
        usable = [i for i in self.impls if i.available(platform)]
        return sorted(usable, key=lambda i: (-i.priority, i.device.span, i.order))

    def _platform(self, args: tuple, kwargs: dict) -> Platform:
        return platform_for(_first_device(args) or _first_device(kwargs.values()) or torch.device("cpu"))

    def _find(self, name: str) -> Impl:
        for impl in self.impls:
            if impl.name == name:
                return impl
        raise ValueError(f"Op {self.name!r} has no impl {name!r} (registered: {[i.name for i in self.impls]})")

    def _choose(self, args: tuple, kwargs: dict, pin: str | None = None, strict: bool = True) -> Impl | None:
        forced = _CONFIG.forced.get(self.name)
        if forced == REFERENCE or self.name in _CONFIG.disabled:
            return None
        if forced is not None:
            return self._find(forced)
        if pin == REFERENCE:
            return None
        platform = self._platform(args, kwargs)
        for impl in [self._find(pin)] if pin is not None else self.candidates(platform):
            if not impl.available(platform) or (pin is None and impl.opt_in):
                continue
            if impl.when is None or impl.when(*args, **kwargs):
                return impl
        if pin is None and strict and _CONFIG.strict and platform.device_type != "cpu":
            raise RuntimeError(f"Op {self.name!r} fell back to the reference on {platform.describe()}")
        return None

    def supports(self, *args, **kwargs) -> bool:
        return self._choose(args, kwargs, strict=False) is not None

    def select(self, *args, **kwargs) -> tuple[str, Callable | None]:
        impl = self._choose(args, kwargs)
        return (REFERENCE, self.reference) if impl is None else (impl.name, impl.fn)

    def explain(self, *args, **kwargs) -> dict[str, str]:
        platform = self._platform(args, kwargs)
        chosen = self._choose(args, kwargs, strict=False)
        ranked = self.candidates(platform)
        ranked += [i for i in self.impls if i not in ranked]
        report = {}
        for impl in ranked:
            if chosen is not None and impl.name == chosen.name:
                report[impl.name] = "selected"
            else:
                fallback = "opt-in (negative priority): pin it" if impl.opt_in else "lower priority"
                report[impl.name] = impl.rejection(platform, args, kwargs) or fallback
        report[REFERENCE] = ("selected" if self.reference is not None else "none shipped: the call raises") \
            if chosen is None else "fallback"
        return report

    def _run(self, impl: Impl | None, args: tuple, kwargs: dict):
        if impl is None:
            if self.reference is None:
                platform = self._platform(args, kwargs)
                reasons = "; ".join(f"{i.name}: {i.rejection(platform, args, kwargs) or 'forced off'}" for i in self.impls)
                raise NoImplementation(
                    f"op {self.name!r}: no implementation applies on {platform.describe()} ({reasons or 'none registered'}) "
                    "and flashim_b200 ships no fallback"
                )
            name, fn = REFERENCE, self.reference
        else:
            name, fn = impl.name, impl.fn
        if not torch.compiler.is_compiling():
            self.calls[name] += 1
        return fn(*args, **kwargs)

    def __call__(self, *args, **kwargs):
        return self._run(self._choose(args, kwargs), args, kwargs)

    def get(self, name: str | None) -> Callable:
        if name is None:
            return self
        if name != REFERENCE:
            self._find(name)

        def pinned(*args, **kwargs):
            return self._run(self._choose(args, kwargs, pin=name), args, kwargs)

        return pinned

    def __repr__(self) -> str:
        return f"Op({self.name}: {', '.join(i.name for i in self.impls) or 'no impls'})"


def reset_call_counts() -> None:
    for op in OPS.values():
        op.calls.clear()


def call_counts() -> dict[str, dict[str, int]]:
    return {name: dict(op.calls) for name, op in OPS.items() if op.calls}
