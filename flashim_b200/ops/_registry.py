"""Ops and their implementations: declaration, registration and per-call dispatch.

The vocabulary and the selection rule are those of FlashIM's op registry (flashim/ops/_registry.py:44-428), so that an
implementation module written for one registers unchanged into the other: an ``Op`` is declared once by name;
implementations attach with ``op.register(name, device=DeviceSpec(...), requires=[features], priority=n, when=predicate)``;
a call goes to the applicable implementation with the highest priority, ties broken by the narrower compute-capability
range and then by registration order; a negative priority means "only when asked for by name". ``op.get(name)`` pins an
implementation, ``op.explain(*args)`` says per implementation why it was or was not taken, ``configure("-op,op:impl")``
disables or forces by name, and strict mode turns a fall-back on a GPU into an error.

One deliberate difference: FlashIM's last resort is a torch reference implementation; this package ships none. An op
declared without a reference raises :class:`NoImplementation` where FlashIM would have fallen back, so a call can never
silently leave the CUDA path.
"""

from __future__ import annotations

import dataclasses
import os
from collections import Counter
from collections.abc import Callable, Iterable
from dataclasses import dataclass

import torch

from flashim_b200.platforms import Feature, Platform, platform_for

REFERENCE = "reference"
OPS: dict[str, "Op"] = {}


class NoImplementation(RuntimeError):
    """No registered implementation applies to the call and the op has no reference to fall back to."""


# ---- where an implementation runs ------------------------------------------------------------------------------------


@dataclass(frozen=True)
class DeviceSpec:
    """A device type (``"cuda"``, ``"cpu"`` or ``"*"``) and, optionally, an inclusive compute-capability range."""

    type: str
    min_capability: tuple[int, int] | None = None
    max_capability: tuple[int, int] | None = None

    def matches(self, platform: Platform) -> bool:
        if self.type != "*" and self.type != platform.device_type:
            return False
        bounded = self.min_capability is not None or self.max_capability is not None
        if not bounded:
            return True
        have = platform.capability
        if have is None:
            return False
        above = self.min_capability is None or have >= self.min_capability
        below = self.max_capability is None or have <= self.max_capability
        return above and below

    @property
    def span(self) -> float:
        """Width of the capability range in (major * 100 + minor) units; a wildcard device is infinitely wide."""
        if self.type == "*":
            return float("inf")
        low = self.min_capability if self.min_capability is not None else (0, 0)
        high = self.max_capability if self.max_capability is not None else (99, 99)
        return (100 * high[0] + high[1]) - (100 * low[0] + low[1])


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

    @property
    def rank(self) -> tuple:
        """Sort key: better implementations first."""
        return (-self.priority, self.device.span, self.order)

    def available(self, platform: Platform) -> bool:
        return self.device.matches(platform) and platform.supports(*self.requires)

    def accepts(self, args: tuple, kwargs: dict) -> bool:
        return self.when is None or bool(self.when(*args, **kwargs))

    def rejection(self, platform: Platform, args: tuple, kwargs: dict) -> str | None:
        """Why this implementation does not serve the call; ``None`` when it would."""
        if not self.device.matches(platform):
            return f"registered for {self.device}, the call is on {platform.device_type} {platform.arch}".rstrip()
        lacking = sorted(feature.value for feature in self.requires if not platform.supports(feature))
        if lacking:
            return "missing features " + ",".join(lacking)
        if not self.accepts(args, kwargs):
            return "its when() predicate declined these arguments"
        return None


# ---- overrides by name -----------------------------------------------------------------------------------------------


class _Overrides:
    """Process-wide switches: ops whose implementations are all off, ops forced to one implementation, strict mode."""

    def __init__(self) -> None:
        self.off: set[str] = set()
        self.forced: dict[str, str] = {}
        self.strict = False

    def parse(self, text: str | None) -> None:
        off, forced = set(), {}
        for item in (text or "").split(","):
            item = item.strip()
            if item == "" or item[0] == "+":  # "+op" = leave enabled (the default): accepted for symmetry
                continue
            if item[0] == "-":
                off.add(item[1:])
                continue
            op_name, colon, impl_name = item.partition(":")
            if not colon:
                raise ValueError(f"cannot read op override {item!r}: write -op to disable or op:impl to force")
            forced[op_name] = impl_name
        self.off, self.forced = off, forced


_OVERRIDES = _Overrides()


def configure(spec: str | None) -> None:
    """Replace the name overrides: ``"-op"`` turns an op's implementations off, ``"op:impl"`` forces one (``op:reference``
    forces the fall-back), comma-separated. ``None`` or ``""`` clears them."""
    _OVERRIDES.parse(spec)


def set_strict(strict: bool) -> None:
    _OVERRIDES.strict = bool(strict)


configure(os.environ.get("FLASHIM_OPS"))
set_strict(os.environ.get("FLASHIM_STRICT_OPS") == "1")


def _device_of(values: Iterable) -> torch.device | None:
    """The device of the first tensor found in the arguments, looking into sequences and dataclass containers."""
    for value in values:
        if isinstance(value, torch.Tensor):
            return value.device
        if dataclasses.is_dataclass(value) and not isinstance(value, type):
            value = [getattr(value, f.name) for f in dataclasses.fields(value)]
        if isinstance(value, (list, tuple)):
            inner = _device_of(value)
            if inner is not None:
                return inner
    return None


# ---- the op ----------------------------------------------------------------------------------------------------------


class Op:
    def __init__(self, name: str, reference: Callable | None = None, *, doc: str = "") -> None:
        if name in OPS:
            raise ValueError(f"an op named {name!r} is already declared")
        self.name = name
        self.reference = reference
        self.impls: list[Impl] = []
        self.calls: Counter = Counter()
        self.__doc__ = doc or getattr(reference, "__doc__", None)
        OPS[name] = self

    def __repr__(self) -> str:
        return f"Op({self.name}: {', '.join(i.name for i in self.impls) or 'no impls'})"

    # -- registration ------------------------------------------------------------------------------------------------
    def register(self, name: str, *, device: DeviceSpec, requires: Iterable[Feature] = (), priority: int = 0,
                 when: Callable[..., bool] | None = None) -> Callable[[Callable], Callable]:
        if name == REFERENCE or name in {impl.name for impl in self.impls}:
            raise ValueError(f"op {self.name!r} already has an implementation named {name!r}")

        def attach(fn: Callable) -> Callable:
            self.impls.append(Impl(name, fn, device, frozenset(requires), priority, when, order=len(self.impls)))
            return fn

        return attach

    def _named(self, name: str) -> Impl:
        for impl in self.impls:
            if impl.name == name:
                return impl
        raise ValueError(f"op {self.name!r} has no implementation {name!r}; registered: {[i.name for i in self.impls]}")

    # -- selection ---------------------------------------------------------------------------------------------------
    def candidates(self, platform: Platform) -> list[Impl]:
        """Implementations usable on ``platform``, best first (the per-call ``when`` predicates are not consulted)."""
        return sorted((impl for impl in self.impls if impl.available(platform)), key=lambda impl: impl.rank)

    def _platform(self, args: tuple, kwargs: dict) -> Platform:
        device = _device_of(args) or _device_of(kwargs.values()) or torch.device("cpu")
        return platform_for(device)

    def _choose(self, args: tuple, kwargs: dict, pin: str | None = None, strict: bool = True) -> Impl | None:
        """The implementation that serves the call, or ``None`` for the fall-back. Precedence: the name overrides, then a
        pin (``get(name)``), then the ranking."""
        forced = _OVERRIDES.forced.get(self.name)
        if self.name in _OVERRIDES.off or forced == REFERENCE:
            return None
        if forced is not None:
            return self._named(forced)
        if pin == REFERENCE:
            return None
        platform = self._platform(args, kwargs)
        if pin is not None:
            impl = self._named(pin)
            return impl if impl.available(platform) and impl.accepts(args, kwargs) else None
        for impl in self.candidates(platform):
            if not impl.opt_in and impl.accepts(args, kwargs):
                return impl
        if strict and _OVERRIDES.strict and platform.device_type != "cpu":
            raise RuntimeError(f"op {self.name!r}: strict mode, and nothing but the fall-back applies on {platform.describe()}")
        return None

    def supports(self, *args, **kwargs) -> bool:
        return self._choose(args, kwargs, strict=False) is not None

    def select(self, *args, **kwargs) -> tuple[str, Callable | None]:
        impl = self._choose(args, kwargs)
        if impl is None:
            return REFERENCE, self.reference
        return impl.name, impl.fn

    def explain(self, *args, **kwargs) -> dict[str, str]:
        """Per implementation (best first, unavailable ones last): ``"selected"``, the reason it was passed over, or
        ``"outranked"``; plus a ``"reference"`` entry for the fall-back."""
        platform = self._platform(args, kwargs)
        winner = self._choose(args, kwargs, strict=False)
        usable = self.candidates(platform)
        listing = usable + [impl for impl in self.impls if impl not in usable]
        report: dict[str, str] = {}
        for impl in listing:
            if winner is not None and impl.name == winner.name:
                report[impl.name] = "selected"
                continue
            reason = impl.rejection(platform, args, kwargs)
            if reason is None:
                reason = "opt-in (negative priority): ask for it by name" if impl.opt_in else "outranked"
            report[impl.name] = reason
        if winner is not None:
            report[REFERENCE] = "fallback"
        else:
            report[REFERENCE] = "selected" if self.reference is not None else "none shipped: the call raises"
        return report

    # -- calling -----------------------------------------------------------------------------------------------------
    def _run(self, impl: Impl | None, args: tuple, kwargs: dict):
        if impl is not None:
            label, fn = impl.name, impl.fn
        elif self.reference is not None:
            label, fn = REFERENCE, self.reference
        else:
            platform = self._platform(args, kwargs)
            why = "; ".join(f"{i.name}: {i.rejection(platform, args, kwargs) or 'forced off'}" for i in self.impls)
            raise NoImplementation(f"op {self.name!r}: no implementation applies on {platform.describe()} "
                                   f"({why or 'none registered'}) and flashim_b200 ships no fallback")
        if not torch.compiler.is_compiling():
            self.calls[label] += 1
        return fn(*args, **kwargs)

    def __call__(self, *args, **kwargs):
        return self._run(self._choose(args, kwargs), args, kwargs)

    def get(self, name: str | None) -> Callable:
        """The op pinned to one implementation (``None``: the dispatching op itself). A pinned implementation whose
        device or predicate does not fit the call hands over to the fall-back, as in FlashIM."""
        if name is None:
            return self
        if name != REFERENCE:
            self._named(name)  # raise now for a name that does not exist

        def pinned(*args, **kwargs):
            return self._run(self._choose(args, kwargs, pin=name), args, kwargs)

        return pinned


def reset_call_counts() -> None:
    for op in OPS.values():
        op.calls.clear()


def call_counts() -> dict[str, dict[str, int]]:
    """``{op: {implementation: calls}}`` for the ops called since the last reset (calls traced by torch.compile are not
    counted)."""
    return {op.name: dict(op.calls) for op in OPS.values() if sum(op.calls.values())}
