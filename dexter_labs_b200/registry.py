"""Kernel registry: many implementations per ``family/mode``, best viable one wins.

Host-side mirror of the reference's ``python/dexter/registry.py`` (``Priority``
:34-48, ``KernelSpec`` :51-67, ``register`` :73-104, ``candidates`` :107-112,
``DEXTER_KERNEL`` pin :115-125, ``select`` :128-152, ``explain`` :155-173) with
the same names and rules:

* capability gates are checked before priority;
* buckets are kept sorted by priority, highest first;
* ``accepts(*shape_args)`` lets a kernel decline a call (it is also called with
  no arguments by benchmarks, and must then answer for the general case);
* ``DEXTER_KERNEL=gemm/w4a16:<name>`` pins one implementation.

A stand-in: it is used only where the reference project is not importable (a machine that has
this package alone).  Where the reference is present its own module is the one in charge --
``ops.register_with`` plugs the kernels into it -- and the tests drive that one
(``tests/test_reference_api.py``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Callable, Dict, Iterator, List, Optional, Union

from .platform import Capability, PlatformInfo, current_platform

__all__ = ["Priority", "KernelSpec", "register", "select", "candidates", "explain"]


class Priority(IntEnum):
    REFERENCE = 0
    PORTABLE = 4
    PERFORMANT = 8
    SPECIALISED = 12


@dataclass(frozen=True)
class KernelSpec:
    name: str
    family: str
    mode: str
    impl: Callable
    capability: Capability = field(default_factory=Capability)
    priority: Union[Priority, int] = Priority.PERFORMANT
    accepts: Optional[Callable[..., bool]] = None

    @property
    def key(self) -> str:
        return f"{self.family}/{self.mode}"


_REGISTRY: Dict[str, List[KernelSpec]] = {}


def register(family: str, mode: str, *, name: str, capability: Optional[Capability] = None,
             priority: Union[Priority, int] = Priority.PERFORMANT,
             accepts: Optional[Callable[..., bool]] = None) -> Callable[[Callable], Callable]:
    """Decorator: add ``fn`` as implementation ``name`` of ``family/mode``."""

    def wrap(fn: Callable) -> Callable:
        spec = KernelSpec(name, family, mode, fn, capability or Capability(), priority, accepts)
        bucket = _REGISTRY.setdefault(spec.key, [])
        if name in (s.name for s in bucket):
            raise ValueError(f"duplicate kernel {spec.key}:{name}")
        bucket.append(spec)
        bucket.sort(key=lambda s: -int(s.priority))  # stable: ties keep registration order
        fn.dexter_spec = spec
        return fn

    return wrap


def candidates(family: str, mode: str,
               platform: Optional[PlatformInfo] = None) -> Iterator[KernelSpec]:
    platform = platform or current_platform()
    return (s for s in _REGISTRY.get(f"{family}/{mode}", []) if s.capability.satisfied_by(platform))


def _pin_for(key: str) -> Optional[str]:
    for item in os.environ.get("DEXTER_KERNEL", "").split(","):
        left, _, right = item.strip().partition(":")
        if left == key and item.strip():
            return right
    return None


def select(family: str, mode: str, *args, **kwargs) -> Callable:
    """Implementation to call for this platform and call shape."""
    key = f"{family}/{mode}"
    viable = list(candidates(family, mode))
    pin = _pin_for(key)
    if pin is not None:
        for spec in viable:
            if spec.name == pin:
                return spec.impl
        raise LookupError(f"DEXTER_KERNEL pinned {key}:{pin}, which is not available here")
    for spec in viable:
        if spec.accepts is None or spec.accepts(*args, **kwargs):
            return spec.impl
    names = [s.name for s in _REGISTRY.get(key, [])] or "none"
    raise LookupError(f"no kernel for {key} on {current_platform().describe()}. Registered: {names}")


def explain(family: str, mode: str, *args, **kwargs) -> str:
    """One line per registered kernel saying why it was or was not picked."""
    key = f"{family}/{mode}"
    platform = current_platform()
    out = [f"{key} on {platform.describe()}"]
    picked = False
    for spec in _REGISTRY.get(key, []):
        if not spec.capability.satisfied_by(platform):
            lacking = sorted(spec.capability.features - platform.features)
            why = f"needs {lacking}" if lacking else "arch gate"
            out.append(f"  - {spec.name:<28} skipped ({why})")
        elif spec.accepts is not None and not spec.accepts(*args, **kwargs):
            out.append(f"  - {spec.name:<28} skipped (shape not accepted)")
        elif not picked:
            picked = True
            out.append(f"  * {spec.name:<28} SELECTED (pri={int(spec.priority)})")
        else:
            out.append(f"  - {spec.name:<28} viable (pri={int(spec.priority)})")
    return "\n".join(out)
