"""What kernel selection may depend on: vendor, architecture, feature set.

Host-side mirror of the part of the reference's ``python/dexter/platform.py``
that the quantised-GEMM path touches (``Capability`` :169-185, ``PlatformInfo``
:129-166, NVIDIA / CPU detection :224-264, ``current_platform`` /
``override_platform`` :267-278), so the backend registers and is selected the
same way with or without the reference installed.

A stand-in: it is used only where the reference project is not importable (a machine that has
this package alone).  Where the reference is present its own module is the one in charge --
``ops.register_with`` plugs the kernels into it -- and the tests drive that one
(``tests/test_reference_api.py``).
"""
from __future__ import annotations

import functools
import os
from dataclasses import dataclass, field
from typing import FrozenSet, NamedTuple, Optional

__all__ = ["ArchVersion", "PlatformInfo", "Capability", "current_platform", "override_platform"]


class ArchVersion(NamedTuple):
    """(major, minor), ordered like a tuple: ``ArchVersion(10, 0)`` is sm_100."""

    major: int
    minor: int = 0


@dataclass(frozen=True)
class PlatformInfo:
    vendor: str           # "nvidia" | "amd" | "cpu"
    arch: str             # "sm100", "cpu", ...
    arch_version: ArchVersion
    family: str
    device_name: str
    compute_units: int
    wavefront: int
    lds_bytes: int
    total_memory: int
    memory_bandwidth: float
    features: FrozenSet[str] = field(default_factory=frozenset)

    def supports(self, *wanted: str) -> bool:
        return set(wanted) <= self.features

    def describe(self) -> str:
        return (f"{self.device_name} [{self.arch} / {self.family}] {self.compute_units} CU, "
                f"wave{self.wavefront}, {self.total_memory / 1e9:.1f} GB @ "
                f"{self.memory_bandwidth:.0f} GB/s")


@dataclass(frozen=True)
class Capability:
    """Requirements a kernel places on the platform; all must hold."""

    vendors: Optional[FrozenSet[str]] = None
    min_arch: Optional[ArchVersion] = None
    max_arch: Optional[ArchVersion] = None
    features: FrozenSet[str] = field(default_factory=frozenset)

    def satisfied_by(self, platform: PlatformInfo) -> bool:
        checks = (
            self.vendors is None or platform.vendor in self.vendors,
            self.min_arch is None or tuple(platform.arch_version) >= tuple(self.min_arch),
            self.max_arch is None or tuple(platform.arch_version) <= tuple(self.max_arch),
            self.features <= platform.features,
        )
        return all(checks)


def _cpu_platform() -> PlatformInfo:
    return PlatformInfo("cpu", "cpu", ArchVersion(0, 0), "CPU", "cpu", os.cpu_count() or 1, 1, 0,
                        0, 0.0, frozenset())


@functools.lru_cache(maxsize=1)
def _probe() -> PlatformInfo:
    import torch

    if not torch.cuda.is_available() or getattr(torch.version, "hip", None):
        return _cpu_platform()
    props = torch.cuda.get_device_properties(torch.cuda.current_device())
    return PlatformInfo(
        vendor="nvidia",
        arch=f"sm{props.major}{props.minor}",
        arch_version=ArchVersion(props.major, props.minor),
        family="NVIDIA",
        device_name=props.name,
        compute_units=props.multi_processor_count,
        wavefront=32,
        lds_bytes=props.shared_memory_per_block,
        total_memory=props.total_memory,
        memory_bandwidth=0.0,
        features=frozenset({"matrix:f16", "matrix:bf16", "mma:mma"}),
    )


_forced: Optional[PlatformInfo] = None


def current_platform() -> PlatformInfo:
    return _forced if _forced is not None else _probe()


def override_platform(platform: Optional[PlatformInfo]) -> None:
    """Pin the platform (tests, gate checks); ``None`` returns to detection."""
    global _forced
    _forced = platform
