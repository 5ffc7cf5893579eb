"""Shared fixtures: the `gpu` marker, the golden cases, and the built libraries."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden" / "wq_cases.npz"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # GPU tests are skipped, not failed, where no device exists, so a plain `pytest` works.
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Case:
    """One golden case: inputs and reference outputs as numpy bit patterns."""

    def __init__(self, name: str, data) -> None:
        self.name = name
        m, k, n, bits, group, sym, with_bias, seed = (int(v) for v in data[f"{name}/meta"])
        self.m, self.k, self.n, self.bits, self.group = m, k, n, bits, group
        self.symmetric, self.seed = bool(sym), seed
        get = lambda key: data[f"{name}/{key}"] if f"{name}/{key}" in data.files else None  # noqa: E731
        self.x, self.w = get("x"), get("w")
        self.qweight, self.scales, self.zeros, self.bias = (get("qweight"), get("scales"),
                                                            get("zeros"), get("bias"))
        self.unpacked, self.dense, self.y = get("unpacked"), get("dense"), get("y")
        self.nbytes = int(data[f"{name}/nbytes"])

    def __repr__(self) -> str:
        return f"Case({self.name})"


def _load_cases():
    data = np.load(GOLDEN)
    return [Case(str(name), data) for name in data["case_names"]]


CASES = _load_cases()


@pytest.fixture(scope="session")
def golden_cases():
    return CASES


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle module with its C library built."""
    from oracle import wq_oracle

    wq_oracle.build()
    return wq_oracle


@pytest.fixture(scope="session")
def b200_lib():
    """Build (if stale) and load the CUDA library; needs nvcc but no GPU."""
    import importlib.util

    # by path: importing the package would load the (possibly stale) library first
    spec = importlib.util.spec_from_file_location("_dxb_build", ROOT / "dexter_labs_b200" / "build.py")
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    b.build()
    from dexter_labs_b200 import _lib

    return _lib.load()
