"""Access to a staged copy of the reference's own Python modules -- TEST INFRASTRUCTURE ONLY.

``make -C oracle ref REF=<reference checkout>`` copies the reference's quantiser, registry,
platform gate, op surface (with its torch REFERENCE kernels), ``Linear`` module and kernel
micro-benchmark, unmodified, to ``oracle/_ref/dexter`` (never committed).  Tests use it to
drive this backend through the reference's real plug-in API; the benchmark's reference arm
uses it to time the reference's own CPU path.  The shipped package never imports this module.
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"


def available() -> bool:
    return (REF_DIR / "dexter" / "ops" / "__init__.py").exists()


def stage(reference_root) -> bool:
    """Run the staging recipe if ``reference_root`` holds a reference checkout."""
    root = Path(reference_root)
    if not (root / "python" / "dexter" / "quant.py").exists():
        return False
    subprocess.run(["make", "-C", str(HERE), "ref", f"REF={root}"], check=True, capture_output=True)
    return available()


def activate():
    """Put the staged copy on ``sys.path`` and import the reference's op surface.

    Returns the ``dexter`` modules this path touches.  Importing ``dexter.ops`` registers the
    reference's own kernels (``python/dexter/ops/__init__.py:151-152`` there).
    """
    if not available():
        raise ImportError("no staged reference: run `make -C oracle ref REF=<reference checkout>`")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import dexter.ops as ops
    import dexter.platform as platform
    import dexter.quant as quant
    import dexter.registry as registry

    return {"ops": ops, "platform": platform, "quant": quant, "registry": registry}
