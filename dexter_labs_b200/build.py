"""In-tree build of the CUDA library (``libdexter_b200.so``) for sm_100a.

``python dexter_labs_b200/build.py`` (run as a script, so the package -- which loads the
library on import -- is not imported first) or :func:`build` runs nvcc on
``csrc/*.cu`` and leaves the shared library next to this file, where
:mod:`dexter_labs_b200._lib` loads it.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SOURCES = [PKG_DIR / "csrc" / "wq_gemm.cu", PKG_DIR / "csrc" / "peer_reduce.cu"]
HEADERS = [PKG_DIR / "csrc" / "sm100_ptx.cuh", PKG_DIR / "csrc" / "wq_common.cuh", PKG_DIR.parent / "include" / "dexter_b200.h"]
LIB_PATH = PKG_DIR / "libdexter_b200.so"
# compiled CPython binding of the hot call (csrc/fastcall.c); plain C, no CUDA
FAST_SOURCE = PKG_DIR / "csrc" / "fastcall.c"
FAST_PATH = PKG_DIR / ("_dxb_fast" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(src.stat().st_mtime > built for src in SOURCES + HEADERS if src.exists())


def fast_is_stale() -> bool:
    if not FAST_PATH.exists():
        return True
    built = FAST_PATH.stat().st_mtime
    return any(src.stat().st_mtime > built for src in (FAST_SOURCE, HEADERS[-1]))


def build_fast(force: bool = False) -> Path:
    """Compile the CPython binding of ``dxb_wq_gemm_ex`` (gcc, no CUDA involved)."""
    if not force and not fast_is_stale():
        return FAST_PATH
    cc = os.environ.get("CC") or shutil.which("gcc") or shutil.which("cc")
    if not cc:
        raise RuntimeError("no C compiler found for csrc/fastcall.c; set CC")
    cmd = [cc, "-O2", "-shared", "-fPIC", "-I", sysconfig.get_paths()["include"], str(FAST_SOURCE),
           "-o", str(FAST_PATH)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"{cc} failed ({proc.returncode}): {' '.join(cmd)}")
    return FAST_PATH


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library (and the CPython binding of its hot call) if missing or older
    than the sources."""
    build_fast(force)
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH), *[str(s) for s in SOURCES]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
