"""ctypes binding of ``libdexter_b200.so`` (declarations: ``include/dexter_b200.h``).

There is no fallback: if the library is missing the import fails with the build
command, and no op in this package computes anything without it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import os

# the in-tree build, unless DEXTER_B200_LIBRARY names another build of the same library
# (e.g. one compiled with -DDXB_TRACE for in-kernel time stamps)
LIB_PATH = Path(os.environ.get("DEXTER_B200_LIBRARY") or Path(__file__).resolve().parent / "libdexter_b200.so")

OK = 0
ERRORS = {
    -1: "DXB_ERR_BITS", -2: "DXB_ERR_NULL", -3: "DXB_ERR_SHAPE", -4: "DXB_ERR_UNSUPPORTED",
    -5: "DXB_ERR_WORKSPACE", -6: "DXB_ERR_TENSORMAP", -7: "DXB_ERR_CUDA",
    -8: "DXB_ERR_KERNEL_TIMEOUT", -9: "DXB_ERR_SCRATCH_LIMIT",
}

LAYOUT_DEXTER, LAYOUT_B200 = 0, 1
EPILOGUE_NONE, EPILOGUE_GELU_TANH = 0, 1


class GemmOpts(ctypes.Structure):
    """``dxb_gemm_opts`` of include/dexter_b200.h."""
    _fields_ = [("weight_layout", c_int), ("epilogue", c_int), ("max_ctas", c_int),
                ("peer_world", c_int), ("peer_rank", c_int),
                ("peer_regions", ctypes.POINTER(c_void_p)), ("peer_capacity_elems", c_int64),
                ("serialize", c_int)]


# name -> (restype, argtypes); one entry per symbol declared in include/dexter_b200.h
SIGNATURES = {
    "dxb_wq_gemm_ex": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                               ctypes.POINTER(GemmOpts), c_void_p]),
    "dxb_fused_reduce_bytes": (c_size_t, [c_int, c_int64]),
    "dxb_relayout_w4": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "dxb_workspace_bytes_ex": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "dxb_dequantize_ex": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p]),
    "dxb_set_wait_limit_ms": (None, [c_int]),
    "dxb_peer_allreduce_bytes": (c_size_t, [c_int, c_int64]),
    "dxb_peer_allreduce": (c_int, [c_void_p, c_void_p, c_int64, ctypes.POINTER(c_void_p), c_int64,
                                   c_int, c_int, c_void_p, c_void_p]),
    "dxb_wq_gemm": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                            c_int, c_void_p]),
    "dxb_wq_gemm_static": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "dxb_w4a16": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_int64, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "dxb_w8a16": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_int64, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "dxb_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "dxb_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_void_p]),
    "dxb_uses_tensor_cores": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "dxb_read_status": (c_int, [c_void_p, c_void_p]),
    "dxb_strerror": (c_char_p, [c_int]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once; raise loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python dexter_labs_b200/build.py` "
            "(needs nvcc; there is no non-CUDA fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def load_fast():
    """``_dxb_fast.gemm`` bound to this library's ``dxb_wq_gemm_ex``, or None when the compiled
    binding has not been built (the ctypes path then serves every call)."""
    lib = load()
    try:
        from . import _dxb_fast
    except ImportError:
        return None
    _dxb_fast.bind(ctypes.cast(lib.dxb_wq_gemm_ex, ctypes.c_void_p).value)
    return _dxb_fast.gemm


def strerror(code: int) -> str:
    return load().dxb_strerror(code).decode()
