"""Generate golden vectors for the weight-only quantised GEMM path FROM THE REFERENCE.

Run once, where the reference project is available:

    PYTHONPATH=<reference>/python python tests/golden/make_golden.py

It imports the reference's own quantiser (``dexter.quant.quantize``), its torch
dequantise (``dexter.ops.reference.gemm.dequantize``) and its registered
REFERENCE kernels (``torch_w4a16`` / ``torch_w8a16`` through ``dexter.ops.linear``)
and stores, per case, the seeded inputs and every output as raw bit patterns in
``tests/golden/wq_cases.npz``.  The tests never import the reference; they only
read that file.  torch version used is recorded in the file.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

import dexter.ops as dexter_ops
from dexter.ops.reference.gemm import dequantize, unpack_int4
from dexter.quant import quantize

OUT = Path(__file__).resolve().parent / "wq_cases.npz"

# (name, M, K, N, bits, group_size (0 = per-channel, i.e. K), symmetric, bias, seed, x_scale, w_scale)
CASES = [
    ("w4_sym_g128", 5, 512, 144, 4, 128, True, False, 0, 1.0, 0.02),
    ("w4_asym_g128_bias", 7, 256, 160, 4, 128, False, True, 1, 1.0, 0.02),
    ("w4_sym_g64", 3, 256, 128, 4, 64, True, False, 2, 1.0, 0.02),
    ("w4_asym_g32", 4, 128, 144, 4, 32, False, False, 3, 0.1, 0.05),
    ("w4_linear_256x128", 8, 256, 128, 4, 128, False, False, 4, 1.0, 256 ** -0.5),
    ("w8_sym_perchannel", 6, 384, 112, 8, 0, True, False, 5, 1.0, 0.02),
    ("w8_asym_g128_bias", 9, 256, 128, 8, 128, False, True, 6, 1.0, 0.02),
    ("w8_sym_g128", 2, 256, 96, 8, 128, True, False, 7, 0.1, 0.05),
    ("w4_sym_g128_ragged_n", 5, 256, 200, 4, 128, True, False, 8, 1.0, 0.02),
    ("w4_sym_m1", 1, 1024, 64, 4, 128, True, True, 9, 1.0, 0.02),
]


# cases whose unquantised weight is stored too (one per bits x symmetric combination)
KEEP_WEIGHT = {"w4_sym_g128", "w4_asym_g128_bias", "w8_sym_perchannel", "w8_asym_g128_bias"}


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main() -> int:
    store = {"torch_version": np.array(torch.__version__), "case_names": np.array([c[0] for c in CASES])}
    for name, m, k, n, bits, group, sym, with_bias, seed, xs, wsc in CASES:
        torch.manual_seed(seed)
        g = group or k
        x = (torch.randn(m, k) * xs).to(torch.bfloat16)
        w = (torch.randn(n, k) * wsc).to(torch.bfloat16)
        bias = torch.randn(n).to(torch.bfloat16) if with_bias else None
        qw = quantize(w, bits=bits, group_size=g, bias=bias, symmetric=sym)
        dense = dequantize(qw.qweight, qw.scales, qw.zeros, g, bits)
        y = dexter_ops.linear(x, qw.qweight, qw.bias, scales=qw.scales, zeros=qw.zeros,
                              group_size=g, bits=bits)
        store[f"{name}/meta"] = np.array([m, k, n, bits, g, int(sym), int(with_bias), seed])
        store[f"{name}/x"] = bits16(x)
        if name in KEEP_WEIGHT:
            store[f"{name}/w"] = bits16(w)  # pins the quantiser itself
        store[f"{name}/qweight"] = qw.qweight.numpy().copy()
        store[f"{name}/scales"] = bits16(qw.scales)
        if qw.zeros is not None:
            store[f"{name}/zeros"] = bits16(qw.zeros)
        if bias is not None:
            store[f"{name}/bias"] = bits16(bias)
        if bits == 4:
            store[f"{name}/unpacked"] = unpack_int4(qw.qweight).numpy().copy()
        store[f"{name}/dense"] = bits16(dense)
        store[f"{name}/y"] = bits16(y)
        store[f"{name}/nbytes"] = np.array(qw.nbytes)
    np.savez_compressed(OUT, **store)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(CASES)} cases)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
