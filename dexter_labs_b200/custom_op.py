"""The quantised GEMM as a ``torch.library`` custom op: ``torch.ops.dexter_b200.wq_gemm``.

The registered kernels (``ops.w4a16`` / ``ops.w8a16``) call the C ABI directly through
ctypes, which is all eager execution and CUDA-graph capture need
(``python/dexter/runtime/graph.py:70-72`` in the reference captures the step that way).
``torch.compile`` and other dispatcher-level tooling cannot see a ctypes call, so the same
computation is also declared to the dispatcher, with a shape-only implementation for
tracing; the registered kernels switch to it by themselves while a graph is being compiled.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

__all__ = ["wq_gemm"]


@torch.library.custom_op("dexter_b200::wq_gemm", mutates_args=(), device_types="cuda")
def wq_gemm(x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor],
            bias: Optional[torch.Tensor], group_size: int, bits: int) -> torch.Tensor:
    """``x @ dequant(qweight) (+ bias)``: the kernel slot of the reference
    (``python/dexter/ops/reference/gemm.py:82-89``) with the bit width as an argument."""
    return ops._run(bits, x, qweight, scales, zeros, bias, group_size)


@wq_gemm.register_fake
def _wq_gemm_shape(x, qweight, scales, zeros, bias, group_size, bits):
    k_dim = qweight.shape[0] * (2 if bits == 4 else 1)
    torch._check(x.shape[-1] == k_dim, lambda: f"x has K={x.shape[-1]} but the packed weight has K={k_dim}")
    return x.new_empty((*x.shape[:-1], qweight.shape[1]))
