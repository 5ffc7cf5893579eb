"""Weight-only quantiser producing the packed layout the GEMM kernel consumes.

Host-side mirror of the reference's offline quantiser
(``python/dexter/quant.py:34-133`` in the reference): same names, arguments,
error behaviour and -- checked bit for bit against vectors the reference
produced (``tests/golden``) -- the same bytes.  When the reference itself is
importable its own ``dexter.quant.quantize`` can be used instead; the kernel
does not care which of the two packed the weight.

Layout (``quant.py:34-72`` in the reference):

* 4 bit: ``qweight`` is ``[K // 2, N]`` uint8; byte ``[i, n]`` has logical row
  ``i`` in its low nibble and row ``i + K // 2`` in its high nibble.
* 8 bit: ``qweight`` is ``[K, N]`` uint8.
* ``scales`` / ``zeros`` are ``[K // group_size, N]`` in the weight's dtype;
  ``zeros`` is ``None`` for the symmetric grid; 4-bit zero points carry
  ``+128`` (``BF16_MAGIC_BIAS``).

A stand-in: it is used only where the reference project is not importable (a machine that has
this package alone).  Where the reference is present its own module is the one in charge --
``ops.register_with`` plugs the kernels into it -- and the tests drive that one
(``tests/test_reference_api.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

__all__ = ["QuantizedWeight", "quantize", "pack_nibbles", "DEFAULT_GROUP_SIZE", "BF16_MAGIC_BIAS"]

DEFAULT_GROUP_SIZE = 128
BF16_MAGIC_BIAS = 128.0


@dataclass
class QuantizedWeight:
    """Packed weight + what is needed to dequantise it (``quant.py:34-59``)."""

    qweight: torch.Tensor
    scales: torch.Tensor
    zeros: Optional[torch.Tensor]
    bias: Optional[torch.Tensor]
    group_size: int
    bits: int
    shape: Tuple[int, int]  # logical (K, N)

    @property
    def nbytes(self) -> int:
        """Bytes the GEMM has to stream: packed values, scales and zero points."""
        parts = [self.qweight, self.scales] + ([] if self.zeros is None else [self.zeros])
        return sum(t.numel() * t.element_size() for t in parts)

    def to(self, device) -> "QuantizedWeight":
        def mv(t):
            return t if t is None else t.to(device)
        return QuantizedWeight(mv(self.qweight), mv(self.scales), mv(self.zeros), mv(self.bias),
                               self.group_size, self.bits, self.shape)


def pack_nibbles(q: torch.Tensor) -> torch.Tensor:
    """``[K, N]`` values 0..15 -> ``[K // 2, N]`` bytes, split-half (``quant.py:62-72``)."""
    k = q.shape[0]
    lower, upper = q[: k // 2], q[k // 2:]
    return torch.bitwise_or(lower, torch.bitwise_left_shift(upper, 4)).contiguous()


def quantize(weight: torch.Tensor, *, bits: int = 4, group_size: int = DEFAULT_GROUP_SIZE,
             bias: Optional[torch.Tensor] = None, symmetric: bool = False) -> QuantizedWeight:
    """Quantise an ``[N, K]`` (``nn.Linear``-style) weight (``quant.py:75-133``).

    All arithmetic is fp32 in the reference's order: the quantised values are
    computed with the fp32 scale, and only afterwards is the scale rounded to
    the weight's dtype.
    """
    if weight.ndim != 2:
        raise ValueError(f"expected a 2D weight, got shape {tuple(weight.shape)}")
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits}")
    n_out, k_in = weight.shape
    if k_in % group_size:
        raise ValueError(f"K={k_in} must be a multiple of group_size={group_size}")

    levels = float(2 ** bits - 1)
    grouped = weight.t().contiguous().float().view(k_in // group_size, group_size, n_out)

    if symmetric:
        peak = grouped.abs().amax(dim=1).clamp(min=1e-8)
        scale = 2 * peak / levels
        zero_pt = None
        shift = float(2 ** (bits - 1))
    else:
        low = grouped.amin(dim=1)
        high = grouped.amax(dim=1)
        scale = ((high - low) / levels).clamp(min=1e-8)
        zero_pt = (-low / scale).round().clamp(0, levels)
        shift = zero_pt.unsqueeze(1)

    codes = (grouped / scale.unsqueeze(1) + shift).round().clamp(0, levels)
    codes = codes.view(k_in, n_out).to(torch.uint8)

    if zero_pt is not None and bits == 4:
        zero_pt = zero_pt + BF16_MAGIC_BIAS  # the kernel's nibble pattern is 128 + q

    store = weight.dtype if weight.dtype.is_floating_point else torch.bfloat16
    return QuantizedWeight(
        qweight=pack_nibbles(codes) if bits == 4 else codes.contiguous(),
        scales=scale.to(store).contiguous(),
        zeros=None if zero_pt is None else zero_pt.to(store).contiguous(),
        bias=bias,
        group_size=group_size,
        bits=bits,
        shape=(k_in, n_out),
    )
