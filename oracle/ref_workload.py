"""The benchmark's workload on the host cores -- TEST INFRASTRUCTURE ONLY.

One block of the backbone's linear set (self q, k, v, o; cross q, k, v, o; FFN up, down; shapes
from ``python/dexter/models/dreamzero/config.py:182-219`` and ``model.py:148-151,204-207,260-261``
of the reference), int4 group 128 symmetric with bias, run on CPU tensors

* through the reference's OWN code when a staged copy is present (``oracle/ref.py``): its
  quantiser ``dexter.quant.quantize`` and its op surface ``dexter.ops.linear``, which selects
  the registered REFERENCE kernel ``torch_w4a16`` (``python/dexter/ops/reference/gemm.py:82-89``)
  -- kind "reference";
* else through the torch restatement in ``oracle/wq_oracle.py`` -- kind "port".

Weights follow the seeds of the GPU arm's layer set (``seed + 1000 * block + index``, weights
N(0, 0.02), bias N(0, 0.1)), so both arms compute the same linears.  Nothing here imports the
shipped package, so the timed process never loads its CUDA library.
"""
from __future__ import annotations

import os
import statistics
import time
from typing import Callable, List, Tuple

import torch

# name -> (dim, ffn_dim, blocks)
PRESETS = {"5b": (3072, 14336, 30), "14b": (5120, 13824, 40)}
# (name, K from, N): the ten linears of one block in execution order
BLOCK_PLAN = (("self_q", "dim", "dim"), ("self_k", "dim", "dim"), ("self_v", "dim", "dim"),
              ("self_o", "dim", "dim"), ("cross_q", "dim", "dim"), ("cross_k", "dim", "dim"),
              ("cross_v", "dim", "dim"), ("cross_o", "dim", "dim"), ("ffn_up", "dim", "ffn"),
              ("ffn_down", "ffn", "dim"))


def use_all_host_threads() -> int:
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the reference arm is
    meant to use every host core it can, whatever launched it."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(n, 1))
    return torch.get_num_threads()


def _port_quantize(w: torch.Tensor, bias, bits: int, group: int):
    """Symmetric grid of the reference quantiser (quant.py:94-129), restated; returns a tuple
    shaped like the reference's QuantizedWeight fields."""
    wt = w.t().float()
    k, n = wt.shape
    grp = wt.reshape(k // group, group, n)
    qmax = float((1 << bits) - 1)
    amax = grp.abs().amax(dim=1).clamp_min(1e-8)
    scale = 2.0 * amax / qmax
    q = torch.round(grp / scale.unsqueeze(1) + float(1 << (bits - 1))).clamp_(0, qmax)
    q = q.reshape(k, n).to(torch.uint8)
    if bits == 4:
        q = q[: k // 2] | (q[k // 2:] << 4)
    return q.contiguous(), scale.to(w.dtype), None, bias


def build_block(preset: str, block: int = 0, seed: int = 0, bits: int = 4, group: int = 128):
    """The ten packed linears of one block and the callable that runs one of them.

    Returns ``(kind, linears, run)``: ``linears`` is a list of ``(name, packed)`` and
    ``run(x, packed)`` the quantised linear on CPU tensors.
    """
    from . import ref

    dim, ffn, _ = PRESETS[preset]
    sizes = {"dim": dim, "ffn": ffn}
    if ref.available():
        mods = ref.activate()
        kind = "reference"

        def quantise(w, b):
            return mods["quant"].quantize(w, bits=bits, group_size=group, bias=b, symmetric=True)

        def run(x, p):
            return mods["ops"].linear(x, p.qweight, p.bias, scales=p.scales, zeros=p.zeros,
                                      group_size=p.group_size, bits=p.bits)
    else:
        from . import wq_oracle

        kind = "port"

        def quantise(w, b):
            return _port_quantize(w, b, bits, group)

        def run(x, p):
            return wq_oracle.torch_wq_gemm(x, p[0], p[1], p[2], p[3], group, bits)

    linears: List[Tuple[str, object]] = []
    for idx, (name, src, dst) in enumerate(BLOCK_PLAN):
        k, n = sizes[src], sizes[dst]
        gen = torch.Generator(device="cpu").manual_seed(seed + 1000 * block + idx)
        w = (torch.randn(n, k, generator=gen) * 0.02).to(torch.bfloat16)
        b = (torch.randn(n, generator=gen) * 0.1).to(torch.bfloat16)
        linears.append((name, quantise(w, b)))
    return kind, linears, run


def block_forward(linears, run: Callable, x: torch.Tensor, ctx: torch.Tensor) -> torch.Tensor:
    """Same order and data flow as the GPU arm's block: the v projections stand in for the
    attention outputs that feed the o projections."""
    p = dict(linears)
    run(x, p["self_q"])
    run(x, p["self_k"])
    v = run(x, p["self_v"])
    x = run(v, p["self_o"])
    run(x, p["cross_q"])
    run(ctx, p["cross_k"])
    cv = run(ctx, p["cross_v"])
    x = run(cv, p["cross_o"])
    h = run(x, p["ffn_up"])
    return run(h, p["ffn_down"])


def time_block(preset: str, tokens: int, reps: int, warmup: int = 1):
    """Median milliseconds of one block on the host cores: ``(ms, threads, kind)``."""
    threads = use_all_host_threads()
    kind, linears, run = build_block(preset)
    dim = PRESETS[preset][0]
    torch.manual_seed(0)
    x = torch.randn(tokens, dim).to(torch.bfloat16)
    ctx = torch.randn(tokens, dim).to(torch.bfloat16)
    for _ in range(max(warmup, 1)):
        block_forward(linears, run, x, ctx)
    times = []
    for _ in range(max(reps, 1)):
        t0 = time.perf_counter()
        block_forward(linears, run, x, ctx)
        times.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(times), threads, kind
