#!/usr/bin/env python3
"""Benchmark of the B200 weight-only quantised GEMM backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (all N): the linear-layer set of the 5B backbone -- 30 blocks x 10 int4
(group 128, symmetric, bias) linears at M = 83 tokens, 300 GEMMs and 2.53 GB of
packed weights per pass, which contains the headline shape M=83, K=3072, N=14336
(FFN-up) 30 times.  One "step" is one pass over the set.  With N > 1 the set is
tensor-parallel (column shards for q/k/v/up, row shards for o/down, the sum over ranks
after each row-parallel linear inside that linear's launch), so scaling is strong.
The headline single GEMM is timed as well (16 rotating weight buffers, 363 MB, so
L2 cannot hold them) and reported under "gemm".

Prints ONE JSON line on rank 0.  `--impl reference` times the reference's own CPU
path (its quantiser and `dexter.ops.linear` from the staged copy under oracle/_ref when
present, else the torch restatement in oracle/) on the host cores for the same metric,
without importing this repository's package; it is the one place besides the
cpu_baseline leg where this file touches oracle/.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# The workload: the 5B layer set at 83 tokens unless `--workload 14b` (the 14B-shaped
# set at 913 tokens, the compute-bound regime) is asked for; main() sets these three.
M_TOKENS = 83
PRESET = "5b"
METRIC = "w4a16_5b_layer_set_ms"
WORKLOADS = {"5b": (83, "w4a16_5b_layer_set_ms"), "14b": (913, "w4a16_14b_layer_set_ms")}
# name -> (dim, ffn_dim, blocks): python/dexter/models/dreamzero/config.py:182-219 of the reference
PRESETS = {"5b": (3072, 14336, 30), "14b": (5120, 13824, 40)}
# DRAM bytes / algorithmic bytes of one wq_gemm_tc launch of the headline shape, from one ncu
# capture (23.27 MB read for 22.71 MB of packed weights + scales); the bench line's
# roofline.traffic is the algorithmic figure scaled by it, not a per-run measurement
DRAM_OVER_ALGORITHMIC = 1.025


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"],
                "tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxes, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxes.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "reasons": sorted(reasons),
                "samples": len(clocks)}


# --------------------------------------------------------------- reference arm
def cpu_block_ms(reps: int, warmup: int = 1):
    """The reference's CPU path on the host cores: one block of the set, median ms."""
    from oracle import ref_workload

    return ref_workload.time_block(PRESET, M_TOKENS, reps, warmup)


def cpu_baseline_entry(per_block_ms: float, threads: int, kind: str, reps: int) -> dict:
    blocks = PRESETS[PRESET][2]
    how = ("the reference's own quantiser and dexter.ops.linear -> torch_w4a16 (staged copy)" if kind == "reference"
           else "torch restatement of the reference's op sequence (dequantise whole weight, matmul, bias)")
    return {"value": per_block_ms * blocks, "unit": "ms", "cores": threads, "kind": kind,
            "sample": f"one block (10 of {10 * blocks} GEMMs), median of {reps}, x{blocks}; {how} on CPU tensors"}


def run_reference(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # each step: one block's ten GEMMs (a bounded sample), scaled to the blocks of a pass
    per_block_ms, threads, kind = cpu_block_ms(max(args.steps, 1), max(args.warmup, 1))
    value = per_block_ms * PRESETS[PRESET][2]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "ms", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": value, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus, args.collective),
        "cpu_baseline": cpu_baseline_entry(per_block_ms, threads, kind, max(args.steps, 1)),
        "e2e": {"value": value, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


COLLECTIVES = {"fused": "the sum over ranks is part of each row-parallel linear's launch (peer stores over NVLink "
                        "from the GEMM epilogue)",
               "peer": "one all-reduce kernel of this library over NVLink peer memory after each row-parallel "
                       "linear",
               "all_reduce": "one NCCL all-reduce after each row-parallel linear",
               "rs_ag": "NCCL reduce-scatter + all-gather after each row-parallel linear"}


def workload_config(n_gpus: int, collective: str = "fused") -> dict:
    dim, ffn, blocks = PRESETS[PRESET]
    set_gb = blocks * (8 * dim * dim + 2 * dim * ffn) * (0.5 + 2.0 / 128) / 1e9
    return {"workload": f"{PRESET.upper()} backbone linear set: {blocks} blocks x (self q,k,v,o; cross q,k,v,o; "
                        f"ffn up,down), int4 group 128 symmetric + bias, M={M_TOKENS}, seeded random weights",
            "gemms_per_step": (10 if n_gpus == 1 else 7) * blocks,
            "schedule": ("per block: self q,k,v and cross k,v on parallel streams, then o, cross q, cross o, "
                         "up, down; one CUDA graph per pass") if n_gpus == 1 else
                        ("per block: self q,k,v as one launch, o with its sum over ranks beside cross k,v as one "
                         "launch on a side stream, cross q, cross o, up, down; one CUDA graph per pass"),
            "tokens": M_TOKENS, "dim": dim, "ffn_dim": ffn,
            "parallelism": f"tp{n_gpus}" if n_gpus > 1 else "single",
            "collectives": COLLECTIVES[collective] if n_gpus > 1 else "none",
            "l2": f"{set_gb:.2f} GB of weights per pass stream through the 126 MB L2; single-GEMM figure "
                  "rotates 16 weight buffers (363 MB)"}


# --------------------------------------------------------------------- our arm
def time_graph(graph, iters: int):
    import torch

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def gemm_figures(d, ops, peaks, m, k, n, bits=4, group=128, rotate=16, reps=7) -> dict:
    """One GEMM shape alone, over `rotate` weight buffers so that weights come from HBM."""
    import torch

    torch.manual_seed(0)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    base = d.quantize((torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16), bits=bits,
                      group_size=group, symmetric=True)
    weights = [(torch.randint(0, 256, base.qweight.shape, dtype=torch.uint8, device="cuda"),
                base.scales.clone()) for _ in range(rotate)]
    fn = ops.w4a16 if bits == 4 else ops.w8a16

    def body():
        for q, s in weights:
            fn(x, q, s, None, None, group)

    body()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    graph.replay()
    torch.cuda.synchronize()
    best = min(time_graph(graph, 4) for _ in range(reps)) * 1e3 / (4 * len(weights))  # us per GEMM
    wbytes = base.nbytes
    flops = 2.0 * m * k * n
    t_mem = wbytes / (peaks["hbm_gbs"] * 1e3)      # us
    t_mma = flops / (peaks["tflops"] * 1e6)        # us
    return {"shape": [m, k, n], "bits": bits, "group": group, "us": best, "tflops": flops / best * 1e-6,
            "gbs": wbytes / best * 1e-3, "frac_hbm": t_mem / best, "frac_tensor": t_mma / best,
            "frac_roofline": max(t_mem, t_mma) / best, "roofline_us": max(t_mem, t_mma),
            "bound": "hbm" if t_mem >= t_mma else "tensor", "launches_timed": reps * 4 * len(weights)}


def single_gemm_figures(d, ops, peaks) -> dict:
    """The headline GEMM alone: M=83, K=3072, N=14336, int4 g128, 16 rotating weights."""
    return gemm_figures(d, ops, peaks, 83, 3072, 14336, 4, 128, rotate=16)


def run_allreduce_only(args) -> int:
    """``--gemm allreduce`` under torch.distributed.run: the 83 x 3072 bf16 sum over ranks with
    the library's peer-memory kernel against NCCL's all-reduce, back to back in a CUDA graph."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2:
        print("--gemm allreduce needs torch.distributed.run with at least 2 ranks", file=sys.stderr)
        return 2
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from dexter_labs_b200 import ops

    torch.manual_seed(rank)
    x = torch.randn(83, 3072, device="cuda").to(torch.bfloat16)
    peer = ops.PeerAllReduce(dist.group.WORLD, x.numel(), torch.device("cuda", local))
    y = x.clone()

    def time_us(fn, per=20, replays=10):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(per):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1e3 / (per * replays)

    peer_us = time_us(lambda: peer(x))
    nccl_us = time_us(lambda: dist.all_reduce(y))
    want = x.clone()
    dist.all_reduce(want)
    got = peer(x)
    torch.cuda.synchronize()
    diff = float((got.float() - want.float()).abs().max() / want.float().abs().max().clamp_min(1e-6))
    if rank == 0:
        print(json.dumps({"metric": "allreduce_83x3072_bf16_us", "n_gpus": world, "peer_us": peer_us,
                          "nccl_us": nccl_us, "max_normalised_diff_vs_nccl": diff,
                          "peer_status": peer.check()}), flush=True)
    finish(world, 0)
    return 0


SWEEP_SHAPES = (("qkv", 3072, 9216), ("o", 3072, 3072), ("up", 3072, 14336), ("down", 14336, 3072))
SWEEP_M = (1, 8, 32, 83, 256, 512, 913)


def run_gemm_only(args) -> int:
    """``--gemm M,K,N[,bits[,group]]``: time that one shape on cuda:0 and print one JSON line.
    ``--gemm sweep``: the M sweep over the 5B linear shapes, int4 group 128 and int8 per
    channel, one JSON line per shape."""
    import torch

    torch.cuda.set_device(0)
    import dexter_labs_b200 as d
    from dexter_labs_b200 import ops

    peaks = load_peaks()

    def one(m, k, n, bits, group, reps, name=None):
        wbytes = (k * n // 2 if bits == 4 else k * n)
        rotate = max(2, min(16, int(400e6 // max(wbytes, 1)) + 1))  # > 126 MB L2 where memory allows
        fig = gemm_figures(d, ops, peaks, m, k, n, bits, group, rotate=rotate, reps=reps)
        fig.update({"metric": "wq_gemm_us", "rotating_weights": rotate, "peak_source": peaks["source"]})
        if name:
            fig["name"] = name
        print(json.dumps(fig), flush=True)

    if args.gemm == "sweep":
        for name, k, n in SWEEP_SHAPES:
            for bits in (4, 8):
                for m in SWEEP_M:
                    one(m, k, n, bits, 128 if bits == 4 else k, min(args.reps, 3), name)
        # the 14B-shaped linears (dim 5120, FFN 13824) at the compute-bound token count
        for name, k, n in (("14b_qkvo", 5120, 5120), ("14b_up", 5120, 13824), ("14b_down", 13824, 5120)):
            one(913, k, n, 4, 128, min(args.reps, 3), name)
        return 0
    parts = [int(v) for v in args.gemm.split(",")]
    m, k, n = parts[:3]
    bits = parts[3] if len(parts) > 3 else 4
    group = parts[4] if len(parts) > 4 else (128 if bits == 4 else k)
    one(m, k, n, bits, group, args.reps)
    return 0


def finish(world: int, code: int) -> None:
    """Leave the process without tearing NCCL down.

    The timed passes are CUDA graphs that contain NCCL kernels; destroying the
    communicator while such graphs are alive can block for ever, so multi-rank runs
    flush their output and exit directly once all work is synchronised.
    """
    import torch

    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        os._exit(code)
    sys.exit(code)


def run_ours(args) -> int:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be launched with torch.distributed.run "
                  f"--nproc-per-node {args.gpus}", file=sys.stderr)
            return 2
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import dexter_labs_b200 as d  # loads the CUDA library; fails loudly if it is missing
    from dexter_labs_b200 import ops, tp

    peaks = load_peaks()
    nccl = args.collective if args.collective in ("all_reduce", "rs_ag") else "all_reduce"
    ls = tp.LayerSet.build(PRESET, rank=rank, world=world, bits=4, group_size=128, symmetric=True,
                           bias=True, device=f"cuda:{local}", seed=0, collective=nccl,
                           concurrent=True, fuse_qkv=world > 1)
    small = M_TOKENS <= 128 and M_TOKENS * ls.dim * 2 <= ops.PeerAllReduce.MAX_BYTES
    if world > 1 and args.collective == "fused" and small:
        # the sum over ranks inside the row-parallel GEMMs (at most 128 tokens); else the peer kernel
        if not ls.enable_fused_reduce(M_TOKENS, f"cuda:{local}") and rank == 0:
            print(f"fused sum unavailable ({getattr(ls, '_peer_error', '?')}); trying the peer all-reduce",
                  file=sys.stderr)
    if world > 1 and args.collective in ("fused", "peer") and ls.collective != "fused" and small:
        # own all-reduce kernel over NVLink peer memory (messages up to 1 MB); NCCL otherwise
        if not ls.enable_peer_reduce(M_TOKENS, f"cuda:{local}") and rank == 0:
            print(f"peer all-reduce unavailable ({getattr(ls, '_peer_error', '?')}); using NCCL",
                  file=sys.stderr)
    torch.manual_seed(0)
    host_x = torch.randn(M_TOKENS, ls.dim).to(torch.bfloat16).pin_memory()
    host_ctx = torch.randn(M_TOKENS, ls.dim).to(torch.bfloat16).pin_memory()
    host_y = torch.empty(M_TOKENS, ls.dim, dtype=torch.bfloat16).pin_memory()
    x = host_x.cuda()
    ctx = host_ctx.cuda()

    # one pass, eagerly, then captured into a CUDA graph (kernels + collectives)
    y = ls.forward(x, ctx)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    use_graph = True
    try:
        with torch.cuda.graph(graph):
            y = ls.forward(x, ctx)
    except Exception as exc:  # noqa: BLE001 - e.g. a collective that cannot be captured
        use_graph = False
        if rank == 0:
            print(f"graph capture failed ({exc}); timing eager launches", file=sys.stderr)

    def step():
        if use_graph:
            graph.replay()
        else:
            ls.forward(x, ctx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = elapsed.item() / args.steps

    # end to end through the public API with host buffers: H2D of x and ctx, the pass, D2H of y
    def e2e_step():
        x.copy_(host_x, non_blocking=True)
        ctx.copy_(host_ctx, non_blocking=True)
        step()
        host_y.copy_(y, non_blocking=True)

    for _ in range(2):
        e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_step()
    f1.record()
    barrier()
    e2e = torch.tensor([f0.elapsed_time(f1)], device="cuda")
    if world > 1:
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    e2e_ms = e2e.item() / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # One GPU only: the same linears with self q/k/v and cross k/v each issued as one
    # N-concatenated launch (same arithmetic per column, but another K-split order, so equal
    # only up to fp32 summation order; 7 launches per block instead of 10; the cross k/v launch
    # on a side stream next to self q/k/v), as an extra.
    # With more than one rank the main arm above already is that fused schedule.
    fused_ms, fused_same, fused_launches = None, None, None
    if world == 1:
        try:
            fused = tp.LayerSet(dim=ls.dim, ffn_dim=ls.ffn_dim, blocks=ls.blocks, rank=rank, world=world,
                                bits=ls.bits, group_size=ls.group_size, collective=ls.collective,
                                fuse_qkv=True, concurrent=True,
                                layers=[tp.LayerSet._fuse(r) for r in ls.layers])
            fused_launches = fused.num_gemms
            yf = fused.forward(x, ctx)
            torch.cuda.synchronize()
            fgraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(fgraph):
                yf = fused.forward(x, ctx)
            for _ in range(3):
                fgraph.replay()
            barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            for _ in range(args.steps):
                fgraph.replay()
            g1.record()
            barrier()
            fused_ms = g0.elapsed_time(g1) / args.steps
            fused_same = float((yf.float() - y.float()).abs().max() / y.float().abs().max().clamp(min=1e-6))
        except Exception as exc:  # noqa: BLE001
            print(f"fused-qkv variant not timed: {exc}", file=sys.stderr)

    # The same launches strictly one after the other (no parallel streams), as an extra.
    sequential_ms = None
    try:
        ls.concurrent = False
        ys = ls.forward(x, ctx)
        torch.cuda.synchronize()
        sgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(sgraph):
            ys = ls.forward(x, ctx)
        for _ in range(3):
            sgraph.replay()
        barrier()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record()
        for _ in range(args.steps):
            sgraph.replay()
        h1.record()
        barrier()
        st = torch.tensor([h0.elapsed_time(h1)], device="cuda")
        if world > 1:
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        sequential_ms = st.item() / args.steps
    except Exception as exc:  # noqa: BLE001
        if rank == 0:
            print(f"sequential variant not timed: {exc}", file=sys.stderr)
    ls.concurrent = True

    # More than one rank: block 0 of the sharded set against the same block unsharded on rank
    # 0's GPU (same seeds), outside every timed region.
    parity = None
    if world > 1:
        yb = ls.block_forward(0, x, ctx)
        torch.cuda.synchronize()
        if rank == 0:
            single = tp.LayerSet.build(PRESET, blocks=1, device=f"cuda:{local}", seed=0)
            want = single.forward(x, ctx).float()
            parity = float((yb.float() - want).abs().max() / want.abs().max().clamp(min=1e-6))
            del single
        dist.barrier()

    # Host time of one eager call of the registered kernel (no graph): the headline shape,
    # launches queued back to back, wall clock per call.
    eager_us = None
    if world == 1:
        up = ls.layers[0][8]
        fn = lambda: ops.w4a16(x, up.weight.qweight, up.weight.scales, up.weight.zeros, up.weight.bias,  # noqa: E731
                               up.weight.group_size, layout=up.layout)
        for _ in range(20):
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(200):
            fn()
        eager_us = (time.perf_counter() - t0) / 200 * 1e6
        torch.cuda.synchronize()

    total_bytes = torch.tensor([float(ls.weight_bytes)], device="cuda")
    if world > 1:
        dist.all_reduce(total_bytes)
    if rank != 0:
        finish(world, 0)

    status = ops.last_status()
    set_flops = 2.0 * M_TOKENS * (8 * ls.dim * ls.dim + 2 * ls.dim * ls.ffn_dim) * ls.blocks
    set_bytes = total_bytes.item()
    launches_per_step = ls.num_gemms
    t_mem_ms = set_bytes / world / (peaks["hbm_gbs"] * 1e6)
    # The 5B pass is 300 short kernels (burst peak); the 14B pass at 913 tokens keeps the tensor
    # pipe busy for tens of milliseconds under the power cap (sustained peak).
    sustained = PRESET == "14b" and peaks.get("tflops_sustained")
    tensor_peak = peaks["tflops_sustained"] if sustained else peaks["tflops"]
    t_mma_ms = set_flops / world / (tensor_peak * 1e9)
    roofline_ms = max(t_mem_ms, t_mma_ms)
    # dominant kernel: wq_gemm_tc (int4, symmetric, repacked weights); averages over the pass, per
    # rank: the pass time divided by its launches, which overlap on parallel streams -- not the
    # duration of one launch (the "gemm" key times one shape's launches back to back)
    pass_us_per_launch = ms_per_step * 1e3 / launches_per_step
    flops_per_launch = set_flops / world / launches_per_step
    bytes_per_launch = set_bytes / world / launches_per_step
    bound = "tensor" if t_mma_ms >= t_mem_ms else "hbm"
    if bound == "tensor":
        achieved, peak, unit = flops_per_launch / pass_us_per_launch * 1e-6, tensor_peak, "TFLOP/s"
    else:
        achieved, peak, unit = bytes_per_launch / pass_us_per_launch * 1e-3, peaks["hbm_gbs"], "GB/s"
    own_collective_kernels = 3 * ls.blocks if (ls._peer is not None and ls.collective == "peer") else 0

    line = {
        "metric": METRIC, "value": ms_per_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world, args.collective),
        "collective_used": ls.collective if world > 1 else "none",
        "clocks": clocks,
        "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": 2 * host_x.numel() * 2,
                "d2h_bytes_per_step": host_y.numel() * 2},
        # GEMM launches, plus this library's all-reduce kernel after each row-parallel linear
        # when the sum is not part of the GEMM launch
        "gpu_launches": (launches_per_step + own_collective_kernels) * args.steps,
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                     "frac": achieved / peak, "traffic": bytes_per_launch * DRAM_OVER_ALGORITHMIC,
                     "traffic_source": "algorithmic bytes x 1.025 (DRAM / algorithmic ratio of one ncu capture "
                                       "of the headline launch); scaled, not measured in this run",
                     "kernel": "wq_gemm_tc<4,false,false,true,kModeWhole/kModeCluster>",
                     "peak_source": f"{peaks['source']} ({'sustained' if sustained else 'burst'})",
                     "algorithmic_bytes_per_launch": bytes_per_launch,
                     "algorithmic_flops_per_launch": flops_per_launch,
                     "pass_us_per_launch": pass_us_per_launch,
                     "frac_hbm": (bytes_per_launch / pass_us_per_launch * 1e-3) / peaks["hbm_gbs"]},
        "sequential": {"ms_per_step": sequential_ms, "note": "the same launches on one stream"},
        "fused_qkv": {"ms_per_step": fused_ms, "launches_per_step": fused_launches,
                      "max_normalised_diff_vs_separate": fused_same,
                      "frac_roofline": None if not fused_ms else roofline_ms / fused_ms},
        "layer_set": {"weight_bytes": set_bytes, "flops": set_flops, "roofline_ms": roofline_ms,
                      "frac_roofline": roofline_ms / ms_per_step, "graph": use_graph,
                      "kernel_status": status},
    }
    if world > 1:
        line["parity_vs_unsharded"] = parity
    if world == 1:
        line["eager_us_per_call"] = eager_us
        line["gemm"] = single_gemm_figures(d, ops, peaks)
        per_block_ms, threads, kind = cpu_block_ms(3)
        line["cpu_baseline"] = cpu_baseline_entry(per_block_ms, threads, kind, 3)
    print(json.dumps(line))
    bad = status != 0 or (parity is not None and not parity <= 1e-2)
    finish(world, 1 if bad else 0)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--collective", choices=("fused", "peer", "all_reduce", "rs_ag"), default="fused",
                    help="how row-parallel partial sums are combined when N > 1: inside the GEMM launch "
                         "(fused), by this library's all-reduce kernel (peer), or by NCCL")
    ap.add_argument("--gemm", default=None, metavar="M,K,N[,bits[,group]] | sweep | allreduce",
                    help="time this one GEMM shape only (1 GPU) instead of the layer set; "
                         "`sweep` = M in {1..913} over the 5B linear shapes, int4 and int8")
    ap.add_argument("--reps", type=int, default=7, help="timed repetitions of --gemm (best is kept)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="5b",
                    help="5b: the 5B layer set at 83 tokens (the headline); 14b: the 14B-shaped set at "
                         "913 tokens")
    args = ap.parse_args()
    global M_TOKENS, PRESET, METRIC
    PRESET = args.workload
    M_TOKENS, METRIC = WORKLOADS[PRESET]
    if args.gemm == "allreduce" and args.impl == "ours":
        return run_allreduce_only(args)
    if args.gemm and args.impl == "ours":
        return run_gemm_only(args)
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
