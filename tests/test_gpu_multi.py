"""Tensor-parallel layer set on 2, 4 and 8 GPUs (each skipped where fewer are visible): NCCL
collectives, the peer all-reduce kernel and the sum fused into the row-parallel GEMMs, every
rank's output against the unsharded result.  -m gpu."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT  # noqa: F401

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from dexter_labs_b200 import ops, tp

        def settled(phase):
            # No kernel of this phase gave up on a bounded wait; then line the ranks up again: a
            # kernel waits about a second for a peer, and eight eagerly launching processes
            # that also pickle results between phases must not drift further apart than that.
            torch.cuda.synchronize()
            code = ops.last_status()
            assert code == 0, (phase, rank, code)
            dist.barrier()

        ls = tp.LayerSet.build("5b", blocks=1, rank=rank, world=world, seed=3, device=f"cuda:{rank}")
        torch.manual_seed(1)
        x = torch.randn(83, 3072).to(torch.bfloat16).cuda()
        ctx = torch.randn(83, 3072).to(torch.bfloat16).cuda()
        y = ls.forward(x, ctx)
        torch.cuda.synchronize()
        results[rank] = y.float().cpu().numpy()
        # the overlapped multi-stream schedule computes the same linears
        ls.concurrent = True
        y2 = ls.forward(x, ctx)
        torch.cuda.synchronize()
        results[rank + world] = y2.float().cpu().numpy()
        # own all-reduce kernel over peer-mapped memory instead of NCCL, eagerly and as a
        # replayed CUDA graph (the epoch lives on the device, so replays keep working)
        if ls.enable_peer_reduce(83, f"cuda:{rank}"):
            y3 = ls.forward(x, ctx)
            torch.cuda.synchronize()
            results[rank + 2 * world] = y3.float().cpu().numpy()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                y4 = ls.forward(x, ctx)
            for _ in range(3):
                y4.zero_()
                graph.replay()
                torch.cuda.synchronize()
                assert torch.equal(y4, y3)
            assert ls._peer.check() == 0
            results["peer"] = True
        else:
            results["peer_error"] = getattr(ls, "_peer_error", "unknown")
        settled("all-reduce and peer kernel")
        # q/k/v fused into one launch, cross k/v overlapped with self o's collective
        fused = tp.LayerSet.build("5b", blocks=1, rank=rank, world=world, seed=3, device=f"cuda:{rank}",
                                  fuse_qkv=True, concurrent=True, collective="all_reduce")
        y5 = fused.forward(x, ctx)
        torch.cuda.synchronize()
        results[rank + 3 * world] = y5.float().cpu().numpy()
        # reduce-scatter + all-gather instead of the all-reduce
        rsag = tp.LayerSet.build("5b", blocks=1, rank=rank, world=world, seed=3, device=f"cuda:{rank}",
                                 collective="rs_ag")
        y6 = rsag.forward(x, ctx)
        torch.cuda.synchronize()
        results[rank + 4 * world] = y6.float().cpu().numpy()
        # the sum over ranks inside the row-parallel GEMM's own launch: plain and overlapped
        # schedules, eagerly and as a replayed CUDA graph
        settled("fused q/k/v and reduce-scatter + all-gather")
        if fused.enable_fused_reduce(83, f"cuda:{rank}"):
            y7 = fused.forward(x, ctx)
            settled("fused sum, overlapped schedule, eager")
            results[rank + 5 * world] = y7.float().cpu().numpy()
            fused.concurrent = False
            dist.barrier()
            y8 = fused.forward(x, ctx)
            settled("fused sum, one stream, eager")
            fused.concurrent = True
            # same linears on another schedule (the capped side-stream launch splits K differently)
            results[rank + 6 * world] = y8.float().cpu().numpy()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                y9 = fused.forward(x, ctx)
            for i in range(3):
                y9.zero_()
                dist.barrier()
                graph.replay()
                settled(f"fused sum, replayed graph {i}")
                assert torch.equal(y9, y7)
            results["fused"] = True
        else:
            results["fused_error"] = getattr(fused, "_peer_error", "unknown")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_layer_set_matches_one_gpu(b200_lib, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from dexter_labs_b200 import tp

    single = tp.LayerSet.build("5b", blocks=1, seed=3)
    torch.manual_seed(1)
    x = torch.randn(83, 3072).to(torch.bfloat16).cuda()
    ctx = torch.randn(83, 3072).to(torch.bfloat16).cuda()
    want = single.forward(x, ctx).float().cpu().numpy()
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert results.get("peer"), f"peer all-reduce could not be set up: {results.get('peer_error')}"
    assert results.get("fused"), f"fused sum could not be set up: {results.get('fused_error')}"
    # NCCL all-reduce (plain, overlapped), peer kernel, fused q/k/v, rs+ag, fused sum: every
    # rank's output against the unsharded result
    for slot in range(7 * world):
        e = np.abs(results[slot] - want).max() / max(np.abs(want).max(), 1e-6)
        assert e < 1e-2, (slot // world, slot % world, e)
    # every rank holds the same bits after the peer all-reduce and after the fused sum (fixed
    # summation order)
    for base in (2 * world, 5 * world):
        for rank in range(1, world):
            assert np.array_equal(results[base], results[base + rank]), (base // world, rank)
