"""The chain entry point (several GEMMs, one launch) against the oracle.  Needs a B200: -m gpu.

Every link must give what the single GEMM gives: checked against the oracle's
restatement of the reference (reference/gemm.py:51-79 in the reference) on the same
inputs, link by link, feeding each dependent link the CHAIN's own output of its
producer so that only that link's arithmetic is compared.  Tolerance: 1e-2
max-normalised, as for the single GEMM.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2


def err(got, want):
    got, want = got.double(), want.double()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)


@pytest.fixture(scope="module")
def d(b200_lib):
    import dexter_labs_b200 as pkg

    return pkg


def make(d, k, n, nbits, group, symmetric, seed, bias=True):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    b = (torch.randn(n, generator=g) * 0.1).to(torch.bfloat16).cuda() if bias else None
    qw = d.quantize(w.cuda(), bits=nbits, group_size=group, symmetric=symmetric)
    return qw, b


def run_chain(d, oracle, spec, nbits, m, symmetric=True, group=128, seed=0):
    """spec: list of (x source, K, N); a source is "x", "ctx" or the index of an earlier link."""
    from dexter_labs_b200 import ops

    g = torch.Generator().manual_seed(seed)
    kx = next(k for s, k, _ in spec if s == "x")
    ext = {"x": torch.randn(m, kx, generator=g).to(torch.bfloat16).cuda()}
    if any(s == "ctx" for s, _, _ in spec):
        kc = next(k for s, k, _ in spec if s == "ctx")
        ext["ctx"] = torch.randn(m, kc, generator=g).to(torch.bfloat16).cuda()
    weights = [make(d, k, n, nbits, group if nbits == 4 else k, symmetric, seed + 1 + i)
               for i, (_, k, n) in enumerate(spec)]
    links = [ops.ChainLink(s if isinstance(s, int) else ext[s], qw.qweight, qw.scales, qw.zeros, b,
                           qw.group_size)
             for (s, _, _), (qw, b) in zip(spec, weights)]
    outs = ops.chain(links, bits=nbits)
    torch.cuda.synchronize()
    assert ops.chain_status() == 0
    for i, ((s, k, n), (qw, b)) in enumerate(zip(spec, weights)):
        xin = outs[s] if isinstance(s, int) else ext[s]
        assert outs[i].shape == (m, n) and outs[i].dtype == torch.bfloat16
        want = oracle.torch_wq_gemm(xin.cpu(), qw.qweight.cpu(), qw.scales.cpu(),
                                    None if qw.zeros is None else qw.zeros.cpu(),
                                    None if b is None else b.cpu(), qw.group_size, nbits)
        e = err(outs[i].cpu().float(), want.float())
        assert e < TOL, f"link {i} ({k}x{n}): {e}"
    return links, outs


def test_chain_single_link(d, oracle):
    run_chain(d, oracle, [("x", 1024, 512)], 4, 83)


def test_chain_independent_links(d, oracle):
    run_chain(d, oracle, [("x", 1024, 384), ("x", 1024, 1024), ("ctx", 2048, 256)], 4, 83)


def test_chain_dependent_links(d, oracle):
    # up -> down -> out, with an independent link in between
    run_chain(d, oracle, [("x", 1024, 4096), ("x", 1024, 1024), (0, 4096, 1024), (2, 1024, 1024)], 4, 83)


@pytest.mark.parametrize("m", [1, 16, 83, 96])
def test_chain_token_counts(d, oracle, m):
    run_chain(d, oracle, [("x", 1024, 1536), (0, 1536, 512)], 4, m)


def test_chain_asymmetric_and_ragged_columns(d, oracle):
    # zero points; N = 1104 is not a multiple of the 128-column tile
    run_chain(d, oracle, [("x", 1024, 1104), ("x", 1024, 2048), (1, 2048, 1104)], 4, 40, symmetric=False)


def test_chain_int8(d, oracle):
    run_chain(d, oracle, [("x", 1024, 2048), (0, 2048, 1024), ("x", 1024, 512)], 8, 83)
    run_chain(d, oracle, [("x", 1024, 2048), (0, 2048, 1024)], 8, 20, symmetric=False)


def test_chain_5b_block_shapes(d, oracle):
    """The ten linears of one 5B block as one chain, in a dependency-friendly order."""
    D, F = 3072, 14336
    spec = [("ctx", D, D), ("x", D, D), ("x", D, D), ("x", D, D), ("ctx", D, D), (0, D, D), (3, D, D),
            (6, D, D), (5, D, F), (8, F, D)]
    run_chain(d, oracle, spec, 4, 83)


def test_chain_replays_in_a_cuda_graph(d, oracle):
    """The kernel leaves its workspace clean, so a captured chain can be replayed."""
    from dexter_labs_b200 import ops

    links, outs = run_chain(d, oracle, [("x", 1024, 2048), (0, 2048, 1024), ("x", 1024, 512)], 4, 83)
    want = [o.clone() for o in outs]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        again = ops.chain(links, bits=4)
    for _ in range(3):
        for o in again:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for a, w in zip(again, want):
            assert torch.equal(a, w)  # same split, same summation order: bit-identical
    assert ops.chain_status() == 0


def test_chain_refuses_what_it_cannot_run(d):
    from dexter_labs_b200 import ops

    qw, b = make(d, 1024, 512, 4, 128, True, 1)
    x = torch.randn(8, 1024).to(torch.bfloat16).cuda()
    with pytest.raises(ValueError):   # a link may only depend on an earlier one
        ops.chain([ops.ChainLink(0, qw.qweight, qw.scales, None, b, 128)], bits=4)
    with pytest.raises(ValueError):   # K mismatch
        ops.chain([ops.ChainLink(x[:, :512], qw.qweight, qw.scales, None, b, 128)], bits=4)
    with pytest.raises(ValueError):
        ops.chain([], bits=4)
    # too few K units for a cluster to share: refused, nothing launched
    qs, bs = make(d, 128, 512, 4, 128, True, 2)
    xs = torch.randn(8, 128).to(torch.bfloat16).cuda()
    with pytest.raises(RuntimeError):
        ops.chain([ops.ChainLink(xs, qs.qweight, qs.scales, None, bs, 128)], bits=4)
    # mixed symmetric / asymmetric links: refused
    qa, ba = make(d, 1024, 512, 4, 128, False, 3)
    with pytest.raises(RuntimeError):
        ops.chain([ops.ChainLink(x, qw.qweight, qw.scales, None, b, 128),
                   ops.ChainLink(x, qa.qweight, qa.scales, qa.zeros, ba, 128)], bits=4)
