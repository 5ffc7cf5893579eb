"""Parity of the CUDA path (through the C ABI) with the oracle.  Needs a B200: -m gpu.

Tolerances: dequantised weights bit-exact; GEMM outputs within 1e-2 under the
reference tests' max-normalised metric (test/test_ops.py:12-15 in the reference),
which is the tolerance the task states for bf16 accumulation-order differences.
"""
import numpy as np
import pytest
import torch

from conftest import CASES

pytestmark = pytest.mark.gpu
TOL = 1e-2


def t16(a, device="cuda"):
    return None if a is None else torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(device)


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def err(got, want):
    got, want = got.double(), want.double()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)


@pytest.fixture(scope="module")
def d(b200_lib):
    import dexter_labs_b200 as pkg

    return pkg


def run(d, nbits, x, qw, bias=None, **kw):
    fn = d.w4a16 if nbits == 4 else d.w8a16
    return fn(x, qw.qweight, qw.scales, qw.zeros, bias, qw.group_size)


# --------------------------------------------------------------- golden vectors
@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_golden_dequantize_bit_exact(case, d):
    q = torch.from_numpy(case.qweight.copy()).cuda()
    dense = d.dequantize(q, t16(case.scales), t16(case.zeros), case.group, case.bits)
    assert np.array_equal(bits(dense), case.dense)


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_golden_gemm(case, d, oracle):
    q = torch.from_numpy(case.qweight.copy()).cuda()
    fn = d.w4a16 if case.bits == 4 else d.w8a16
    y = fn(t16(case.x), q, t16(case.scales), t16(case.zeros), t16(case.bias), case.group)
    assert y.shape == (case.m, case.n) and y.dtype == torch.bfloat16
    want = torch.from_numpy(oracle.bf16_bits_to_f32(case.y))
    assert err(y.cpu().float(), want) < TOL
    # and against the C oracle (fp32 accumulation like the kernel): tighter
    yc = oracle.c_wq_gemm(case.x, case.qweight, case.scales, case.zeros, case.bias, case.group,
                          case.bits)
    assert err(y.cpu().float(), torch.from_numpy(oracle.bf16_bits_to_f32(yc))) < 5e-3


# ------------------------------------------------------- the benchmark configs
def seeded(d, m, k, n, nbits, group, symmetric, seed, bias=False):
    torch.manual_seed(seed)
    x = torch.randn(m, k).to(torch.bfloat16)
    w = (torch.randn(n, k) * 0.02).to(torch.bfloat16)
    b = torch.randn(n).to(torch.bfloat16) if bias else None
    qw = d.quantize(w.cuda(), bits=nbits, group_size=group, symmetric=symmetric)
    return x, qw, b


CONFIGS = [
    # (id, M, K, N, bits, group, symmetric, seed, bias)
    ("cfg1_w4_up", 83, 3072, 14336, 4, 128, True, 0, False),
    ("cfg1_w4_up_asym_bias", 83, 3072, 14336, 4, 128, False, 0, True),
    ("cfg2_w8_up", 83, 3072, 14336, 8, 3072, True, 0, False),
    ("cfg2_w8_down", 83, 14336, 3072, 8, 14336, True, 1, False),
    ("w8_up_asym_g128_bias", 83, 3072, 14336, 8, 128, False, 2, True),
    ("w4_down", 83, 14336, 3072, 4, 128, True, 3, False),
    ("w4_o", 83, 3072, 3072, 4, 128, True, 4, True),
    ("w4_qkv", 83, 3072, 9216, 4, 128, True, 5, False),
    ("reference_test_shape_w4", 125, 3072, 8192, 4, 128, False, 6, False),
    ("reference_test_shape_w8", 125, 3072, 8192, 8, 128, True, 7, False),
]


@pytest.mark.parametrize("cfg", CONFIGS, ids=lambda c: c[0])
def test_full_size_configs_against_cpu_oracle(cfg, d, oracle):
    _, m, k, n, nbits, group, sym, seed, with_bias = cfg
    x, qw, b = seeded(d, m, k, n, nbits, group, sym, seed, with_bias)
    q_np = qw.qweight.cpu().numpy()
    s_np, z_np = bits(qw.scales), (None if qw.zeros is None else bits(qw.zeros))
    dense = d.dequantize(qw.qweight, qw.scales, qw.zeros, group, nbits)
    assert np.array_equal(bits(dense), oracle.c_dequantize(q_np, s_np, z_np, group, nbits))
    y = run(d, nbits, x.cuda(), qw, None if b is None else b.cuda())
    want = oracle.c_wq_gemm(bits(x), q_np, s_np, z_np, None if b is None else bits(b), group, nbits)
    e = err(y.cpu().float(), torch.from_numpy(oracle.bf16_bits_to_f32(want)))
    assert e < TOL, e
    assert torch.isfinite(y.float()).all()
    assert d.ops.last_status() == 0


SHAPES = {"qkv": (3072, 9216), "o": (3072, 3072), "up": (3072, 14336), "down": (14336, 3072)}


@pytest.mark.parametrize("m", [1, 8, 32, 83, 256, 512, 913])
@pytest.mark.parametrize("shape", ["qkv", "o", "up", "down"])
@pytest.mark.parametrize("nbits", [4, 8])
def test_m_sweep_against_torch_restatement(m, shape, nbits, d, oracle):
    k, n = SHAPES[shape]
    group = 128 if nbits == 4 else k  # int8 per output channel
    x, qw, _ = seeded(d, m, k, n, nbits, group, True, seed=m + n)
    xg = x.cuda()
    y = run(d, nbits, xg, qw)
    want = oracle.torch_wq_gemm(xg, qw.qweight, qw.scales, qw.zeros, None, group, nbits)
    assert err(y.float(), want.float()) < TOL
    # exact scaling property: doubling the activations doubles every output bit for bit
    y2 = run(d, nbits, (xg * 2).contiguous(), qw)
    assert torch.equal(y2.float(), y.float() * 2)
    # determinism (the split-K reduction order is fixed)
    assert torch.equal(run(d, nbits, xg, qw).view(torch.int16), y.view(torch.int16))
    assert d.ops.last_status() == 0


# ------------------------------------------------------------------- edge cases
def test_zero_activations_give_the_bias(d):
    _, qw, b = seeded(d, 9, 3072, 3072, 4, 128, False, 0, bias=True)
    y = run(d, 4, torch.zeros(9, 3072, dtype=torch.bfloat16, device="cuda"), qw, b.cuda())
    assert torch.equal(y.cpu().float(), b.float().expand(9, -1))


def test_empty_and_leading_dims_and_strides(d, oracle):
    x, qw, _ = seeded(d, 12, 512, 256, 4, 128, True, 1)
    xg = x.cuda()
    assert run(d, 4, xg[:0], qw).shape == (0, 256)
    y = run(d, 4, xg, qw)
    y3 = run(d, 4, xg.view(2, 6, 512), qw)
    assert y3.shape == (2, 6, 256) and torch.equal(y3.view(12, 256), y)
    wide = torch.randn(12, 1024, device="cuda").to(torch.bfloat16)
    wide[:, :512] = xg
    assert torch.equal(run(d, 4, wide[:, :512], qw), y)              # row stride 1024
    tr = xg.t().contiguous().t()                                        # inner stride != 1
    assert torch.equal(run(d, 4, tr, qw), y)
    with pytest.raises(ValueError):
        run(d, 4, xg[:, :256], qw)                                      # K mismatch
    with pytest.raises(ValueError):
        d.linear(xg, qw.qweight, None, scales=qw.scales, bits=3)


@pytest.mark.parametrize("m,k,n,nbits,group", [(7, 512, 200, 4, 128), (5, 256, 144, 4, 32),
                                              (3, 384, 48, 8, 128), (130, 256, 16, 4, 128),
                                              (4, 256, 128, 4, 128)])
def test_small_and_ragged_shapes(m, k, n, nbits, group, d, oracle):
    # N not a multiple of 16, groups below 64 rows, K/2 not a multiple of 64: CUDA-core kernel
    x, qw, b = seeded(d, m, k, n, nbits, group, False, seed=n, bias=True)
    y = run(d, nbits, x.cuda(), qw, b.cuda())
    want = oracle.c_wq_gemm(bits(x), qw.qweight.cpu().numpy(), bits(qw.scales), bits(qw.zeros),
                            bits(b), group, nbits)
    assert err(y.cpu().float(), torch.from_numpy(oracle.bf16_bits_to_f32(want))) < TOL


def test_linear_dispatch_and_registry(d):
    # mirror of the reference's test_linear_dispatches_on_bits_not_dtype (test/test_ops.py:106-115)
    from dexter_labs_b200 import registry

    assert "SELECTED" in registry.explain("gemm", "w4a16").split("\n")[1]
    assert registry.select("gemm", "w4a16") is d.w4a16
    for nbits in (4, 8):
        x, qw, _ = seeded(d, 8, 256, 128, nbits, 128, False, seed=nbits)
        y = d.linear(x.cuda(), qw.qweight, None, scales=qw.scales, zeros=qw.zeros,
                     group_size=128, bits=nbits)
        assert y.shape == (8, 128) and torch.isfinite(y.float()).all()


def test_cuda_graph_replay_is_idempotent(d):
    # a shape that takes the split-K path: the tile counters must reset themselves
    x, qw, _ = seeded(d, 83, 3072, 3072, 4, 128, True, 9)
    xg = x.cuda()
    want = run(d, 4, xg, qw)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        run(d, 4, xg, qw)  # warm-up on the capture stream (allocates its workspace)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = run(d, 4, xg, qw)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)


def test_one_block_layer_set_matches_oracle_chain(d, oracle):
    from dexter_labs_b200 import tp

    def oracle_gemm(x, w):
        return oracle.torch_wq_gemm(x, w.qweight, w.scales, w.zeros, w.bias, w.group_size, w.bits)

    ls = tp.LayerSet.build("5b", blocks=1, seed=3)
    torch.manual_seed(1)
    x = torch.randn(83, 3072, device="cuda").to(torch.bfloat16)
    ctx = torch.randn(83, 3072, device="cuda").to(torch.bfloat16)
    got = ls.forward(x, ctx)
    ls.gemm = oracle_gemm
    want = ls.forward(x, ctx)
    assert err(got.float(), want.float()) < TOL
    assert ls.num_gemms == 10


# ------------------------------------------------- launch regimes of the tensor-core kernel
@pytest.mark.parametrize("m,k,n,nbits,max_ctas,why", [
    (83, 512, 20480, 4, 0, "160 tiles > SMs: stream-K with global partials and counters"),
    (83, 3072, 3072, 4, 7, "explicit cap below the tile count: stream-K, several tiles per CTA"),
    (83, 3072, 3072, 4, 1, "one CTA walks every tile"),
    (64, 3072, 3072, 8, 60, "cap that still allows a cluster of 2 per tile"),
    (83, 3072, 3072, 4, 0, "24 tiles: cluster split with the DSMEM reduce"),
    (83, 14336, 3072, 4, 0, "row-parallel shape, 112 units per tile, cluster split"),
    (128, 3072, 3072, 4, 0, "128 tokens: cluster split, receive buffers laid over the idle rings"),
    (100, 14336, 3072, 8, 0, "100 tokens, long K, int8: cluster split with aliased receive buffers"),
    (97, 3072, 3072, 4, 40, "aliased receive buffers under a CTA cap"),
    (83, 3072, 14336, 4, 0, "112 tiles: one CTA per tile"),
])
def test_launch_regimes(m, k, n, nbits, max_ctas, why, d, oracle):
    group = 128
    x, qw, b = seeded(d, m, k, n, nbits, group, False, seed=k + n + max_ctas, bias=True)
    xg, bg = x.cuda(), b.cuda()
    fn = d.w4a16 if nbits == 4 else d.w8a16
    y = fn(xg, qw.qweight, qw.scales, qw.zeros, bg, group, max_ctas=max_ctas)
    want = oracle.torch_wq_gemm(xg, qw.qweight, qw.scales, qw.zeros, bg, group, nbits)
    assert err(y.float(), want.float()) < TOL, why
    again = fn(xg, qw.qweight, qw.scales, qw.zeros, bg, group, max_ctas=max_ctas)
    assert torch.equal(again.view(torch.int16), y.view(torch.int16)), "not deterministic: " + why
    assert d.ops.last_status() == 0


def test_back_to_back_launches_with_dependent_launch(d, oracle):
    # consecutive GEMMs on one stream overlap (programmatic dependent launch); a chain in
    # which each GEMM consumes the previous output must still see finished inputs
    _, q1, _ = seeded(d, 83, 3072, 3072, 4, 128, True, seed=31)
    _, q2, _ = seeded(d, 83, 3072, 3072, 4, 128, True, seed=32)
    torch.manual_seed(5)
    x = torch.randn(83, 3072, device="cuda").to(torch.bfloat16)
    got = x
    for _ in range(4):
        got = d.w4a16(d.w4a16(got, q1.qweight, q1.scales, None, None, 128),
                      q2.qweight, q2.scales, None, None, 128)
    want = x
    for _ in range(4):
        want = oracle.torch_wq_gemm(oracle.torch_wq_gemm(want, q1.qweight, q1.scales, None, None, 128, 4),
                                    q2.qweight, q2.scales, None, None, 128, 4)
    assert err(got.float(), want.float()) < 5 * TOL  # eight chained GEMMs accumulate rounding
    assert torch.isfinite(got.float()).all()


# ------------------------------------------- 14B-shaped linears at M = 913
@pytest.mark.parametrize("shape", [("qkv_like", 5120, 5120), ("up", 5120, 13824), ("down", 13824, 5120)])
def test_14b_shapes_m913(shape, d, oracle):
    _, k, n = shape
    x, qw, b = seeded(d, 913, k, n, 4, 128, True, seed=k + n, bias=True)
    xg, bg = x.cuda(), b.cuda()
    y = run(d, 4, xg, qw, bg)
    want = oracle.torch_wq_gemm(xg, qw.qweight, qw.scales, qw.zeros, bg, 128, 4)
    assert err(y.float(), want.float()) < TOL
    dense = d.dequantize(qw.qweight, qw.scales, qw.zeros, 128, 4)
    assert torch.equal(dense.view(torch.int16),
                       oracle.torch_dequantize(qw.qweight, qw.scales, qw.zeros, 128, 4).view(torch.int16))
    assert d.ops.last_status() == 0


# -------------------------------------------------- shapes a tensor-parallel shard produces
@pytest.mark.parametrize("m,k,n,nbits", [
    (83, 384, 3072, 4),     # 5B o-projection, K sharded 8 ways: 3 units per tile (odd)
    (83, 1792, 3072, 4),    # 5B FFN-down, K sharded 8 ways
    (83, 3072, 384, 4),     # 5B q/k/v, N sharded 8 ways: 3 tiles
    (83, 3072, 1792, 4),    # 5B FFN-up, N sharded 8 ways: 14 tiles
    (83, 768, 1536, 8),     # int8, per-channel, 2-way shards
])
def test_shard_sized_shapes(m, k, n, nbits, d, oracle):
    group = 128 if nbits == 4 else k
    x, qw, b = seeded(d, m, k, n, nbits, group, False, seed=k * 7 + n, bias=True)
    xg, bg = x.cuda(), b.cuda()
    y = run(d, nbits, xg, qw, bg)
    want = oracle.c_wq_gemm(bits(x), qw.qweight.cpu().numpy(), bits(qw.scales), bits(qw.zeros),
                            bits(b), group, nbits)
    assert err(y.cpu().float(), torch.from_numpy(oracle.bf16_bits_to_f32(want))) < TOL
    assert d.ops.last_status() == 0


def test_two_streams_do_not_share_scratch(d, oracle):
    # stream-K launches keep their partial sums in a per-stream workspace
    x, qw, _ = seeded(d, 83, 512, 20480, 4, 128, True, seed=77)
    xg = x.cuda()
    want = run(d, 4, xg, qw)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs = []
    for _ in range(3):
        with torch.cuda.stream(s1):
            a = run(d, 4, xg, qw)
        with torch.cuda.stream(s2):
            b = run(d, 4, xg, qw)
        outs += [a, b]
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o.view(torch.int16), want.view(torch.int16))


# ------------------------------------------------ more than 128 tokens, both plans
@pytest.mark.parametrize("m,k,n,nbits", [(300, 1024, 2048, 4), (913, 3072, 3072, 4), (257, 2048, 1040, 8)])
def test_large_m_one_launch_and_block_by_block_agree(m, k, n, nbits, d, oracle, b200_lib):
    """M > 128: one launch over all token blocks when the workspace holds that plan's partial
    sums, block-by-block launches through a workspace sized for 128 tokens otherwise.  Both are
    checked against the oracle and against each other."""
    import ctypes

    x, qw, bias = seeded(d, m, k, n, nbits, 128 if nbits == 4 else k, True, 5, bias=True)
    x, bias = x.cuda(), bias.cuda()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(nbytes):
        ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = b200_lib.dxb_wq_gemm(nbits, ctypes.c_void_p(x.data_ptr()), k,
                                  ctypes.c_void_p(qw.qweight.data_ptr()),
                                  ctypes.c_void_p(qw.scales.data_ptr()), None,
                                  ctypes.c_void_p(bias.data_ptr()), ctypes.c_void_p(out.data_ptr()), n,
                                  m, n, k, qw.group_size, ctypes.c_void_p(ws.data_ptr()), nbytes, 0,
                                  stream)
        assert rc == 0, b200_lib.dxb_strerror(rc)
        assert b200_lib.dxb_read_status(ctypes.c_void_p(ws.data_ptr()), stream) == 0
        return out

    full = b200_lib.dxb_workspace_bytes(m, n, k, nbits)
    # what block-by-block launches need: blocks of 128 tokens, or 96 for few-tile weights
    one_block = max(b200_lib.dxb_workspace_bytes(128, n, k, nbits),
                    b200_lib.dxb_workspace_bytes(96, n, k, nbits))
    assert full >= one_block
    y_one_launch = call(full)
    y_blocks = call(one_block)
    want = oracle.torch_wq_gemm(x.cpu(), qw.qweight.cpu(), qw.scales.cpu(), None, bias.cpu(),
                                qw.group_size, nbits).float()
    assert err(y_one_launch.cpu().float(), want) < TOL
    assert err(y_blocks.cpu().float(), want) < TOL
    assert err(y_one_launch.cpu().float(), y_blocks.cpu().float()) < TOL
