"""Load-time re-layout of int4 weights, the GELU epilogue, grid caps with an exactly sized
workspace, and a bounded wait that runs out -- all through the C ABI on a B200.  -m gpu."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import CASES

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max-normalised, the reference's metric (test/test_ops.py:12-15) at the tighter bound


def err(got, want):
    got, want = got.double(), want.double()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)


def t16(a):
    return None if a is None else torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.fixture(scope="module")
def d(b200_lib):
    import dexter_labs_b200 as pkg

    return pkg


def _problem(d, m, k, n, nbits, group, symmetric, seed, bias=True):
    torch.manual_seed(seed)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    b = (torch.randn(n, device="cuda") * 0.1).to(torch.bfloat16) if bias else None
    return x, d.quantize(w, bits=nbits, group_size=group, symmetric=symmetric), b


# ------------------------------------------------------------------ re-layout
@pytest.mark.parametrize("case", [c for c in CASES if c.bits == 4 and c.k % 4 == 0 and c.n % 4 == 0],
                         ids=lambda c: c.name)
def test_relayout_round_trip_and_dequantize_on_golden_cases(d, case):
    q = torch.from_numpy(case.qweight).cuda()
    relaid = d.ops.relayout_w4(q)
    assert relaid.shape == q.shape and relaid.dtype == torch.uint8
    back = d.ops.relayout_w4(relaid, inverse=True)
    assert torch.equal(back, q)  # derived from, and returns to, the reference's bytes
    scales = t16(case.scales).cuda()
    zeros = None if case.zeros is None else t16(case.zeros).cuda()
    dense = d.ops.dequantize(relaid, scales, zeros, case.group, 4, layout="b200")
    assert np.array_equal(bits(dense), case.dense)  # bit-exact against the reference's dequantize


def test_relayout_is_local_to_blocks_of_2_rows_by_4_columns(d):
    torch.manual_seed(3)
    q = torch.randint(0, 256, (128, 64), dtype=torch.uint8, device="cuda")
    full = d.ops.relayout_w4(q)
    # slices on block boundaries of the repacked tensor are the repacked slices
    assert torch.equal(d.ops.relayout_w4(q[:, 16:48].contiguous()), full[:, 16:48])
    assert torch.equal(d.ops.relayout_w4(q[32:96].contiguous()), full[32:96])
    # in place
    clone = q.clone()
    d.ops.relayout_w4(clone, out=clone)
    assert torch.equal(clone, full)
    # one word: nibble b = column b of the even row, nibble 4+b = column b of the odd row (low plane)
    words = full.cpu().numpy().view(np.uint32)
    qq = q.cpu().numpy()
    w_even = int(words[0, 0])
    for b in range(4):
        assert (w_even >> (4 * b)) & 0xF == qq[0, b] & 0xF
        assert (w_even >> (16 + 4 * b)) & 0xF == qq[1, b] & 0xF
    w_odd = int(words[1, 0])
    for b in range(4):
        assert (w_odd >> (4 * b)) & 0xF == qq[0, b] >> 4
        assert (w_odd >> (16 + 4 * b)) & 0xF == qq[1, b] >> 4
    with pytest.raises(ValueError):
        d.ops.relayout_w4(q[:, :6].contiguous())


@pytest.mark.parametrize("m,k,n,group,sym,max_ctas", [
    (83, 3072, 14336, 128, True, 0),     # 112 tiles on 148 SMs: equal unit ranges, shared tiles
    (83, 3072, 3072, 128, False, 0),     # cluster split, zero points
    (83, 14336, 3072, 128, True, 0),     # long K, cluster split
    (1, 3072, 9216, 128, True, 0),       # one token
    (32, 3072, 14336, 64, False, 0),     # group 64
    (83, 3072, 3072, 128, True, 7),      # capped grid: several tiles per CTA
    (300, 3072, 3072, 128, True, 0),     # several token blocks
    (913, 1024, 2048, 128, False, 0),
])
def test_gemm_on_repacked_weights_is_bit_identical(d, m, k, n, group, sym, max_ctas):
    x, qw, bias = _problem(d, m, k, n, 4, group, sym, seed=m + n)
    relaid = d.ops.relayout_w4(qw.qweight)
    before = d.ops._AUTO_RELAYOUT
    d.ops._AUTO_RELAYOUT = False  # first arm: the kernel that reads the reference layout
    try:
        plain = d.ops.w4a16(x, qw.qweight, qw.scales, qw.zeros, bias, group, max_ctas=max_ctas)
    finally:
        d.ops._AUTO_RELAYOUT = before
    packed = d.ops.w4a16(x, relaid, qw.scales, qw.zeros, bias, group, max_ctas=max_ctas, layout="b200")
    torch.cuda.synchronize()
    assert d.ops.last_status() == 0
    assert torch.equal(plain.view(torch.int16), packed.view(torch.int16))
    # and the default call (repack made on first use, cached) gives the same bits
    auto = d.ops.w4a16(x, qw.qweight, qw.scales, qw.zeros, bias, group, max_ctas=max_ctas)
    assert torch.equal(auto.view(torch.int16), packed.view(torch.int16))


def test_cached_repack_follows_the_weight(d, oracle):
    x, qw, _ = _problem(d, 16, 512, 256, 4, 128, True, seed=5, bias=False)
    y0 = d.ops.w4a16(x, qw.qweight, qw.scales, None, None, 128)
    assert id(qw.qweight) in d.ops._relaid
    relaid0 = d.ops._relaid[id(qw.qweight)][2]
    d.ops.w4a16(x, qw.qweight, qw.scales, None, None, 128)
    assert d.ops._relaid[id(qw.qweight)][2] is relaid0  # reused, not rebuilt
    qw.qweight.bitwise_xor_(0x11)  # modified in place: the cached copy is stale and is rebuilt
    y1 = d.ops.w4a16(x, qw.qweight, qw.scales, None, None, 128)
    want = oracle.torch_wq_gemm(x.cpu(), qw.qweight.cpu(), qw.scales.cpu(), None, None, 128, 4)
    assert err(y1.float().cpu(), want.float()) < TOL
    assert not torch.equal(y0, y1)
    key = id(qw.qweight)
    del qw, y0, y1
    import gc

    gc.collect()
    assert key not in d.ops._relaid  # dropped with the weight


# -------------------------------------------------------------- GELU epilogue
@pytest.mark.parametrize("m,k,n,nbits,group,bias,max_ctas", [
    (83, 3072, 14336, 4, 128, True, 0),    # the FFN up projection: shared tiles
    (83, 3072, 3072, 4, 128, True, 0),     # cluster split
    (83, 3072, 3072, 4, 128, False, 7),    # whole tiles, several per CTA
    (40, 3072, 14336, 8, 3072, True, 0),   # int8 per channel
    (300, 1024, 2048, 4, 128, True, 0),    # several token blocks
    (5, 256, 200, 4, 128, True, 0),        # plain CUDA-core kernel (ragged N)
])
def test_gelu_epilogue_matches_reference_sequence(d, oracle, m, k, n, nbits, group, bias, max_ctas):
    x, qw, b = _problem(d, m, k, n, nbits, group, False, seed=n + nbits, bias=bias)
    fn = d.ops.w4a16 if nbits == 4 else d.ops.w8a16
    got = fn(x, qw.qweight, qw.scales, qw.zeros, b, group, max_ctas=max_ctas, epilogue="gelu_tanh")
    # the reference: quantised linear, then torch's tanh-GELU on its bf16 output
    # (python/dexter/models/dreamzero/model.py:279-285)
    lin = oracle.torch_wq_gemm(x.cpu(), qw.qweight.cpu(), qw.scales.cpu(), qw.zeros.cpu(),
                               None if b is None else b.cpu(), group, nbits)
    want = torch.nn.functional.gelu(lin, approximate="tanh")
    assert err(got.float().cpu(), want.float()) < TOL
    # on the SAME bf16 linear output the activation itself is exact up to one bf16 rounding
    lin_gpu = fn(x, qw.qweight, qw.scales, qw.zeros, b, group, max_ctas=max_ctas)
    ref = torch.nn.functional.gelu(lin_gpu.float(), approximate="tanh").to(torch.bfloat16)
    assert (got.float() - ref.float()).abs().max().item() <= 2.0 ** -7 * ref.float().abs().max().item()
    if m <= 128:
        short = d.ops.w4a16_gelu if nbits == 4 else d.ops.w8a16_gelu
        assert torch.equal(short(x, qw.qweight, qw.scales, qw.zeros, b, group), fn(
            x, qw.qweight, qw.scales, qw.zeros, b, group, epilogue="gelu_tanh"))


# ------------------------------------- grid caps with an exactly sized workspace
def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("m,k,n", [(83, 3072, 14336), (83, 3072, 3072), (83, 14336, 3072), (913, 5120, 5120)])
def test_capped_grids_run_in_the_uncapped_workspace(d, b200_lib, m, k, n):
    x, qw, bias = _problem(d, m, k, n, 4, 128, True, seed=k)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = b200_lib.dxb_workspace_bytes(m, n, k, 4)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")  # exactly what the header asks for
    want = None
    for cap in (0, 148, 100, 60, 24, 7, 1):
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = b200_lib.dxb_wq_gemm(4, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), None, _ptr(bias),
                                  _ptr(got), n, m, n, k, 128, _ptr(ws), need, cap, stream)
        assert rc == 0, (cap, b200_lib.dxb_strerror(rc))
        assert b200_lib.dxb_read_status(_ptr(ws), stream) == 0
        assert b200_lib.dxb_workspace_bytes_ex(m, n, k, 4, cap) >= 256
        if want is None:
            want = got
        assert err(got.float(), want.float()) < TOL, cap  # only the K-split order differs (a bf16 ulp)


# ----------------------------------------------- a bounded wait that runs out
def test_peer_wait_runs_out_without_hanging(d, b200_lib):
    """Rank 0 of a two-rank sum whose second rank never shows up: both "regions" are ordinary
    local buffers and nobody plays rank 1, so the kernel's wait for it runs out after the
    (shortened) limit, reports DXB_ERR_KERNEL_TIMEOUT in the status word, and the stream
    and the library stay usable.  Nothing faults; the wait is a bounded poll."""
    elems = 83 * 3072
    nbytes = b200_lib.dxb_peer_allreduce_bytes(2, elems)
    regions = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    ptrs = (ctypes.c_void_p * 2)(*[r.data_ptr() for r in regions])
    partial = torch.randn(elems, device="cuda").to(torch.bfloat16)
    out = torch.zeros_like(partial)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    b200_lib.dxb_set_wait_limit_ms(5)
    try:
        rc = b200_lib.dxb_peer_allreduce(_ptr(partial), _ptr(out), elems, ptrs, elems, 0, 2, _ptr(status), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == -8
    finally:
        b200_lib.dxb_set_wait_limit_ms(1000)
    # a one-rank "sum" on the same stream afterwards is just a copy, and a GEMM still works
    status.zero_()
    solo = torch.zeros(b200_lib.dxb_peer_allreduce_bytes(1, elems), dtype=torch.uint8, device="cuda")
    ptr1 = (ctypes.c_void_p * 1)(solo.data_ptr())
    rc = b200_lib.dxb_peer_allreduce(_ptr(partial), _ptr(out), elems, ptr1, elems, 0, 1, _ptr(status), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(out, partial)
    x, qw, _ = _problem(d, 8, 256, 128, 4, 128, True, seed=1, bias=False)
    y = d.ops.w4a16(x, qw.qweight, qw.scales, None, None, 128)
    assert torch.isfinite(y.float()).all() and d.ops.last_status() == 0


def test_fused_sum_wait_runs_out_without_hanging(d, b200_lib):
    """The same for the sum fused into the GEMM: rank 0 of two, the other rank never runs.
    The kernel gives up after the shortened limit and leaves the timeout code in the
    workspace status word; the next ordinary call on the stream is correct."""
    from dexter_labs_b200 import _lib

    m, k, n = 83, 3072, 3072
    x, qw, bias = _problem(d, m, k, n, 4, 128, True, seed=2)
    nbytes = b200_lib.dxb_fused_reduce_bytes(2, m * n)
    regions = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    ptrs = (ctypes.c_void_p * 2)(*[r.data_ptr() for r in regions])
    need = b200_lib.dxb_workspace_bytes(m, n, k, 4)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    opts = _lib.GemmOpts(0, 0, 0, 2, 0, ptrs, m * n)
    b200_lib.dxb_set_wait_limit_ms(5)
    try:
        rc = b200_lib.dxb_wq_gemm_ex(4, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), None, _ptr(bias),
                                     _ptr(out), n, m, n, k, 128, _ptr(ws), need, ctypes.byref(opts), stream)
        assert rc == 0, b200_lib.dxb_strerror(rc)
        assert b200_lib.dxb_read_status(_ptr(ws), stream) == -8
    finally:
        b200_lib.dxb_set_wait_limit_ms(1000)
    ws.zero_()
    rc = b200_lib.dxb_wq_gemm(4, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), None, _ptr(bias),
                              _ptr(out), n, m, n, k, 128, _ptr(ws), need, 0, stream)
    assert rc == 0 and b200_lib.dxb_read_status(_ptr(ws), stream) == 0
    want = d.ops.w4a16(x, qw.qweight, qw.scales, None, bias, 128)
    assert err(out.float(), want.float()) < 5e-3


def test_fused_sum_with_one_rank_equals_the_plain_call(d, b200_lib):
    """world = 1 is the plain GEMM; world = 2 with BOTH ranks played by this GPU one after the
    other cannot be run (a kernel waiting for a later launch), so the two-rank arithmetic is
    covered on two GPUs (test_gpu_multi.py) and here only the option plumbing."""
    from dexter_labs_b200 import _lib

    m, k, n = 40, 1024, 512
    x, qw, bias = _problem(d, m, k, n, 4, 128, False, seed=4)
    need = b200_lib.dxb_workspace_bytes(m, n, k, 4)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    opts = _lib.GemmOpts(0, 0, 0, 1, 0, None, 0)
    rc = b200_lib.dxb_wq_gemm_ex(4, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), _ptr(qw.zeros), _ptr(bias),
                                 _ptr(out), n, m, n, k, 128, _ptr(ws), need, ctypes.byref(opts), stream)
    assert rc == 0
    torch.cuda.synchronize()
    before = d.ops._AUTO_RELAYOUT
    d.ops._AUTO_RELAYOUT = False
    try:
        want = d.ops.w4a16(x, qw.qweight, qw.scales, qw.zeros, bias, 128)
    finally:
        d.ops._AUTO_RELAYOUT = before
    assert torch.equal(out, want)
    # refusals: too many tokens, bad rank, missing regions
    opts = _lib.GemmOpts(0, 0, 0, 2, 5, None, m * n)
    rc = b200_lib.dxb_wq_gemm_ex(4, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), None, None,
                                 _ptr(out), n, m, n, k, 128, _ptr(ws), need, ctypes.byref(opts), stream)
    assert rc == -3
    opts = _lib.GemmOpts(0, 0, 0, 2, 0, None, m * n)
    rc = b200_lib.dxb_wq_gemm_ex(4, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), None, None,
                                 _ptr(out), n, m, n, k, 128, _ptr(ws), need, ctypes.byref(opts), stream)
    assert rc == -2
    opts = _lib.GemmOpts(1, 0, 0, 0, 0, None, 0)  # the repacked layout exists for int4 only
    rc = b200_lib.dxb_wq_gemm_ex(8, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), None, None,
                                 _ptr(out), n, m, n, k // 2, 128, _ptr(ws), need, ctypes.byref(opts), stream)
    assert rc == -4


# ------------------------------------------------------------ dispatcher-level op
def test_custom_op_matches_the_direct_call_and_traces(d):
    x, qw, bias = _problem(d, 83, 1024, 512, 4, 128, False, seed=9)
    direct = d.ops.w4a16(x, qw.qweight, qw.scales, qw.zeros, bias, 128)
    via_op = torch.ops.dexter_b200.wq_gemm(x, qw.qweight, qw.scales, qw.zeros, bias, 128, 4)
    assert torch.equal(direct, via_op)
    torch.library.opcheck(torch.ops.dexter_b200.wq_gemm.default, (x, qw.qweight, qw.scales, qw.zeros, bias, 128, 4),
                          test_utils=("test_schema", "test_faketensor"))

    def fn(inp):
        return d.ops.w4a16(inp * 2, qw.qweight, qw.scales, qw.zeros, bias, 128) + 1

    compiled = torch.compile(fn, backend="eager", fullgraph=True)  # the op must trace as one node
    assert torch.equal(compiled(x), fn(x))
