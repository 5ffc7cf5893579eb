"""The allocation-free entry point `dxb_wq_gemm_static`, called straight through the C ABI.

Some callers of this library are not allowed to allocate device memory: a plugin
running inside a serving runtime that has already handed out the whole GPU, or code
whose host forbids allocator calls on its threads.  For them the split-K scratch sits
in a fixed 24 MiB array inside the library instead of a caller-provided workspace.
This test checks that the result equals the regular entry point's (and the CPU oracle's),
twice in a row (the second call sees whatever the first one left in the array), that the
call leaves the amount of free device memory and torch's allocator untouched, that its
status word can be read without a pointer to the scratch, and that a problem needing
more than the built-in scratch is refused without a launch.

Collected last on purpose (file name), so a run that stops at the first failure has
already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2  # the max-normalised tolerance the parity tests use


def _err(got, want):
    got, want = got.double(), want.double()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)


def _problem(d, m, k, n, nbits, group, symmetric, seed):
    torch.manual_seed(seed)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    return x, d.quantize(w, bits=nbits, group_size=group, symmetric=symmetric), bias


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _call_both(lib, x, qw, bias):
    m, k = x.shape
    n = qw.qweight.shape[1]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.dxb_workspace_bytes(m, n, k, qw.bits)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")  # the regular path's workspace
    want = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    rc = lib.dxb_wq_gemm(qw.bits, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), _ptr(qw.zeros),
                         _ptr(bias), _ptr(want), n, m, n, k, qw.group_size, _ptr(ws), need, 0, stream)
    assert rc == 0, lib.dxb_strerror(rc)
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc = lib.dxb_wq_gemm_static(qw.bits, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales),
                                _ptr(qw.zeros), _ptr(bias), _ptr(got), n, m, n, k, qw.group_size,
                                stream)
    assert rc == 0, lib.dxb_strerror(rc)
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_matches_workspace_path_twice(b200_lib, oracle):
    import dexter_labs_b200 as d

    # the shapes split tiles across CTAs (clusters; equal unit ranges through the scratch), so
    # counters and partial sums in the array are used
    first = _problem(d, 83, 3072, 3072, 4, 128, True, seed=21)
    second = _problem(d, 40, 14336, 3072, 8, 14336, False, seed=22)
    third = _problem(d, 83, 1024, 14336, 4, 128, True, seed=23)
    for x, qw, bias in (first, second, third, first):
        got, want = _call_both(b200_lib, x, qw, bias)
        assert torch.isfinite(got.float()).all()
        assert _err(got.float(), want.float()) < TOL
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))  # same kernel, same order
        ref = oracle.torch_wq_gemm(x.cpu(), qw.qweight.cpu(), qw.scales.cpu(),
                                   None if qw.zeros is None else qw.zeros.cpu(), bias.cpu(),
                                   qw.group_size, qw.bits)
        assert _err(got.float().cpu(), ref.float()) < TOL
    # the status word of the built-in scratch is readable without its address
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert b200_lib.dxb_read_status(None, stream) == 0


def test_static_call_allocates_nothing(b200_lib):
    import dexter_labs_b200 as d

    x, qw, bias = _problem(d, 83, 1024, 14336, 4, 128, True, seed=24)
    m, k = x.shape
    n = qw.qweight.shape[1]
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call():
        rc = b200_lib.dxb_wq_gemm_static(qw.bits, _ptr(x), k, _ptr(qw.qweight), _ptr(qw.scales), None,
                                         _ptr(bias), _ptr(out), n, m, n, k, qw.group_size, stream)
        assert rc == 0, b200_lib.dxb_strerror(rc)

    call()  # first call on the device: looks the array's address up, loads the kernel
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    torch_bytes0 = torch.cuda.memory_allocated()
    torch_reserved0 = torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0  # cudaMemGetInfo: not a byte of device memory was taken
    assert torch.cuda.memory_allocated() == torch_bytes0
    assert torch.cuda.memory_reserved() == torch_reserved0


def test_static_scratch_refuses_oversized_problem(b200_lib):
    # 128 tokens x 65536 columns would need ~100 MiB of partial sums: refused before any launch,
    # so dummy (never dereferenced) pointers are enough here
    fake = ctypes.c_void_p(256)
    rc = b200_lib.dxb_wq_gemm_static(4, fake, 3072, fake, fake, None, None, fake, 65536, 128, 65536,
                                     3072, 128, None)
    assert rc == -9
    assert b"24 MiB" in b200_lib.dxb_strerror(rc)
