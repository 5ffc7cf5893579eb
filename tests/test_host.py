"""Host-side logic that needs no GPU: quantiser mirror, registry, platform, C ABI surface."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import CASES, ROOT


def t16(a):
    return None if a is None else torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


# ------------------------------------------------------------------ quantiser
@pytest.mark.parametrize("case", [c for c in CASES if c.w is not None], ids=lambda c: c.name)
def test_quantize_matches_reference_bytes(case, b200_lib):
    from dexter_labs_b200.quant import quantize

    qw = quantize(t16(case.w).view(case.n, case.k), bits=case.bits, group_size=case.group,
                  symmetric=case.symmetric)
    assert np.array_equal(qw.qweight.numpy(), case.qweight)
    assert np.array_equal(bits(qw.scales), case.scales)
    assert (qw.zeros is None) == (case.zeros is None)
    if qw.zeros is not None:
        assert np.array_equal(bits(qw.zeros), case.zeros)
    assert qw.shape == (case.k, case.n) and qw.bits == case.bits and qw.group_size == case.group
    assert qw.nbytes == case.nbytes


def test_quantize_errors_and_defaults(b200_lib):
    from dexter_labs_b200.quant import BF16_MAGIC_BIAS, DEFAULT_GROUP_SIZE, quantize

    w = torch.randn(16, 256).to(torch.bfloat16)
    with pytest.raises(ValueError):
        quantize(w.view(-1))
    with pytest.raises(ValueError):
        quantize(w, bits=3)
    with pytest.raises(ValueError):
        quantize(w, group_size=96)
    qw = quantize(w)  # reference defaults: 4 bit, group 128, asymmetric
    assert DEFAULT_GROUP_SIZE == 128 and BF16_MAGIC_BIAS == 128.0
    assert qw.bits == 4 and qw.group_size == 128 and qw.zeros is not None
    assert qw.qweight.shape == (128, 16) and qw.scales.shape == (2, 16)
    assert float(qw.zeros.float().min()) >= 128.0  # 4-bit zero points carry the +128 bias
    q8 = quantize(w, bits=8, symmetric=True)
    assert q8.zeros is None and q8.qweight.shape == (256, 16)
    bias = torch.zeros(16, dtype=torch.bfloat16)
    assert quantize(w, bias=bias).bias is bias
    moved = qw.to("cpu")
    assert moved.shape == qw.shape and torch.equal(moved.qweight, qw.qweight)


def test_round_trip_error_bounds(b200_lib, oracle):
    # the reference's own bound (test/test_model.py:116-124): < 0.12 for int4, < 0.01 for int8
    from dexter_labs_b200.quant import quantize

    torch.manual_seed(0)
    w = torch.randn(256, 512).to(torch.bfloat16) * 0.05
    for nbits, tol in ((4, 0.12), (8, 0.01)):
        for sym in (False, True):
            qw = quantize(w, bits=nbits, symmetric=sym)
            dense = oracle.c_dequantize(qw.qweight.numpy(), bits(qw.scales),
                                        None if qw.zeros is None else bits(qw.zeros), 128, nbits)
            back = oracle.bf16_bits_to_f32(dense).T
            err = oracle.max_normalised_error(back, w.float().numpy())
            assert err < tol, (nbits, sym, err)


# ------------------------------------------------------------------- registry
def _fresh_registry():
    import importlib

    import dexter_labs_b200.registry as reg

    return importlib.reload(reg) if False else reg


def test_registry_selection_rules(b200_lib, monkeypatch):
    from dexter_labs_b200 import platform as plat
    from dexter_labs_b200 import registry as reg

    fam, mode = "testfam", "m1"
    calls = []

    @reg.register(fam, mode, name="ref", priority=reg.Priority.REFERENCE)
    def ref_impl(*a):
        calls.append("ref")

    @reg.register(fam, mode, name="fast", priority=reg.Priority.SPECIALISED,
                  capability=plat.Capability(vendors=frozenset({"nvidia"}),
                                             min_arch=plat.ArchVersion(10, 0)),
                  accepts=lambda *a: not a or a[0] != "decline")
    def fast_impl(*a):
        calls.append("fast")

    with pytest.raises(ValueError):
        reg.register(fam, mode, name="fast")(lambda: None)  # duplicate name

    cpu = plat.PlatformInfo("cpu", "cpu", plat.ArchVersion(0, 0), "CPU", "cpu", 1, 1, 0, 0, 0.0)
    b200 = plat.PlatformInfo("nvidia", "sm100", plat.ArchVersion(10, 0), "NVIDIA", "B200", 148, 32,
                             49152, 1 << 37, 0.0,
                             frozenset({"matrix:f16", "matrix:bf16", "mma:mma"}))
    h100 = plat.PlatformInfo("nvidia", "sm90", plat.ArchVersion(9, 0), "NVIDIA", "H100", 132, 32,
                             49152, 1 << 36, 0.0, frozenset({"matrix:bf16"}))
    try:
        plat.override_platform(cpu)
        assert reg.select(fam, mode) is ref_impl  # gate fails -> reference
        plat.override_platform(h100)
        assert reg.select(fam, mode) is ref_impl  # arch gate
        plat.override_platform(b200)
        assert reg.select(fam, mode) is fast_impl
        assert reg.select(fam, mode, "ok") is fast_impl
        assert reg.select(fam, mode, "decline") is ref_impl  # accepts() declined the shape
        assert [s.name for s in reg.candidates(fam, mode)] == ["fast", "ref"]
        text = reg.explain(fam, mode)
        assert "fast" in text and "SELECTED (pri=12)" in text and "viable (pri=0)" in text
        monkeypatch.setenv("DEXTER_KERNEL", f"other/x:y, {fam}/{mode}:ref")
        assert reg.select(fam, mode) is ref_impl  # pinned
        monkeypatch.setenv("DEXTER_KERNEL", f"{fam}/{mode}:nope")
        with pytest.raises(LookupError):
            reg.select(fam, mode)
        monkeypatch.delenv("DEXTER_KERNEL")
        with pytest.raises(LookupError):
            reg.select(fam, "unregistered")
    finally:
        plat.override_platform(None)


def test_b200_kernels_registered_and_gated(b200_lib):
    import dexter_labs_b200 as d
    from dexter_labs_b200 import platform as plat
    from dexter_labs_b200 import registry as reg

    for mode in ("w4a16", "w8a16"):
        specs = reg._REGISTRY[f"gemm/{mode}"]
        spec = next(s for s in specs if s.name == d.KERNEL_NAMES[mode])
        assert int(spec.priority) == int(reg.Priority.SPECIALISED)
        assert spec.capability.vendors == frozenset({"nvidia"})
        assert tuple(spec.capability.min_arch) == (10, 0)
        assert spec.accepts() is True  # benchmarks call accepts() with no arguments
    if not torch.cuda.is_available():
        assert plat.current_platform().vendor == "cpu"
        with pytest.raises(LookupError):  # no CPU fallback is registered
            reg.select("gemm", "w4a16")


def test_accepts_predicate(b200_lib):
    from dexter_labs_b200.ops import accepts

    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    q = torch.zeros(128, 16, dtype=torch.uint8)
    s = torch.zeros(2, 16, dtype=torch.bfloat16)
    assert accepts() is True
    assert accepts(x, q, s) is False  # CPU tensors are not ours
    assert accepts(x.float(), q, s) is False


def test_no_cpu_path(b200_lib):
    import dexter_labs_b200 as d

    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    q = torch.zeros(128, 16, dtype=torch.uint8)
    s = torch.zeros(2, 16, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        d.w4a16(x, q, s, None, None, 128)
    with pytest.raises(RuntimeError):
        d.dequantize(q, s, None, 128, 4)
    with pytest.raises(ValueError):
        d.linear(x, q, None, scales=s, bits=5)
    with pytest.raises(NotImplementedError):
        d.linear(x, q, None)


# --------------------------------------------------------------------- C ABI
def test_library_exports_every_declared_symbol(b200_lib):
    header = (ROOT / "include" / "dexter_b200.h").read_text()
    declared = set(re.findall(r"\b(dxb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    from dexter_labs_b200 import _lib

    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"
    for name in declared:
        assert hasattr(b200_lib, name), f"{name} is declared but not exported"


def test_strerror_and_argument_checks(b200_lib):
    # these entry points return before touching the device
    assert b200_lib.dxb_strerror(0) == b"ok"
    assert b"bits" in b200_lib.dxb_strerror(-1)
    vp = ctypes.c_void_p
    rc = b200_lib.dxb_wq_gemm(5, vp(16), 256, vp(16), vp(16), None, None, vp(16), 16, 1, 16, 256, 128,
                              None, 0, 0, None)
    assert rc == -1  # DXB_ERR_BITS
    rc = b200_lib.dxb_wq_gemm(4, None, 256, vp(16), vp(16), None, None, vp(16), 16, 1, 16, 256, 128,
                              None, 0, 0, None)
    assert rc == -2  # DXB_ERR_NULL
    rc = b200_lib.dxb_wq_gemm(4, vp(16), 256, vp(16), vp(16), None, None, vp(16), 16, 1, 16, 256, 96,
                              None, 0, 0, None)
    assert rc == -3  # K not a multiple of the group
    rc = b200_lib.dxb_wq_gemm(4, vp(16), 128, vp(16), vp(16), None, None, vp(16), 16, 1, 16, 256, 128,
                              None, 0, 0, None)
    assert rc == -3  # ldx < K
    assert b200_lib.dxb_dequantize(vp(16), vp(16), None, vp(16), 16, 256, 128, 3, None) == -1
    assert b200_lib.dxb_uses_tensor_cores(83, 14336, 3072, 128, 4) == 1
    assert b200_lib.dxb_uses_tensor_cores(83, 200, 3072, 128, 4) == 0   # N % 16
    assert b200_lib.dxb_uses_tensor_cores(83, 256, 256, 32, 4) == 0     # group < 64 rows
    assert b200_lib.dxb_uses_tensor_cores(913, 3072, 3072, 128, 4) == 1  # token blocks of 128
    assert b200_lib.dxb_uses_tensor_cores(83, 3072, 3072, 3072, 8) == 1   # int8: units of 128 rows
    assert b200_lib.dxb_uses_tensor_cores(83, 3072, 192, 64, 8) == 0      # int8 with K % 128 != 0


def test_compiled_binding_reaches_the_same_entry_point(b200_lib):
    """`_dxb_fast.gemm` (csrc/fastcall.c) is dxb_wq_gemm_ex with integer arguments: the argument
    checks answer exactly as through ctypes, before anything touches the device."""
    from dexter_labs_b200 import _lib

    fast = _lib.load_fast()
    assert fast is not None, "the compiled binding was not built (dexter_labs_b200/build.py)"

    def call(bits=4, x=16, ldx=256, k=256, group=128):
        # bits, x, ldx, qweight, scales, zeros, bias, out, ldo, M, N, K, group, ws, ws_bytes,
        # layout, epilogue, max_ctas, serialize, stream
        return fast(bits, x, ldx, 16, 16, 0, 0, 16, 16, 1, 16, k, group, 0, 0, 0, 0, 0, 0, 0)

    assert call(bits=5) == -1        # DXB_ERR_BITS
    assert call(x=0) == -2           # DXB_ERR_NULL
    assert call(group=96) == -3      # K not a multiple of the group
    assert call(ldx=128) == -3       # ldx < K
    with pytest.raises(TypeError):
        fast(4, 16, 256)
    with pytest.raises((TypeError, OverflowError)):
        fast(*(["x"] + [0] * 19))
    # an unknown layout is refused by the option check, as through ctypes
    assert fast(4, 16, 256, 16, 16, 0, 0, 16, 16, 1, 16, 256, 128, 0, 0, 7, 0, 0, 0, 0) != 0


def test_peer_and_option_entry_points_check_their_arguments(b200_lib):
    """Argument checks of the all-reduce, re-layout and option entry points return before any launch."""
    from dexter_labs_b200 import _lib

    vp = ctypes.c_void_p
    assert ctypes.sizeof(_lib.GemmOpts) == 48  # 5 ints, padding, a pointer, an int64, an int, padding
    assert b200_lib.dxb_relayout_w4(None, vp(16), 256, 64, 0, None) == -2
    assert b200_lib.dxb_relayout_w4(vp(16), vp(16), 254, 64, 0, None) == -3   # whole row pairs
    assert b200_lib.dxb_relayout_w4(vp(16), vp(16), 256, 62, 0, None) == -3   # whole 32-bit words
    assert b200_lib.dxb_fused_reduce_bytes(9, 1024) == 0 and b200_lib.dxb_fused_reduce_bytes(2, 0) == 0
    assert b200_lib.dxb_fused_reduce_bytes(8, 1024) > b200_lib.dxb_fused_reduce_bytes(2, 1024) > 2 * 2 * 1024 * 2
    bad = _lib.GemmOpts(7, 0, 0, 0, 0, None, 0)  # unknown layout
    assert b200_lib.dxb_wq_gemm_ex(4, vp(16), 3072, vp(16), vp(16), None, None, vp(16), 3072, 83, 3072, 3072,
                                   128, None, 0, ctypes.byref(bad), None) == -4
    bad = _lib.GemmOpts(0, 9, 0, 0, 0, None, 0)  # unknown epilogue
    assert b200_lib.dxb_wq_gemm_ex(4, vp(16), 3072, vp(16), vp(16), None, None, vp(16), 3072, 83, 3072, 3072,
                                   128, None, 0, ctypes.byref(bad), None) == -4
    bad = _lib.GemmOpts(0, 0, 0, 9, 0, None, 0)  # more ranks than one NVLink domain holds
    assert b200_lib.dxb_wq_gemm_ex(4, vp(16), 3072, vp(16), vp(16), None, None, vp(16), 3072, 83, 3072, 3072,
                                   128, None, 0, ctypes.byref(bad), None) == -3
    assert b200_lib.dxb_dequantize_ex(vp(16), vp(16), None, vp(16), 16, 256, 128, 8, 1, None) == -4
    assert b200_lib.dxb_workspace_bytes_ex(83, 3072, 3072, 4, 0) == b200_lib.dxb_workspace_bytes(83, 3072, 3072, 4)
    # peer all-reduce: region size is plain arithmetic; bad ranks and sizes are refused
    one = b200_lib.dxb_peer_allreduce_bytes(2, 1024)
    assert one > 2 * 2 * 1024 * 2 and b200_lib.dxb_peer_allreduce_bytes(8, 1024) > one
    assert b200_lib.dxb_peer_allreduce_bytes(9, 1024) == 0
    assert b200_lib.dxb_peer_allreduce_bytes(2, 0) == 0
    regions = (vp * 2)(vp(256), vp(512))
    assert b200_lib.dxb_peer_allreduce(None, vp(16), 8, regions, 8, 0, 2, None, None) == -2
    assert b200_lib.dxb_peer_allreduce(vp(16), vp(16), 8, regions, 8, 2, 2, None, None) == -3   # rank
    assert b200_lib.dxb_peer_allreduce(vp(16), vp(16), 12, regions, 16, 0, 2, None, None) == -3  # % 8
    assert b200_lib.dxb_peer_allreduce(vp(16), vp(16), 16, regions, 8, 0, 2, None, None) == -3   # capacity


def test_custom_op_is_declared_with_a_shape_function(b200_lib):
    """torch.ops.dexter_b200.wq_gemm traces without a GPU: output shape, dtype and device come
    from the shape-only implementation; a K mismatch is refused while tracing."""
    import dexter_labs_b200  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(2, 83, 3072, dtype=torch.bfloat16, device="cuda")
        q4 = torch.empty(1536, 14336, dtype=torch.uint8, device="cuda")
        q8 = torch.empty(3072, 512, dtype=torch.uint8, device="cuda")
        s = torch.empty(24, 14336, dtype=torch.bfloat16, device="cuda")
        y = torch.ops.dexter_b200.wq_gemm(x, q4, s, None, None, 128, 4)
        assert y.shape == (2, 83, 14336) and y.dtype == torch.bfloat16 and y.device.type == "cuda"
        y = torch.ops.dexter_b200.wq_gemm(x, q8, s[:, :512], None, None, 128, 8)
        assert y.shape == (2, 83, 512)
        with pytest.raises(Exception):
            torch.ops.dexter_b200.wq_gemm(x, q8, s, None, None, 128, 4)  # K = 6144 != 3072
