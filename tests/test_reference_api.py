"""This backend through the reference's REAL plug-in API: its registry, its platform gate, its
op surface, its ``Linear`` module and its kernel micro-benchmark, from the staged copy of
the reference's own modules (``make -C oracle ref REF=<checkout>``; skipped where that
copy does not exist).  The package's own ``quant`` / ``registry`` / ``platform`` modules are
stand-ins for machines without the reference; nothing here uses them.

Reference interfaces exercised (paths inside the reference project):
  python/dexter/registry.py:73-152          register, candidates, select, DEXTER_KERNEL pin
  python/dexter/registry.py:155-173         explain
  python/dexter/platform.py:168-185,275-278 Capability.satisfied_by, override_platform
  python/dexter/ops/__init__.py:89-113      ops.linear
  python/dexter/models/layers.py:35-50      Linear.quantize_ / forward
  python/dexter/bench/kernels.py:59-74      the quantised rows of `dexter-bench kernels`
"""
import numpy as np
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="no staged reference under oracle/_ref")
TOL = 1e-2


def err(got, want):
    got, want = got.double(), want.double()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-6)


@pytest.fixture(scope="module")
def dexter(b200_lib):
    mods = ref.activate()
    import dexter_labs_b200 as pkg

    pkg.ops.register_with(mods["registry"], mods["platform"])
    mods["pkg"] = pkg
    return mods


def _fake_nvidia(platform, major, name):
    return platform.PlatformInfo(vendor="nvidia", arch=f"sm{major}0", arch_version=platform.ArchVersion(major, 0),
                                 family="NVIDIA", device_name=f"{name} (faked for the gate)", compute_units=148,
                                 wavefront=32, lds_bytes=49152, total_memory=180 << 30, memory_bandwidth=0.0,
                                 features=frozenset({"matrix:f16", "matrix:bf16", "mma:mma"}))


def _fake_b200(platform):
    return _fake_nvidia(platform, 10, "NVIDIA B200")


def _fake_hopper(platform):
    return _fake_nvidia(platform, 9, "NVIDIA H100")


class forced:
    """`with forced(platform_module, info):` around the reference's override_platform
    (python/dexter/platform.py:275-278), which is a plain setter."""

    def __init__(self, platform, info):
        self.platform, self.info = platform, info

    def __enter__(self):
        self.platform.override_platform(self.info)

    def __exit__(self, *exc):
        self.platform.override_platform(None)


# ----------------------------------------------------------------- no GPU needed
def test_registration_is_idempotent_and_visible(dexter):
    reg, pkg = dexter["registry"], dexter["pkg"]
    pkg.ops.register_with(reg, dexter["platform"])  # a second time: nothing is added, nothing raises
    for mode in ("w4a16", "w8a16"):
        names = [s.name for s in reg._REGISTRY[f"gemm/{mode}"]]
        assert names.count(pkg.KERNEL_NAMES[mode]) == 1
        assert f"torch_{mode}" in names
        ours = next(s for s in reg._REGISTRY[f"gemm/{mode}"] if s.name == pkg.KERNEL_NAMES[mode])
        assert int(ours.priority) == int(reg.Priority.SPECIALISED) == 12
        assert reg._REGISTRY[f"gemm/{mode}"][0] is ours  # buckets are sorted by priority


def test_selected_on_a_b200_platform_and_only_there(dexter):
    reg, platform, pkg = dexter["registry"], dexter["platform"], dexter["pkg"]
    with forced(platform, _fake_b200(platform)):
        text = reg.explain("gemm", "w4a16")
        line = next(ln for ln in text.splitlines() if "b200_w4a16_tcgen05" in ln)
        assert "SELECTED (pri=12)" in line
        # the kernel micro-benchmark asks with no shape arguments (bench/kernels.py:66)
        assert reg.select("gemm", "w8a16").__defaults__[0] is pkg.ops.w8a16
        assert reg.select("gemm", "w4a16").__defaults__[0] is pkg.ops.w4a16
    with forced(platform, _fake_hopper(platform)):  # below sm_100: gated off
        assert "skipped" in next(ln for ln in reg.explain("gemm", "w4a16").splitlines()
                                 if "b200_w4a16_tcgen05" in ln)
        ref_impl = next(s.impl for s in reg._REGISTRY["gemm/w4a16"] if s.name == "torch_w4a16")
        assert reg.select("gemm", "w4a16") is ref_impl
    # on this machine's real platform (the CPU fallback here, a B200 on the GPU box) the answer
    # follows the same gate
    real = platform.current_platform()
    chosen = reg.select("gemm", "w4a16")
    if real.vendor == "nvidia" and real.arch_version >= platform.ArchVersion(10, 0):
        assert chosen.__defaults__[0] is pkg.ops.w4a16
    else:
        assert chosen is next(s.impl for s in reg._REGISTRY["gemm/w4a16"] if s.name == "torch_w4a16")


def test_dexter_kernel_pin_selects_the_reference_or_us(dexter, monkeypatch):
    reg, platform, pkg = dexter["registry"], dexter["platform"], dexter["pkg"]
    ref_impl = next(s.impl for s in reg._REGISTRY["gemm/w4a16"] if s.name == "torch_w4a16")
    with forced(platform, _fake_b200(platform)):
        monkeypatch.setenv("DEXTER_KERNEL", "gemm/w4a16:torch_w4a16")
        assert reg.select("gemm", "w4a16") is ref_impl
        monkeypatch.setenv("DEXTER_KERNEL", "gemm/w4a16:b200_w4a16_tcgen05")
        assert reg.select("gemm", "w4a16").__defaults__[0] is pkg.ops.w4a16
        monkeypatch.setenv("DEXTER_KERNEL", "gemm/w4a16:no_such_kernel")
        with pytest.raises(LookupError):
            reg.select("gemm", "w4a16")
    with forced(platform, _fake_hopper(platform)):
        monkeypatch.setenv("DEXTER_KERNEL", "gemm/w4a16:b200_w4a16_tcgen05")
        with pytest.raises(LookupError):  # pinned, but not available on that platform
            reg.select("gemm", "w4a16")


def test_cpu_tensors_fall_through_to_the_reference_kernel(dexter):
    """`accepts` declines CPU tensors, so on a faked B200 platform a CPU call still lands on the
    reference's torch kernel (python/dexter/registry.py:144-147): the backend has no CPU path
    and does not pretend to."""
    ops, quant, platform = dexter["ops"], dexter["quant"], dexter["platform"]
    torch.manual_seed(0)
    x = torch.randn(4, 256).to(torch.bfloat16)
    p = quant.quantize((torch.randn(128, 256) * 0.05).to(torch.bfloat16), bits=4)
    with forced(platform, _fake_b200(platform)):
        y = ops.linear(x, p.qweight, None, scales=p.scales, zeros=p.zeros, group_size=128, bits=4)
    ref_impl = next(s.impl for s in dexter["registry"]._REGISTRY["gemm/w4a16"] if s.name == "torch_w4a16")
    assert torch.equal(y, ref_impl(x, p.qweight, p.scales, p.zeros, None, 128))


def test_stand_in_quantiser_equals_the_reference_quantiser(dexter):
    """The package's quantiser stand-in against the reference's own, on fresh random weights."""
    from dexter_labs_b200.quant import quantize as ours

    theirs = dexter["quant"].quantize
    torch.manual_seed(11)
    w = (torch.randn(96, 512) * 0.03).to(torch.bfloat16)
    for bits in (4, 8):
        for sym in (True, False):
            a, b = ours(w, bits=bits, group_size=128, symmetric=sym), theirs(w, bits=bits, group_size=128,
                                                                            symmetric=sym)
            assert torch.equal(a.qweight, b.qweight) and torch.equal(a.scales, b.scales)
            assert (a.zeros is None) == (b.zeros is None)
            if a.zeros is not None:
                assert torch.equal(a.zeros, b.zeros)
            assert a.nbytes == b.nbytes and tuple(a.shape) == tuple(b.shape)


# --------------------------------------------------------------------- on a B200
def _reference_impl(dexter, mode):
    return next(s.impl for s in dexter["registry"]._REGISTRY[f"gemm/{mode}"] if int(s.priority) == 0)


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("shape", [(3072, 3072, True, 83), (256, 128, False, 8)])
def test_reference_linear_module_runs_on_this_backend(dexter, bits, shape):
    k, n, bias, m = shape
    from dexter.models.layers import Linear

    torch.manual_seed(bits + k)
    layer = Linear(k, n, bias=bias).cuda()
    if bias:
        torch.nn.init.normal_(layer.bias, std=0.1)
    x = torch.randn(2, m, k, device="cuda").to(torch.bfloat16)  # leading dims, as the model passes them
    layer.quantize_(bits)  # the model path: asymmetric grid, group 128 (models/layers.py:35-43)
    assert layer.packed is not None and layer.packed.zeros is not None and layer.weight is None
    line = next(ln for ln in dexter["registry"].explain("gemm", f"w{bits}a16").splitlines()
                if f"b200_w{bits}a16_tcgen05" in ln)
    assert "SELECTED" in line  # the real platform detection on this box picks the backend
    y = layer(x)
    p = layer.packed
    want = _reference_impl(dexter, f"w{bits}a16")(x, p.qweight, p.scales, p.zeros, p.bias, p.group_size)
    assert y.shape == (2, m, n) and y.dtype == torch.bfloat16 and torch.isfinite(y.float()).all()
    assert err(y.float(), want.float()) < TOL
    assert dexter["pkg"].ops.last_status() == 0


@pytest.mark.gpu
def test_reference_test_shape_through_ops_linear(dexter):
    """The reference's own kernel test (test/test_ops.py:68-80): 125 x 3072 x 8192, both widths,
    both grids, selected kernel against the REFERENCE kernel -- at 1e-2 instead of its 3e-2."""
    ops, quant = dexter["ops"], dexter["quant"]
    torch.manual_seed(0)
    m, k, n = 125, 3072, 8192
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16) * 0.1
    w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.05
    for bits in (4, 8):
        for sym in (False, True):
            p = quant.quantize(w, bits=bits, group_size=128, symmetric=sym)
            got = ops.linear(x, p.qweight, None, scales=p.scales, zeros=p.zeros, group_size=128, bits=bits)
            want = _reference_impl(dexter, f"w{bits}a16")(x, p.qweight, p.scales, p.zeros, None, 128)
            assert err(got.float(), want.float()) < TOL, (bits, sym)
            dense = x @ w.t()
            assert err(got.float(), dense.float()) < (0.25 if bits == 4 else 0.05)


@pytest.mark.gpu
def test_reference_kernel_benchmark_times_this_backend(dexter):
    """The quantised rows of the reference's `dexter-bench kernels` select with no shape
    arguments and time whatever comes back (bench/kernels.py:59-74): it must be this backend."""
    from dexter.bench import kernels

    reg, pkg = dexter["registry"], dexter["pkg"]
    for mode, fn in (("w4a16", pkg.ops.w4a16), ("w8a16", pkg.ops.w8a16)):
        assert reg.select("gemm", mode).__defaults__[0] is fn
    rows = kernels.run()
    quant_rows = {r["op"]: r for r in rows if r["op"].startswith("gemm w")}
    assert set(quant_rows) == {"gemm w8a16", "gemm w4a16"}
    for r in quant_rows.values():
        assert np.isfinite(r["fused_ms"]) and r["fused_ms"] > 0 and r["gbps"] > 0
