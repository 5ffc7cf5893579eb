"""The ``gemm/w4a16`` and ``gemm/w8a16`` kernels for B200, and their registration.

The two functions here have the reference's kernel-slot signature
``impl(x, qweight, scales, zeros, bias, group_size) -> Tensor``
(``python/dexter/ops/reference/gemm.py:82-89``; host glue mirrored from
``python/dexter/ops/gfx1151/gemm/quantized.py:223-263``): leading dimensions of
``x`` are flattened, a non-unit inner stride is made contiguous, a K mismatch is
a ``ValueError``, and a new ``[..., N]`` tensor is returned.  All arithmetic runs
in the CUDA library behind ``include/dexter_b200.h``; torch only provides device
memory and the current stream.  Nothing here runs without that library.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from .platform import ArchVersion, Capability
from .registry import Priority, register, select

__all__ = ["w4a16", "w8a16", "linear", "dequantize", "accepts", "KERNEL_NAMES", "register_with",
           "last_status", "chain", "chain_status", "ChainLink", "CHAIN_MAX", "PeerAllReduce"]

KERNEL_NAMES = {"w4a16": "b200_w4a16_tcgen05", "w8a16": "b200_w8a16_tcgen05"}

_LIB = _lib.load()

# One workspace per (device, stream): status word, tile counters and split-K
# partial sums.  Zero-filled when created; the kernel leaves it clean.
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _raise(code: int) -> None:
    text = f"{_lib.ERRORS.get(code, code)}: {_lib.strerror(code)}"
    if code in (-1, -3):
        raise ValueError(text)
    raise RuntimeError(text)


def _run(bits: int, x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
         zeros: Optional[torch.Tensor], bias: Optional[torch.Tensor], group_size: int,
         max_ctas: int = 0) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("the B200 backend needs CUDA tensors; there is no CPU path")
    if x.dtype != torch.bfloat16 or scales.dtype != torch.bfloat16:
        raise RuntimeError("the B200 backend computes bf16 activations with bf16 scales only")
    if qweight.dtype != torch.uint8:
        raise ValueError("packed weights must be uint8")
    k_dim = qweight.shape[0] * (2 if bits == 4 else 1)
    *lead, k_in = x.shape
    if k_in != k_dim:
        raise ValueError(f"x has K={k_in} but the packed weight has K={k_dim}")
    n = qweight.shape[1]
    qweight = qweight if qweight.is_contiguous() else qweight.contiguous()
    scales = scales if scales.is_contiguous() else scales.contiguous()
    if zeros is not None and not zeros.is_contiguous():
        zeros = zeros.contiguous()
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()

    x2 = x.reshape(-1, k_in)
    if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    m = x2.shape[0]
    out = torch.empty((m, n), device=x.device, dtype=x.dtype)
    if m == 0:
        return out.view(*lead, n)

    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        need = _LIB.dxb_workspace_bytes(m, n, k_dim, bits)
        ws = _workspace(x.device, stream, need)
        rc = _LIB.dxb_wq_gemm(bits, x2.data_ptr(), x2.stride(0), qweight.data_ptr(),
                              scales.data_ptr(), _ptr(zeros), _ptr(bias), out.data_ptr(), n, m, n,
                              k_dim, group_size, ws.data_ptr(), ws.numel(), max_ctas,
                              ctypes.c_void_p(stream))
        if rc != _lib.OK:
            _raise(rc)
        if os.environ.get("DEXTER_B200_CHECK"):
            code = _LIB.dxb_read_status(ws.data_ptr(), ctypes.c_void_p(stream))
            if code != _lib.OK:
                ws.zero_()
                _raise(code)
    return out.view(*lead, n)


def last_status(device: Optional[torch.device] = None) -> int:
    """Synchronise and return the kernel status word of the current stream's workspace."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream().cuda_stream
        ws = _workspaces.get((device.index, stream))
        if ws is None:
            return _lib.OK
        return _LIB.dxb_read_status(ws.data_ptr(), ctypes.c_void_p(stream))


def accepts(*args) -> bool:
    """Shape predicate of the registered kernels (``registry.py:58-60`` in the reference).

    Called with ``(x, qweight, scales)`` by ``linear`` and with no arguments by
    benchmarks that only want the kernel for this platform.
    """
    if not args:
        return True
    x, qweight, scales = args[:3]
    return bool(x.is_cuda and x.dtype == torch.bfloat16 and scales.dtype == torch.bfloat16
                and qweight.dtype == torch.uint8 and qweight.ndim == 2 and scales.ndim == 2)


def w4a16(x, qweight, scales, zeros, bias, group_size, *, max_ctas: int = 0):
    """int4 weight-only GEMM, bf16 in / bf16 out.

    ``max_ctas`` (an extension, not part of the reference signature) caps the SMs the
    launch may use, for callers that run independent GEMMs on parallel streams.
    """
    return _run(4, x, qweight, scales, zeros, bias, group_size, max_ctas)


def w8a16(x, qweight, scales, zeros, bias, group_size, *, max_ctas: int = 0):
    """int8 weight-only GEMM, bf16 in / bf16 out (``max_ctas``: see :func:`w4a16`)."""
    return _run(8, x, qweight, scales, zeros, bias, group_size, max_ctas)


CHAIN_MAX = _lib.DXB_CHAIN_MAX


class ChainLink:
    """One GEMM of a :func:`chain`: the kernel-slot arguments plus where ``x`` comes from.

    ``x`` is either a tensor that is ready before the call, or the integer index of an
    EARLIER link whose output is this link's activations.
    """

    __slots__ = ("x", "qweight", "scales", "zeros", "bias", "group_size")

    def __init__(self, x, qweight, scales, zeros=None, bias=None, group_size=128):
        self.x, self.qweight, self.scales = x, qweight, scales
        self.zeros, self.bias, self.group_size = zeros, bias, group_size


# One chain workspace per (device, stream): zero-filled when created; the kernel leaves it clean.
_chain_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def chain(links, *, bits: int = 4, max_ctas: int = 0):
    """Run a list of quantised GEMMs (at most ``CHAIN_MAX``) as ONE launch.

    Each link computes what ``w4a16`` / ``w8a16`` would; links are started in list order
    by one persistent grid, and a link whose ``x`` is an index waits in the kernel for
    that link's output instead of for a kernel boundary.  Returns the list of outputs.
    All links need at most 128 token rows and shapes the tensor-core kernel takes;
    otherwise the library refuses (``RuntimeError``) and the caller should issue the
    GEMMs one by one.
    """
    if bits not in (4, 8):
        raise ValueError(f"weight-only quantisation supports 4 or 8 bits, got {bits}")
    links = list(links)
    if not 1 <= len(links) <= CHAIN_MAX:
        raise ValueError(f"a chain holds 1..{CHAIN_MAX} GEMMs, got {len(links)}")
    items = (_lib.ChainItem * len(links))()
    outs, keep = [], []
    device = links[0].qweight.device
    if device.type != "cuda":
        raise RuntimeError("the B200 backend needs CUDA tensors; there is no CPU path")
    for i, ln in enumerate(links):
        k_dim = ln.qweight.shape[0] * (2 if bits == 4 else 1)
        n = ln.qweight.shape[1]
        if isinstance(ln.x, int):
            if not 0 <= ln.x < i:
                raise ValueError(f"link {i} depends on link {ln.x}, which does not come before it")
            x2, dep = outs[ln.x], ln.x
        else:
            x2, dep = ln.x.reshape(-1, ln.x.shape[-1]), -1
            if x2.dtype != torch.bfloat16:
                raise RuntimeError("the B200 backend computes bf16 activations only")
            if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
                x2 = x2.contiguous()
        if x2.shape[1] != k_dim:
            raise ValueError(f"link {i}: x has K={x2.shape[1]} but the packed weight has K={k_dim}")
        if ln.qweight.dtype != torch.uint8 or ln.scales.dtype != torch.bfloat16:
            raise ValueError("packed weights must be uint8 with bf16 scales")
        qweight, scales = ln.qweight.contiguous(), ln.scales.contiguous()
        zeros = None if ln.zeros is None else ln.zeros.contiguous()
        bias = None if ln.bias is None else ln.bias.contiguous()
        m = x2.shape[0]
        out = torch.empty((m, n), device=device, dtype=torch.bfloat16)
        keep.append((x2, qweight, scales, zeros, bias))
        outs.append(out)
        it = items[i]
        it.x, it.ldx = x2.data_ptr(), x2.stride(0)
        it.qweight, it.scales = qweight.data_ptr(), scales.data_ptr()
        it.zeros, it.bias = _ptr(zeros), _ptr(bias)
        it.out, it.ldo = out.data_ptr(), n
        it.M, it.N, it.K, it.group_size = m, n, k_dim, ln.group_size
        it.depends_on = dep
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream().cuda_stream
        need = _LIB.dxb_chain_workspace_bytes(bits, items, len(links), max_ctas)
        if need == 0:
            # let the launch call report why
            need = 256
        key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
        ws = _chain_workspaces.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.zeros(max(need, 256), dtype=torch.uint8, device=device)
            _chain_workspaces[key] = ws
        rc = _LIB.dxb_wq_gemm_chain(bits, items, len(links), ws.data_ptr(), ws.numel(), max_ctas,
                                    ctypes.c_void_p(stream))
        if rc != _lib.OK:
            _raise(rc)
        if os.environ.get("DEXTER_B200_CHECK"):
            code = _LIB.dxb_read_status(ws.data_ptr(), ctypes.c_void_p(stream))
            if code != _lib.OK:
                ws.zero_()
                _raise(code)
    return outs


def chain_status(device: Optional[torch.device] = None) -> int:
    """Synchronise and return the status word of the current stream's chain workspace."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream().cuda_stream
        ws = _chain_workspaces.get((device.index, stream))
        if ws is None:
            return _lib.OK
        return _LIB.dxb_read_status(ws.data_ptr(), ctypes.c_void_p(stream))


class PeerAllReduce:
    """Sum of bf16 partial outputs over the ranks of one NVLink domain (``dxb_peer_allreduce``).

    Built once per process group (a collective: every rank must construct it at the same
    point): allocates this rank's region of peer-mapped memory through
    ``torch.distributed._symmetric_memory``, zero-fills it and exchanges the mappings.
    ``__call__(partial)`` then returns the full sum on every rank with one kernel launch on
    the current stream; all ranks must make the same calls in the same order.
    """

    MAX_BYTES = 1 << 20  # larger messages belong to the library collectives

    def __init__(self, group, capacity_elems: int, device: torch.device) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.capacity = (int(capacity_elems) + 7) // 8 * 8
        nbytes = _LIB.dxb_peer_allreduce_bytes(self.world, self.capacity)
        if nbytes == 0:
            raise RuntimeError("peer all-reduce supports at most 8 ranks")
        name = group.group_name
        # plain peer mappings are all the kernel uses: keep the region off NVLink multicast
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        with torch.cuda.device(device):
            self.region = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            self.region.zero_()
            self.handle = symm_mem.rendezvous(self.region, name)
            self.status = torch.zeros(1, dtype=torch.int32, device=device)
            torch.cuda.synchronize()
        dist.barrier(group)  # every region is zero before anyone's first call
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)

    def __call__(self, partial: torch.Tensor) -> torch.Tensor:
        if partial.dtype != torch.bfloat16 or not partial.is_contiguous():
            raise RuntimeError("peer all-reduce takes contiguous bf16 tensors")
        n = partial.numel()
        if n % 8 or n > self.capacity:
            raise ValueError(f"peer all-reduce: {n} elements (capacity {self.capacity}, multiple of 8)")
        out = torch.empty_like(partial)
        with torch.cuda.device(partial.device):
            stream = torch.cuda.current_stream().cuda_stream
            rc = _LIB.dxb_peer_allreduce(partial.data_ptr(), out.data_ptr(), n, self._ptrs,
                                         self.capacity, self.rank, self.world,
                                         self.status.data_ptr(), ctypes.c_void_p(stream))
        if rc != _lib.OK:
            _raise(rc)
        return out

    def check(self) -> int:
        """Synchronise and return the error word (0, or DXB_ERR_KERNEL_TIMEOUT)."""
        return int(self.status.item())


def dequantize(qweight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor],
               group_size: int, bits: int) -> torch.Tensor:
    """Dense ``[K, N]`` bf16 weight from the CUDA kernel's own arithmetic.

    Counterpart of the reference's ``dequantize`` (``reference/gemm.py:51-73``);
    exists so the dequantisation can be compared bit for bit.
    """
    if bits not in (4, 8):
        raise ValueError(f"weight-only quantisation supports 4 or 8 bits, got {bits}")
    if not qweight.is_cuda:
        raise RuntimeError("the B200 backend needs CUDA tensors; there is no CPU path")
    k_dim = qweight.shape[0] * (2 if bits == 4 else 1)
    n = qweight.shape[1]
    out = torch.empty((k_dim, n), device=qweight.device, dtype=torch.bfloat16)
    with torch.cuda.device(qweight.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = _LIB.dxb_dequantize(qweight.contiguous().data_ptr(), scales.contiguous().data_ptr(),
                                 None if zeros is None else zeros.contiguous().data_ptr(),
                                 out.data_ptr(), n, k_dim, group_size, bits,
                                 ctypes.c_void_p(stream))
    if rc != _lib.OK:
        _raise(rc)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
           scales: Optional[torch.Tensor] = None, zeros: Optional[torch.Tensor] = None,
           group_size: int = 128, bits: int = 4) -> torch.Tensor:
    """Op-surface dispatcher with the reference's signature (``ops/__init__.py:89-113``).

    Only the quantised branch belongs to this backend; a dense call (no
    ``scales``) is outside it and is rejected rather than silently served.
    """
    if scales is None:
        raise NotImplementedError("dense gemm is not part of the B200 weight-only backend")
    if bits not in (4, 8):
        raise ValueError(f"weight-only quantisation supports 4 or 8 bits, got {bits}")
    mode = f"w{bits}a16"
    return select("gemm", mode, x, weight, scales)(x, weight, scales, zeros, bias, group_size)


_CAPABILITY = dict(vendors=frozenset({"nvidia"}), features=frozenset({"matrix:bf16"}))

register("gemm", "w4a16", name=KERNEL_NAMES["w4a16"], priority=Priority.SPECIALISED,
         capability=Capability(min_arch=ArchVersion(10, 0), **_CAPABILITY), accepts=accepts)(w4a16)
register("gemm", "w8a16", name=KERNEL_NAMES["w8a16"], priority=Priority.SPECIALISED,
         capability=Capability(min_arch=ArchVersion(10, 0), **_CAPABILITY), accepts=accepts)(w8a16)


def register_with(dexter_registry, dexter_platform) -> None:
    """Register both kernels in the reference's own registry (``registry.py:73-104``).

    ``dexter_registry`` / ``dexter_platform`` are the imported ``dexter.registry``
    and ``dexter.platform`` modules.  After this, ``dexter.ops.linear``,
    ``dexter.models.layers.Linear`` and ``dexter-bench kernels`` select the B200
    kernels on an sm_100 device with no change to the reference.
    """
    cap = dexter_platform.Capability(vendors=frozenset({"nvidia"}),
                                     min_arch=dexter_platform.ArchVersion(10, 0),
                                     features=frozenset({"matrix:bf16"}))
    for mode, fn in (("w4a16", w4a16), ("w8a16", w8a16)):
        bucket = dexter_registry._REGISTRY.get(f"gemm/{mode}", [])
        if any(spec.name == KERNEL_NAMES[mode] for spec in bucket):
            continue

        def impl(x, qweight, scales, zeros, bias, group_size, _fn=fn):
            return _fn(x, qweight, scales, zeros, bias, group_size)

        dexter_registry.register("gemm", mode, name=KERNEL_NAMES[mode], capability=cap,
                                 priority=dexter_registry.Priority.SPECIALISED,
                                 accepts=accepts)(impl)
