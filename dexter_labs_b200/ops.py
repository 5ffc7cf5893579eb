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
import weakref
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from .platform import ArchVersion, Capability
from .registry import Priority, register, select

__all__ = ["w4a16", "w8a16", "w4a16_gelu", "w8a16_gelu", "linear", "dequantize", "accepts", "KERNEL_NAMES",
           "register_with", "last_status", "PeerAllReduce",
           "FusedReduce", "relayout_w4", "prepared_w4", "set_wait_limit_ms"]

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


_LAYOUTS = {"dexter": _lib.LAYOUT_DEXTER, "b200": _lib.LAYOUT_B200}
_EPILOGUES = {None: _lib.EPILOGUE_NONE, "gelu_tanh": _lib.EPILOGUE_GELU_TANH}
_need_cache: Dict[Tuple[int, int, int, int, int], int] = {}  # workspace bytes per problem
_opts_cache: Dict[tuple, "_lib.GemmOpts"] = {}  # option structs of calls without a fused sum
# (device, stream) -> (workspace tensor, its address, its size): see _workspace
_ws_fast: Dict[Tuple[int, int], Tuple[torch.Tensor, int, int]] = {}
_GEMM = _LIB.dxb_wq_gemm_ex
_FAST = None if os.environ.get("DEXTER_B200_FASTCALL", "1") == "0" else _lib.load_fast()
_raw_stream = torch._C._cuda_getCurrentRawStream
_current_device = torch.cuda.current_device


def _run(bits: int, x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
         zeros: Optional[torch.Tensor], bias: Optional[torch.Tensor], group_size: int,
         max_ctas: int = 0, *, layout: str = "dexter", epilogue: Optional[str] = None,
         reduce: Optional["FusedReduce"] = None) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("the B200 backend needs CUDA tensors; there is no CPU path")
    if x.dtype != torch.bfloat16 or scales.dtype != torch.bfloat16:
        raise RuntimeError("the B200 backend computes bf16 activations with bf16 scales only")
    if qweight.dtype != torch.uint8:
        raise ValueError("packed weights must be uint8")
    rows, n = qweight.shape
    k_dim = rows * 2 if bits == 4 else rows
    k_in = x.shape[-1]
    if k_in != k_dim:
        raise ValueError(f"x has K={k_in} but the packed weight has K={k_dim}")
    # A weight tensor that has to be copied here is written by the kernel right before the
    # GEMM on this stream, which the GEMM must then not overtake (it normally starts early
    # and reads its weights at once): such a call is launched in plain stream order.
    copied = False
    if not qweight.is_contiguous():
        if layout != "dexter":
            raise ValueError("a re-laid-out weight must be contiguous")
        qweight, copied = qweight.contiguous(), True
    if not scales.is_contiguous():
        scales, copied = scales.contiguous(), True
    if zeros is not None and not zeros.is_contiguous():
        zeros, copied = zeros.contiguous(), True
    if bias is not None and not bias.is_contiguous():
        bias, copied = bias.contiguous(), True

    x2 = x if x.dim() == 2 else x.reshape(-1, k_in)
    if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    m = x2.shape[0]
    out = torch.empty((m, n), device=x.device, dtype=torch.bfloat16)
    if m == 0:
        return out if x.dim() == 2 else out.view(*x.shape[:-1], n)

    dev = x.device.index
    if dev != _current_device():
        with torch.cuda.device(dev):
            return _run(bits, x, qweight, scales, zeros, bias, group_size, max_ctas, layout=layout,
                        epilogue=epilogue, reduce=reduce)
    if layout == "dexter" and bits == 4:
        # load-time repack, cached per weight tensor (see prepared_w4)
        relaid = None if copied else prepared_w4(qweight, m, n, k_dim, group_size)
        if relaid is not None:
            # a copy made just now was written by the kernel right before this GEMM
            copied = relaid[1]
            qweight, layout = relaid[0], "b200"
    stream = _raw_stream(dev)
    ws = _ws_fast.get((dev, stream))
    key = (m, n, k_dim, bits, max_ctas)
    need = _need_cache.get(key)
    if need is None:
        need = _need_cache[key] = _LIB.dxb_workspace_bytes_ex(m, n, k_dim, bits, max_ctas)
    if ws is None or ws[2] < need:
        t = _workspace(x.device, stream, need)
        ws = _ws_fast[(dev, stream)] = (t, t.data_ptr(), t.numel())
    if reduce is None and _FAST is not None:
        # compiled binding: same entry point, arguments as plain integers (0 = NULL)
        rc = _FAST(bits, x2.data_ptr(), x2.stride(0), qweight.data_ptr(), scales.data_ptr(),
                   0 if zeros is None else zeros.data_ptr(), 0 if bias is None else bias.data_ptr(),
                   out.data_ptr(), n, m, n, k_dim, group_size, ws[1], ws[2], _LAYOUTS[layout],
                   _EPILOGUES[epilogue], max_ctas, 1 if copied else 0, stream)
        if rc != 0:
            _raise(rc)
        if _CHECK:
            code = _LIB.dxb_read_status(ws[1], ctypes.c_void_p(stream))
            if code != _lib.OK:
                ws[0].zero_()
                _raise(code)
        return out if x.dim() == 2 else out.view(*x.shape[:-1], n)
    if reduce is None:
        okey = (layout, epilogue, max_ctas, copied)
        opts = _opts_cache.get(okey)  # read-only for the library: one struct per combination
        if opts is None:
            opts = _opts_cache[okey] = _lib.GemmOpts(_LAYOUTS[layout], _EPILOGUES[epilogue], max_ctas, 0, 0,
                                                     None, 0, 1 if copied else 0)
    else:
        opts = _lib.GemmOpts(_LAYOUTS[layout], _EPILOGUES[epilogue], max_ctas, reduce.world, reduce.rank,
                             reduce._ptrs, reduce.capacity, 1 if copied else 0)
    rc = _GEMM(bits, x2.data_ptr(), x2.stride(0), qweight.data_ptr(), scales.data_ptr(),
               None if zeros is None else zeros.data_ptr(), None if bias is None else bias.data_ptr(),
               out.data_ptr(), n, m, n, k_dim, group_size, ws[1], ws[2], opts, stream)
    if rc != 0:
        _raise(rc)
    if _CHECK:
        code = _LIB.dxb_read_status(ws[1], ctypes.c_void_p(stream))
        if code != _lib.OK:
            ws[0].zero_()
            _raise(code)
    return out if x.dim() == 2 else out.view(*x.shape[:-1], n)


_CHECK = bool(os.environ.get("DEXTER_B200_CHECK"))

# ------------------------------------------------------------ load-time re-layout (int4)
# id(qweight) -> (weak reference to it, its version counter, the repacked copy)
_relaid: Dict[int, Tuple[object, int, torch.Tensor]] = {}
_AUTO_RELAYOUT = os.environ.get("DEXTER_B200_RELAYOUT", "1") != "0"


def relayout_w4(qweight: torch.Tensor, *, inverse: bool = False,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Repack an int4 ``qweight`` ``[K/2, N]`` for the tensor-core kernel (``layout="b200"``).

    The reference names this as its own next step ("pack into int32 words",
    ``README.md:147-150`` there): inside every block of 2 packed rows x 4 columns the
    nibbles are regrouped so that a 32-bit word holds, for four columns, the two values
    of consecutive k the tensor-core operand pairs up.  Same shape; ``inverse=True`` gives
    the reference layout back bit for bit; ``out`` may be ``qweight`` itself.
    """
    if qweight.dtype != torch.uint8 or qweight.ndim != 2 or not qweight.is_cuda:
        raise ValueError("relayout_w4 takes a 2-D uint8 CUDA tensor")
    rows, n = qweight.shape
    if rows % 2 or n % 4:
        raise ValueError("relayout_w4 needs an even number of packed rows and N % 4 == 0")
    src = qweight if qweight.is_contiguous() else qweight.contiguous()
    dst = torch.empty_like(src) if out is None else out
    if dst.shape != src.shape or not dst.is_contiguous() or dst.dtype != torch.uint8:
        raise ValueError("out must be a contiguous uint8 tensor of the same shape")
    with torch.cuda.device(qweight.device):
        stream = _raw_stream(qweight.device.index)
        rc = _LIB.dxb_relayout_w4(src.data_ptr(), dst.data_ptr(), 2 * rows, n, 1 if inverse else 0,
                                  ctypes.c_void_p(stream))
    if rc != _lib.OK:
        _raise(rc)
    return dst


def prepared_w4(qweight: torch.Tensor, m: int, n: int, k_dim: int,
                group_size: int) -> Optional[Tuple[torch.Tensor, bool]]:
    """The cached repacked copy of ``qweight`` for calls that come in with the reference
    layout (the registered kernels), as ``(copy, made_just_now)``, or None where the repack
    does not apply: shapes the plain CUDA-core kernel serves, a stream that is being captured
    before the copy exists, ``DEXTER_B200_RELAYOUT=0``.  The copy is made on the first call
    with a given tensor object and dropped when that tensor is freed or modified in place."""
    if not _AUTO_RELAYOUT:
        return None
    key = id(qweight)
    hit = _relaid.get(key)
    if hit is not None and hit[0]() is qweight and hit[1] == qweight._version:
        return hit[2], False
    if (qweight.shape[0] % 2 or n % 4 or qweight.data_ptr() % 16
            or not _LIB.dxb_uses_tensor_cores(m, n, k_dim, group_size, 4)
            or torch.cuda.is_current_stream_capturing()):
        return None
    relaid = relayout_w4(qweight)
    _relaid[key] = (weakref.ref(qweight, lambda _r, key=key: _relaid.pop(key, None)),
                    qweight._version, relaid)
    return relaid, True


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


def w4a16(x, qweight, scales, zeros, bias, group_size, *, max_ctas: int = 0, layout: str = "dexter",
          epilogue: Optional[str] = None, reduce: Optional["FusedReduce"] = None):
    """int4 weight-only GEMM, bf16 in / bf16 out.

    Extensions beyond the reference's kernel-slot signature, all keyword-only:
    ``max_ctas`` caps the SMs the launch may use, for callers that run independent GEMMs
    on parallel streams; ``layout="b200"`` says ``qweight`` already went through
    :func:`relayout_w4` (with the default the repack is made once and cached);
    ``epilogue="gelu_tanh"`` applies the tanh-GELU of the FFN to the result;
    ``reduce`` (a :class:`FusedReduce`) makes the call one rank's K-shard of a
    row-parallel linear and returns the sum over ranks.
    """
    if _plain_call(max_ctas, layout, epilogue, reduce) and torch.compiler.is_compiling():
        return torch.ops.dexter_b200.wq_gemm(x, qweight, scales, zeros, bias, group_size, 4)
    return _run(4, x, qweight, scales, zeros, bias, group_size, max_ctas, layout=layout,
                epilogue=epilogue, reduce=reduce)


def _plain_call(max_ctas, layout, epilogue, reduce) -> bool:
    return max_ctas == 0 and layout == "dexter" and epilogue is None and reduce is None


def w8a16(x, qweight, scales, zeros, bias, group_size, *, max_ctas: int = 0,
          epilogue: Optional[str] = None, reduce: Optional["FusedReduce"] = None):
    """int8 weight-only GEMM, bf16 in / bf16 out (keywords: see :func:`w4a16`)."""
    if _plain_call(max_ctas, "dexter", epilogue, reduce) and torch.compiler.is_compiling():
        return torch.ops.dexter_b200.wq_gemm(x, qweight, scales, zeros, bias, group_size, 8)
    return _run(8, x, qweight, scales, zeros, bias, group_size, max_ctas, epilogue=epilogue,
                reduce=reduce)


def w4a16_gelu(x, qweight, scales, zeros, bias, group_size):
    """``gelu_tanh(w4a16(x, ...))`` in one launch: the FFN up-projection with the activation
    the reference applies between its packed FFN linears
    (``python/dexter/models/dreamzero/model.py:279-285``) in the GEMM epilogue."""
    return _run(4, x, qweight, scales, zeros, bias, group_size, epilogue="gelu_tanh")


def w8a16_gelu(x, qweight, scales, zeros, bias, group_size):
    """int8 counterpart of :func:`w4a16_gelu`."""
    return _run(8, x, qweight, scales, zeros, bias, group_size, epilogue="gelu_tanh")


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


class FusedReduce:
    """Peer-mapped memory for the sum over ranks that ``w4a16(..., reduce=...)`` fuses into a
    row-parallel GEMM (``dxb_wq_gemm_ex`` with ``peer_*`` options).

    Built once per process group (a collective: every rank constructs it at the same point):
    allocates this rank's region through ``torch.distributed._symmetric_memory``, zero-fills
    it and exchanges the mappings.  Every rank then makes the same sequence of
    ``reduce=``-calls with the same M and N (at most 128 tokens, ``M * N <= capacity``),
    passes the FULL bias, and gets the full result.
    """

    def __init__(self, group, capacity_elems: int, device: torch.device) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.capacity = (int(capacity_elems) + 7) // 8 * 8
        nbytes = _LIB.dxb_fused_reduce_bytes(self.world, self.capacity)
        if nbytes == 0:
            raise RuntimeError("the fused sum over ranks supports at most 8 ranks")
        # plain peer mappings are all the kernel uses: keep the region off NVLink multicast
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        with torch.cuda.device(device):
            self.region = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            self.region.zero_()
            self.handle = symm_mem.rendezvous(self.region, group.group_name)
            torch.cuda.synchronize()
        dist.barrier(group)  # every region is zero before anyone's first call
        self._ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self.handle.buffer_ptrs])


def set_wait_limit_ms(ms: int) -> None:
    """Upper bound of a kernel's wait for another GPU (``dxb_set_wait_limit_ms``)."""
    _LIB.dxb_set_wait_limit_ms(int(ms))


def dequantize(qweight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor],
               group_size: int, bits: int, *, layout: str = "dexter") -> torch.Tensor:
    """Dense ``[K, N]`` bf16 weight from the CUDA kernel's own arithmetic.

    Counterpart of the reference's ``dequantize`` (``reference/gemm.py:51-73``);
    exists so the dequantisation can be compared bit for bit.  ``layout="b200"``:
    ``qweight`` went through :func:`relayout_w4`.
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
        rc = _LIB.dxb_dequantize_ex(qweight.contiguous().data_ptr(), scales.contiguous().data_ptr(),
                                    None if zeros is None else zeros.contiguous().data_ptr(),
                                    out.data_ptr(), n, k_dim, group_size, bits, _LAYOUTS[layout],
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
