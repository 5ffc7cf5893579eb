"""B200 (sm_100a) backend for dexter's weight-only quantised GEMM (gemm/w4a16, gemm/w8a16).

Importing the package loads the CUDA library (and fails loudly if it has not
been built), registers the two kernels in this package's registry and, when the
reference project is importable, in ``dexter.registry`` as well.
"""
from . import platform, quant, registry  # noqa: F401
from . import ops  # noqa: F401  (loads libdexter_b200.so, registers the kernels)
from . import custom_op  # noqa: F401  (declares torch.ops.dexter_b200.wq_gemm)
from .ops import KERNEL_NAMES, dequantize, linear, w4a16, w8a16  # noqa: F401
from .quant import QuantizedWeight, quantize  # noqa: F401

try:  # the reference is optional; when present, plug into its registry
    import dexter.platform as _dexter_platform
    import dexter.registry as _dexter_registry
except Exception:  # noqa: BLE001 - absent or not importable here
    _dexter_registry = None
else:
    ops.register_with(_dexter_registry, _dexter_platform)

__all__ = ["ops", "quant", "registry", "platform", "quantize", "QuantizedWeight", "linear",
           "w4a16", "w8a16", "dequantize", "KERNEL_NAMES"]
