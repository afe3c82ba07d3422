"""B200-native drop-in for PyTorch/XLA's weight-quantized linear path.

Importing the package registers ``torch.ops.xla.quantized_matmul``,
``torch.ops.xla.quantized_matmul_int8``, ``torch.ops.xla_b200.quantized_matmul_packed`` and
``torch.ops.xla_b200.quantized_gate_up`` for the CUDA dispatch key.  The kernels live in ``xla_b200/lib/libqmm_b200.so`` (C ABI:
``include/qmm_b200.h``); build it with ``python -m xla_b200._build``.
"""
from . import _capi  # noqa: F401
from .quantized_matmul import (XlaQuantizedLinear, force_variant, quantize_tensor,  # noqa: F401
                               set_activation_limbs, set_activation_saturation, set_prepack_cache)
from . import custom_kernel  # noqa: F401
from . import packed  # noqa: F401
from .packed import pack_int4, quantized_matmul_packed, unpack_int4  # noqa: F401
from . import mlp  # noqa: F401
from .mlp import concat_projections, interleave_gate_up, quantized_gate_up, split_outputs  # noqa: F401
from .host import HostLinear, HostPipeline  # noqa: F401

__all__ = [
    "XlaQuantizedLinear", "force_variant", "quantize_tensor", "set_activation_limbs", "set_activation_saturation", "set_prepack_cache", "pack_int4",
    "unpack_int4", "quantized_matmul_packed", "interleave_gate_up", "quantized_gate_up", "concat_projections",
    "split_outputs", "HostPipeline", "HostLinear"
]
