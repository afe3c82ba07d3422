"""``torch.ops.xla.quantized_matmul_int8`` on B200.

Host-side mirror of the W8A8 entry of the reference's Pallas registry
(torch_xla/experimental/custom_kernel.py:1066-1106 wrapper, :1742-1782 schema and kernels;
kernel body torch_xla/experimental/pallas_kernels/quantized_matmul_kernel.py:38-126, 171-310).

Same schema; the result always has ``x.dtype`` (:1105-1106, quantized_matmul_kernel.py:297).
Like the reference wrapper, caller-supplied block sizes are accepted and ignored (:1088): tiling is
the kernel's own business (128x256x128 tcgen05 tiles here, the tuned TPU table there).
``zero_point`` and ``quant_block_size`` are rejected like the Pallas wrapper does
(quantized_matmul_kernel.py:192-193).
"""
import torch

from . import _capi
from . import quantized_matmul as _qm

SCHEMA = ("quantized_matmul_int8(Tensor x, Tensor w, Tensor scalar, Tensor? zero_point=None, "
          "Tensor? quant_block_size=None, bool quantize_activation=False, int? batch_block_size=None, "
          "int? out_block_size=None, int? in_block_size=None) -> Tensor")

if not _qm.has_xla_op("quantized_matmul_int8"):
  _qm.XLA_LIB.define(SCHEMA)


def quantized_matmul_int8(x, w, scalar, zero_point=None, quant_block_size=None,
                          quantize_activation=False, batch_block_size=None, out_block_size=None,
                          in_block_size=None):
  assert zero_point is None, "Not implemented: zero_point is not supported."
  assert quant_block_size is None, "Not implemented: quant_block_size is not supported."
  assert x.dim() == 2, f"x is expected to be 2D [bs, n_input_features], got {x.dim()}D Tensor."
  _capi.require_cuda(x, w, scalar)
  _qm._check_per_channel_quant_weight_dtype_shapes(x.shape[1], scalar.shape[0], w, scalar, None)
  x2 = _qm._rows(x)
  M, K = x2.shape
  N = w.shape[0]
  w = w if w.is_contiguous() else w.contiguous()
  s32 = _qm._f32(scalar)
  with torch.cuda.device(x.device):
    if quantize_activation:
      return _qm._w8a8(x2, w, s32, None, x.dtype)
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    ws, ws_bytes = _capi.workspace(x.device, M, K)
    _capi.check(_capi.lib().qmm_weight_only(
        8, _capi.ptr(x2), _capi.dtype_code(x2.dtype), _capi.ptr(w), _capi.ptr(s32), None, _capi.ptr(out),
        _capi.dtype_code(x.dtype), M, N, K, 0, _capi.VARIANTS[_qm.current_variant()], ws, ws_bytes,
        _capi.stream_ptr(x.device)))
    return out


def quantized_matmul_int8_meta(x, w, scalar, zero_point=None, quant_block_size=None,
                               quantize_activation=False, batch_block_size=None, out_block_size=None,
                               in_block_size=None):
  # shape-only kernel used while tracing (reference: custom_kernel.py:1764-1782)
  return torch.empty(x.shape[0], w.shape[0], device=x.device, dtype=x.dtype)


_qm.XLA_LIB.impl("quantized_matmul_int8", quantized_matmul_int8, "CUDA")
_qm.XLA_LIB.impl("quantized_matmul_int8", quantized_matmul_int8_meta, "Meta")
