"""Weight preparation for the quantized linear: round-to-nearest quantizer and module swap.

The reference keeps these pieces in its test helper (test/quantized_ops/test_quantized_matmul.py:25-105,
``weight_quantization_rtn`` and ``replace_with_xla_quantized_matmul``) and sketches the module swap in
docs/source/perf/quantized_ops.md:92-109.  This module gives them as library functions that produce
exactly the tensors ``XlaQuantizedLinear.load_quantized_weight`` expects:

  per-channel : weight int8 [out, in],            scaler [out],           zero_point [out] or None
  blockwise   : weight int8 [in/bs, bs, out],     scaler [in/bs, out],    zero_point [in/bs, out] or None

The zero point is returned in scaled floating units (``zero_point_int * scaler``), which is what the
operator subtracts (the reference test does the same multiplication before loading).
Works on CPU and CUDA tensors (plain PyTorch arithmetic; this is off-line preparation, not a hot path).
"""
import torch
from torch.ao.quantization.utils import determine_qparams

from .quantized_matmul import XlaQuantizedLinear


def quantize_rtn(w_fp, n_bits=8, block_size=-1, symmetric=True):
  """Round-to-nearest quantization of a Linear weight [out, in] to ``n_bits`` (held in int8)."""
  assert w_fp.dim() == 2, "expected a Linear weight [out_features, in_features]"
  out_dim, in_dim = w_fp.shape
  groups = w_fp
  if block_size != -1:
    assert in_dim % block_size == 0, (f"input_dim should be divisible by block_size, "
                                      f"got input_dim: {in_dim}, block_size: {block_size}.")
    groups = w_fp.reshape(out_dim * in_dim // block_size, block_size)
  lo, hi = torch.aminmax(groups, dim=1)
  qmin, qmax = -2**(n_bits - 1), 2**(n_bits - 1) - 1
  scheme = torch.per_channel_symmetric if symmetric else torch.per_channel_affine
  scale, zp_int = determine_qparams(lo, hi, qmin, qmax, dtype=torch.int8,
                                    eps=torch.tensor([1e-5], device=w_fp.device), has_customized_qrange=False,
                                    qscheme=scheme)
  scale = scale.to(w_fp.dtype).to(w_fp.device)
  zp_int = zp_int.to(w_fp.device)
  q = torch.clamp(torch.round(groups / scale.unsqueeze(1)) + zp_int.unsqueeze(1), qmin, qmax).to(torch.int8)
  zero_point = None if symmetric else zp_int.to(w_fp.dtype) * scale
  if block_size != -1:
    s = in_dim // block_size
    q = q.reshape(out_dim, s, block_size).permute(1, 2, 0).contiguous()
    scale = scale.reshape(out_dim, s).permute(1, 0).contiguous()
    if zero_point is not None:
      zero_point = zero_point.reshape(out_dim, s).permute(1, 0).contiguous()
  return q, scale, zero_point


def quantize_linear(linear, n_bits=8, block_size=-1, symmetric=True, quantize_activation=False):
  """An ``XlaQuantizedLinear`` holding the RTN-quantized weight of ``linear`` (bias-free, like the reference)."""
  assert isinstance(linear, torch.nn.Linear)
  assert linear.bias is None, "XlaQuantizedLinear has no bias"
  w_int, scaler, zero_point = quantize_rtn(linear.weight.data, n_bits, block_size, symmetric)
  q = XlaQuantizedLinear(linear.in_features, linear.out_features, is_symmetric=symmetric, block_size=block_size,
                         int4_weight=(n_bits == 4), quantize_activation=quantize_activation)
  q.load_quantized_weight(w_int, scaler, zero_point)
  return q


def swap_linears(model, predicate=None, **quant_args):
  """Replaces every bias-free ``nn.Linear`` of ``model`` (for which ``predicate(name, module)`` holds) in place."""
  for name, child in list(model.named_children()):
    if isinstance(child, torch.nn.Linear) and child.bias is None and (predicate is None or predicate(name, child)):
      setattr(model, name, quantize_linear(child, **quant_args))
    else:
      swap_linears(child, predicate, **quant_args)
  return model
