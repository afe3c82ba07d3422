"""Sibling operator for kernel-native weight layouts: ``torch.ops.xla_b200.quantized_matmul_packed``.

The reference operator stores int4 weights unpacked (one value per int8) and blockwise weights
N-minor ([in/block, block, out]); it has no ``weight_is_packed`` argument, so adding one to the
``xla::`` schema would break signature identity.  This op carries the same argument list plus
``weight_is_packed`` and takes K-minor weights, the layout the decode and tensor-core kernels
stream at full HBM speed:

  per-channel : w int8 [N, K]           (or uint8 [N, K/2] when weight_is_packed)
  blockwise   : w int8 [N, K]           (or uint8 [N, K/2] when weight_is_packed), scaler [K/bs, N]

Packed byte j of a row holds k = 2j in its low nibble and k = 2j+1 in its high nibble (two's
complement).  ``pack_int4`` / ``unpack_int4`` convert from the reference layouts on the device.
"""
import torch

from . import _capi
from . import quantized_matmul as _qm

LIB = torch.library.Library("xla_b200", "FRAGMENT")
try:
  getattr(torch.ops.xla_b200, "quantized_matmul_packed")
except (AttributeError, RuntimeError):
  LIB.define("quantized_matmul_packed(Tensor x, Tensor w, Tensor scale, Tensor? zero_point=None, "
             "int block_size=-1, bool int4_weight=False, bool weight_is_packed=False, "
             "bool quantize_activation=False, ScalarType? out_dtype=None) -> Tensor")


def pack_int4(w, layout="nk"):
  """int8 container of int4 values -> uint8 [N, K/2].  layout "nk": w is [N,K]; "sbn": [S,bs,N]."""
  _capi.require_cuda(w)
  assert w.dtype == torch.int8, f"Weight dtype is expected to be torch.int8, got {w.dtype}."
  w = w.contiguous()
  L = _capi.lib()
  with torch.cuda.device(w.device):
    if layout == "nk":
      n, k = w.shape
      assert k % 2 == 0, "packing int4 needs an even in_features"
      out = torch.empty((n, k // 2), dtype=torch.uint8, device=w.device)
      _capi.check(L.qmm_pack_int4_nk(_capi.ptr(w), _capi.ptr(out), n, k, _capi.stream_ptr(w.device)))
    elif layout == "sbn":
      s, bs, n = w.shape
      assert (s * bs) % 2 == 0, "packing int4 needs an even in_features"
      out = torch.empty((n, s * bs // 2), dtype=torch.uint8, device=w.device)
      _capi.check(L.qmm_pack_int4_sbn(_capi.ptr(w), _capi.ptr(out), s, bs, n, _capi.stream_ptr(w.device)))
    else:
      raise ValueError(f"unknown layout {layout!r}")
  return out


def unpack_int4(wp):
  """uint8 [N, K/2] -> int8 [N, K]."""
  _capi.require_cuda(wp)
  assert wp.dtype == torch.uint8 and wp.dim() == 2
  wp = wp.contiguous()
  n, kh = wp.shape
  out = torch.empty((n, kh * 2), dtype=torch.int8, device=wp.device)
  with torch.cuda.device(wp.device):
    _capi.check(_capi.lib().qmm_unpack_int4_nk(_capi.ptr(wp), _capi.ptr(out), n, kh * 2,
                                               _capi.stream_ptr(wp.device)))
  return out


def _shapes(x, w, scaler, zero_point, block_size, weight_is_packed):
  K = x.shape[-1]
  assert w.dim() == 2, f"Weight tensor is expected to be 2D, got {w.dim()}D Tensor."
  if weight_is_packed:
    assert w.dtype == torch.uint8, f"Packed weight dtype is expected to be torch.uint8, got {w.dtype}."
    assert K % 2 == 0 and w.shape[1] * 2 == K, (
        f"Packed weight shape is expected to be [output_dim, input_dim / 2], input_dim: {K}, got {list(w.shape)}.")
  else:
    assert w.dtype == torch.int8, f"Weight dtype is expected to be torch.int8, got {w.dtype}."
    assert w.shape[1] == K, (
        f"Weight shape is expected to be [output_dim, input_dim], input_dim: {K}, but got {list(w.shape)}.")
  N = w.shape[0]
  if block_size == -1:
    assert scaler.dim() == 1 and scaler.shape[0] == N, (
        f"weight scaler shape is expect to be [out_channel,], got {scaler.shape}, weight shape {list(w.shape)}.")
    if zero_point is not None:
      assert zero_point.dim() == 1 and zero_point.shape[0] == N, (
          f"zero point shape is expect to be [out_channel,], got {zero_point.shape}, weight shape {list(w.shape)}.")
  else:
    assert block_size > 0 and K % block_size == 0, (
        f"input_dim should be divisible by block_size, got input_dim: {K}, block_size: {block_size}.")
    S = K // block_size
    assert scaler.dim() == 2 and tuple(scaler.shape) == (S, N), (
        f"weight scaler shape is expect to be [in_channel / block_size, out_channel], got {scaler.shape}.")
    if zero_point is not None:
      assert zero_point.dim() == 2 and tuple(zero_point.shape) == (S, N), (
          f"zero_point shape is expect to be [in_channel / block_size, out_channel], got {zero_point.shape}.")
  return N, K


def quantized_matmul_packed(x, w, scaler, zero_point=None, block_size=-1, int4_weight=False,
                            weight_is_packed=False, quantize_activation=False, out_dtype=None, out=None):
  """CUDA kernel of ``torch.ops.xla_b200.quantized_matmul_packed``.  ``out`` (Python callers only, not part of
  the operator schema) is a preallocated contiguous [M, N] result buffer, e.g. a peer-mapped one."""
  _capi.require_cuda(x, w, scaler, zero_point)
  N, K = _shapes(x, w, scaler, zero_point, block_size, weight_is_packed)
  if block_size != -1:
    assert quantize_activation == False, (  # noqa: E712
        "Blockwise quantization does not support activation quantization.")
  if out_dtype is None:
    out_dtype = _qm._out_dtype(x, scaler, zero_point)
  x2 = _qm._rows(x)
  M = x2.shape[0]
  w = w if w.is_contiguous() else w.contiguous()
  s32, zp32 = _qm._f32(scaler), _qm._f32(zero_point)
  L = _capi.lib()
  variant = _capi.VARIANTS[_qm.current_variant()]
  zp_after = not quantize_activation and _qm._zero_point_outside(M, x2, zero_point)
  out_buf = None if quantize_activation else out

  def run():
    if quantize_activation:
      if weight_is_packed:
        raise NotImplementedError("W4A8 (packed int4 weights with activation quantization) is not supported")
      return _qm._w8a8(x2, w, s32, zp32, out_dtype)
    kdt = torch.float32 if zp_after else out_dtype
    if out_buf is not None and not zp_after:
      assert out_buf.shape == (M, N) and out_buf.dtype == kdt and out_buf.is_contiguous() and out_buf.device == x.device
      out = out_buf
    else:
      out = torch.empty((M, N), dtype=kdt, device=x.device)
    st = _capi.stream_ptr(x.device)
    ws, ws_bytes = _capi.workspace(x.device, M, K, N, 4 if weight_is_packed else 8)
    _capi.check(L.qmm_weight_only(4 if weight_is_packed else 8, x2.data_ptr(), _capi.dtype_code(x2.dtype), w.data_ptr(),
                                  s32.data_ptr(), None if zp_after else _capi.ptr(zp32), out.data_ptr(), _capi.dtype_code(kdt),
                                  M, N, K, 0 if block_size == -1 else block_size, variant, ws, ws_bytes, st))
    if zp_after:
      out = _qm._subtract_zero_point(out, x2, zp32, block_size).to(out_dtype)
      if out_buf is not None:
        out = out_buf.copy_(out)
    return out

  out = _capi.on_device(x.device, run)
  return out if x.dim() == 2 else out.reshape(x.shape[:-1] + (N,))


def _meta(x, w, scaler, zero_point=None, block_size=-1, int4_weight=False, weight_is_packed=False,
          quantize_activation=False, out_dtype=None):
  if out_dtype is None:
    out_dtype = _qm._out_dtype(x, scaler, zero_point)
  return torch.empty(x.shape[:-1] + (w.shape[0],), dtype=out_dtype, device=x.device)


LIB.impl("quantized_matmul_packed", quantized_matmul_packed, "CUDA")
LIB.impl("quantized_matmul_packed", _meta, "Meta")
