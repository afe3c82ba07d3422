"""``torch.ops.xla.quantized_matmul`` and ``XlaQuantizedLinear`` on B200.

Host-side mirror of torch_xla/experimental/xla_quantized_matmul.py: the same operator schema
(:7-9), the same shape checks and messages (:12-53), the same module constructor, buffer names and
``load_quantized_weight`` (:186-243).  The arithmetic runs in the sm_100a kernels behind the C ABI
(include/qmm_b200.h); the kernel is registered for the CUDA dispatch key, plus a Meta kernel for
tracing.  There is no CPU kernel here: CPU tensors fail in the dispatcher.

Importing this module registers the ops, like importing the reference module does.
"""
import torch

from . import _capi

SCHEMA = ("quantized_matmul(Tensor x, Tensor w, Tensor scale, Tensor? zero_point=None, "
          "int? block_size=-1, bool? int4_weight=False, bool? quantize_activation=False) -> Tensor")


def has_xla_op(name):
  try:
    getattr(torch.ops.xla, name)
    return True
  except (AttributeError, RuntimeError):
    return False


# A FRAGMENT attaches to the ``xla`` namespace whether or not torch_xla created it first; the schema
# is defined here only when nobody else has (torch_xla's own definition is byte-identical).
XLA_LIB = torch.library.Library("xla", "FRAGMENT")
if not has_xla_op("quantized_matmul"):
  XLA_LIB.define(SCHEMA)

# Per-thread settings: the kernel family forced inside a `force_variant` block ("auto" otherwise) and how the
# activation quantizer converts a pre-cast +128 - saturate to 127 (what an XLA device does, the default) or wrap to
# -128 (what the reference's eager CPU kernel does).  Thread-local, so that concurrent callers do not see each other's.
import threading

_tls = threading.local()


def current_variant():
  return getattr(_tls, "variant", "auto")


def current_saturation():
  return getattr(_tls, "saturate", True)


class force_variant:
  """Context manager: run this thread's ops with one kernel family ("generic", "gemv", "tcgen05", "mma", "i8tc", "auto")."""

  def __init__(self, name):
    assert name in _capi.VARIANTS, name
    self.name = name

  def __enter__(self):
    self.prev = current_variant()
    _tls.variant = self.name

  def __exit__(self, *exc):
    _tls.variant = self.prev


def set_activation_saturation(saturate: bool):
  """True (default): int8 conversion clamps; False: wraps +128 to -128 like eager CPU.  Applies to the calling thread."""
  _tls.saturate = bool(saturate)


# ---- shape checks ---------------------------------------------------------------------------------
# Conditions and AssertionError texts match the reference's validators (:12-53) so that code and
# tests written against them see the same failures.


def _expect(ok, message):
  if not ok:
    raise AssertionError(message)


def _check_int8_rank(w, rank):
  _expect(w.dtype == torch.int8, f"Weight dtype is expected to be torch.int8, got {w.dtype}.")
  _expect(w.dim() == rank, f"Weight tensor is expected to be {rank}D, got {w.dim()}D Tensor.")


def _check_per_channel_quant_weight_dtype_shapes(input_dim, output_dim, w, w_scaler, zero_point):
  _check_int8_rank(w, 2)
  dims = list(w.shape)
  _expect(
      dims == [output_dim, input_dim],
      f"Weight shape is expected to be [output_dim, input_dim], output_dim: {output_dim}, "
      f"input_dim: {input_dim}, but got {dims}.")
  _expect(
      w_scaler.dim() == 1 and w_scaler.shape[0] == dims[0],
      f"weight scaler shape is expect to be [out_channel,], got {w_scaler.shape}, weight shape {dims}.")
  if zero_point is not None:
    # (the reference tests the scaler's length here a second time; the kernels index zero_point[n] for every n,
    # so its own length is what has to match)
    _expect(
        zero_point.dim() == 1 and zero_point.shape[0] == dims[0],
        f"zero point shape is expect to be [out_channel,], got {zero_point.shape}, weight shape {dims}.")


def _check_blockwise_quant_weight_dtype_shapes(input_dim, output_dim, block_size, w, w_scaler,
                                               zero_point):
  _check_int8_rank(w, 3)
  dims = list(w.shape)
  _expect(
      input_dim % block_size == 0, f"input_dim should be divisible by block_size, "
      f"got input_dim: {input_dim}, block_size: {block_size}.")
  _expect(
      dims[0] == input_dim / block_size and dims[1] == block_size,
      f"Weight shape is expected to be [input_dim / block_size, block_size, output_dim], "
      f"input_dim: {input_dim}, block_size: {block_size}, output_dim: {output_dim}, "
      f"but got {dims}.")
  for name, t in (("weight scaler", w_scaler), ("zero_point", zero_point)):
    if t is None:
      continue
    _expect(t.dim() == 2, f"{name} is expected to be 2D, got {t.dim()}D Tensor.")
    _expect(
        t.shape[0] == dims[0] and t.shape[1] == dims[-1],
        f"{name} shape is expect to be [in_channel / block_size, out_channel], "
        f"got {t.shape}, weight shape {dims}.")


# ---- helpers ------------------------------------------------------------------------------------


def _out_dtype(x, scaler, zero_point):
  """The reference's output dtype is whatever type promotion of its eager ops gives (:158-182)."""
  dt = torch.promote_types(x.dtype, scaler.dtype)
  if zero_point is not None:
    dt = torch.promote_types(dt, zero_point.dtype)
  return dt


def _f32(t):
  if t is None:
    return None
  return t.contiguous() if t.dtype == torch.float32 else t.float().contiguous()


def _zero_point_outside(M, x2, zero_point):
  """True when the zero-point term is applied after the kernel: the tensor-core and register-dequant
  kernels take symmetric weights only, and the any-shape kernel that does take a zero point is far slower
  than one of them plus a rank-S update (S = number of scale blocks)."""
  return (zero_point is not None and M > 8 and current_variant() == "auto" and
          x2.dtype in (torch.bfloat16, torch.float16))


def _subtract_zero_point(y32, x2, zp32, block_size):
  """y32[m,n] -= sum_b (sum_{k in block b} x[m,k]) * zp[b,n], in fp32 (the reference's second term, :159, :170)."""
  M, K = x2.shape
  S = 1 if block_size == -1 else K // block_size
  xs = x2.float().reshape(M, S, K // S).sum(-1)
  return y32.addmm_(xs, zp32.reshape(S, -1), alpha=-1.0)


def _rows(x):
  """x as a contiguous [M, K] matrix."""
  if x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
    raise TypeError(f"quantized_matmul: activation dtype {x.dtype} is not supported")
  if x.dim() == 2 and x.is_contiguous():
    return x  # the common case: no view to build
  k = x.shape[-1]
  x2 = x.reshape(-1, k)
  return x2 if x2.is_contiguous() else x2.contiguous()


def quantize_tensor(x, saturate=None):
  """``_quantize_tensor`` of the reference (:56-73) as one kernel; returns (int8, scale in x.dtype)."""
  _capi.require_cuda(x)
  x2 = _rows(x)
  M, K = x2.shape
  xq = torch.empty((M, K), dtype=torch.int8, device=x.device)
  xs = torch.empty((M,), dtype=torch.float32, device=x.device)
  sat = current_saturation() if saturate is None else saturate
  with torch.cuda.device(x.device):
    _capi.check(_capi.lib().qmm_quantize_activation(
        _capi.ptr(x2), _capi.dtype_code(x2.dtype), _capi.ptr(xq), _capi.ptr(xs), None, M, K, int(sat),
        _capi.stream_ptr(x.device)))
  return xq.reshape(x.shape), xs.to(x.dtype).reshape(x.shape[:-1] + (1,))


def _w8a8(x2, w, scaler, zero_point, out_dtype):
  L = _capi.lib()
  M, K = x2.shape
  N = w.shape[0]
  out = torch.empty((M, N), dtype=out_dtype, device=x2.device)
  if M * N == 0:
    return out
  nbytes = L.qmm_workspace_size(_capi.OP_W8A8_PERCHANNEL, M, N, K)
  ws = torch.empty((nbytes,), dtype=torch.uint8, device=x2.device)
  _capi.check(L.qmm_w8a8_perchannel(
      _capi.ptr(x2), _capi.dtype_code(x2.dtype), _capi.ptr(w), _capi.ptr(scaler), _capi.ptr(zero_point),
      _capi.ptr(out), _capi.dtype_code(out_dtype), M, N, K, int(current_saturation()), _capi.VARIANTS[current_variant()],
      _capi.ptr(ws), nbytes, _capi.stream_ptr(x2.device)))
  return out


# K-minor copies of blockwise weights that arrive in the reference layout [in/block, block, out] (N minor), keyed by
# the weight tensor object: id -> (weak reference, version counter, storage address, converted weight, is_packed).
# An entry dies with its tensor (weak-reference callback) and is rebuilt when the tensor was written in place.
_kminor_cache = {}
_kminor_enabled = True


def set_activation_limbs(limbs: int):
  """Precision of the split-activation kernel above 32 tokens (process-wide).  0, the default: bf16 / f16 outputs take
  two int8 limbs per activation (error at most 2^-15 of the row's largest |x| each), fp32 outputs three; 3: three
  limbs everywhere, the accuracy of an fp32 accumulation, at a third more tensor-core columns per token."""
  _capi.check(_capi.lib().qmm_set_activation_limbs(int(limbs)))


def set_prepack_cache(enabled: bool):
  """Turns the operator's K-minor weight cache on or off (off: every blockwise call on the reference layout runs
  the any-shape kernel) and drops what it holds."""
  global _kminor_enabled
  _kminor_enabled = bool(enabled)
  _kminor_cache.clear()


def _kminor_weight(w, int4_weight):
  """[S, bs, N] int8 -> (packed int4 [N, K/2], True) or (int8 [N, K], False), converted once per weight tensor."""
  import weakref
  key = id(w)
  hit = _kminor_cache.get(key)
  if hit is not None and hit[0]() is w and hit[1] == w._version and hit[2] == w.data_ptr():
    return hit[3], hit[4]
  K = w.shape[0] * w.shape[1]
  if int4_weight and K % 2 == 0:
    from . import packed
    conv, is_packed = packed.pack_int4(w, layout="sbn"), True
  else:
    conv, is_packed = w.reshape(K, -1).t().contiguous(), False
  try:
    ref = weakref.ref(w, lambda _r, k=key: _kminor_cache.pop(k, None))
  except TypeError:
    return conv, is_packed  # not weak-referenceable: convert every time rather than risk a stale entry
  _kminor_cache[key] = (ref, w._version, w.data_ptr(), conv, is_packed)
  return conv, is_packed


def quantized_matmul_cuda(x, w, scaler, zero_point=None, block_size=-1, int4_weight=False,
                          quantize_activation=False):
  """CUDA-key kernel of ``xla::quantized_matmul``; argument meaning as in the reference (:76-99)."""
  block_size = -1 if block_size is None else block_size
  quantize_activation = bool(quantize_activation)
  _capi.require_cuda(x, w, scaler, zero_point)
  K = x.shape[-1]
  if block_size == -1:
    _check_per_channel_quant_weight_dtype_shapes(K, scaler.shape[0], w, scaler, zero_point)
    N = w.shape[0]
  else:
    assert quantize_activation == False, (  # noqa: E712 (kept as in the reference)
        "Blockwise quantization does not support activation quantization.")
    _check_blockwise_quant_weight_dtype_shapes(K, w.shape[-1], block_size, w, scaler, zero_point)
    N = w.shape[-1]
  out_dtype = _out_dtype(x, scaler, zero_point)
  if (block_size != -1 and _kminor_enabled and current_variant() == "auto" and w.is_contiguous() and
      (id(w) in _kminor_cache or not torch.cuda.is_current_stream_capturing())):
    # The streaming kernels read K-minor rows; the reference layout is N minor.  The weight is converted once (a
    # device-side transpose / int4 pack, cached per weight tensor) and the call continues on the packed operator.
    from . import packed
    wk, is_packed = _kminor_weight(w, bool(int4_weight))
    return packed.quantized_matmul_packed(x, wk, scaler, zero_point, block_size=block_size, int4_weight=bool(int4_weight),
                                          weight_is_packed=is_packed, out_dtype=out_dtype)
  x2 = _rows(x)
  M = x2.shape[0]
  w = w if w.is_contiguous() else w.contiguous()
  scaler32, zp32 = _f32(scaler), _f32(zero_point)
  L = _capi.lib()
  # per-channel weights reach the fast kernels directly; their zero point is applied afterwards
  zp_after = block_size == -1 and not quantize_activation and _zero_point_outside(M, x2, zero_point)

  def run():
    if quantize_activation:
      return _w8a8(x2, w, scaler32, zp32, out_dtype)
    kdt = torch.float32 if zp_after else out_dtype
    out = torch.empty((M, N), dtype=kdt, device=x.device)
    args = (x2.data_ptr(), _capi.dtype_code(x2.dtype), w.data_ptr(), scaler32.data_ptr(),
            None if zp_after else _capi.ptr(zp32), out.data_ptr(), _capi.dtype_code(kdt), M, N, K)
    if block_size == -1:
      ws, ws_bytes = _capi.workspace(x.device, M, K)
      _capi.check(L.qmm_weight_only(8, *args, 0, _capi.VARIANTS[current_variant()], ws, ws_bytes, _capi.stream_ptr(x.device)))
    else:
      _capi.check(L.qmm_blockwise_sbn(*args, block_size, _capi.VARIANTS[current_variant()], _capi.stream_ptr(x.device)))
    if zp_after:
      out = _subtract_zero_point(out, x2, zp32, -1).to(out_dtype)
    return out

  out = _capi.on_device(x.device, run)
  return out if x.dim() == 2 else out.reshape(x.shape[:-1] + (N,))


def quantized_matmul_meta(x, w, scaler, zero_point=None, block_size=-1, int4_weight=False,
                          quantize_activation=False):
  """Shape/dtype-only kernel for fake tensors (torch.compile tracing)."""
  block_size = -1 if block_size is None else block_size
  n = w.shape[0] if block_size == -1 else w.shape[-1]
  return torch.empty(x.shape[:-1] + (n,), dtype=_out_dtype(x, scaler, zero_point), device=x.device)


XLA_LIB.impl("quantized_matmul", quantized_matmul_cuda, "CUDA")
XLA_LIB.impl("quantized_matmul", quantized_matmul_meta, "Meta")


class XlaQuantizedLinear(torch.nn.Module):
  """Drop-in for the reference module (:186-243): same constructor, buffers and methods.

  Buffers (and ``state_dict`` keys): ``weight`` int8, ``weight_scaler``, ``zero_point`` (only when
  not symmetric).  Blockwise weights use the reference layout [in/block, block, out].

  ``prepack=True`` additionally keeps a kernel-native, K-minor copy of the weight where that helps (int4
  packed two per byte along K, for blockwise and per-channel int4 weights; blockwise int8 transposed to
  [out, in]; built on first use on the GPU); the copy is derived state and is not saved.
  """

  def __init__(self, input_dim, output_dim, is_symmetric: bool = False, block_size: int = -1,
               int4_weight: bool = False, quantize_activation: bool = False, prepack: bool = True):
    super().__init__()
    self.input_dim = input_dim
    self.output_dim = output_dim
    self.is_symmetric = is_symmetric
    self.block_size = block_size
    self.int4_weight = int4_weight
    self.quantize_activation = quantize_activation
    self.prepack = prepack
    self._packed = None
    self.register_buffer('weight', torch.zeros(output_dim, input_dim).to(torch.int8))
    self.register_buffer('weight_scaler', torch.zeros(output_dim))
    if not self.is_symmetric:
      self.register_buffer('zero_point', torch.zeros(output_dim))
    else:
      self.zero_point = None

  def load_quantized_weight(self, weight, weight_scaler, zero_point=None):
    '''
    weight (Tensor):
      per-channel quant: [out_channel, in_channel].
      block_wise quant: [in_channel / block_size, block_size, out_channel].

    weight_scaler (Tensor):
      per-channel quant: [out_channel,].
      blockwise quant: [in_channel / block_size, out_channel].
    '''
    if self.block_size == -1:
      _check_per_channel_quant_weight_dtype_shapes(self.input_dim, self.output_dim, weight,
                                                   weight_scaler, zero_point)
    else:
      _check_blockwise_quant_weight_dtype_shapes(self.input_dim, self.output_dim, self.block_size,
                                                 weight, weight_scaler, zero_point)
    self.weight = weight
    self.weight_scaler = weight_scaler
    self.zero_point = zero_point
    self._packed = None

  def _packed_weight(self):
    """Kernel-native (K-minor) copy of the weight: packed int4 [N,K/2] (blockwise or per-channel int4), or
    int8 [N,K] for a blockwise int8 weight."""
    w = self.weight
    key = (w.data_ptr(), w._version, w.device)
    if self._packed is None or self._packed[0] != key:
      from . import packed
      if self.int4_weight and self.input_dim % 2 == 0:
        self._packed = (key, packed.pack_int4(w, layout="sbn" if w.dim() == 3 else "nk"), True)
      else:
        self._packed = (key, w.reshape(self.input_dim, -1).t().contiguous(), False)  # [S,bs,N] -> [N,K]
    return self._packed[1], self._packed[2]

  def forward(self, x):
    blockwise = self.block_size != -1 and self.weight.dim() == 3
    per_channel_int4 = (self.block_size == -1 and self.int4_weight and self.weight.dim() == 2 and
                        self.input_dim % 2 == 0 and not self.quantize_activation)
    if self.prepack and self.weight.is_cuda and (blockwise or per_channel_int4):
      from . import packed
      w, is_packed = self._packed_weight()
      return packed.quantized_matmul_packed(
          x, w, self.weight_scaler, self.zero_point, block_size=self.block_size, int4_weight=self.int4_weight,
          weight_is_packed=is_packed, out_dtype=_out_dtype(x, self.weight_scaler, self.zero_point))
    return torch.ops.xla.quantized_matmul(
        x,
        self.weight,
        self.weight_scaler,
        self.zero_point,
        block_size=self.block_size,
        int4_weight=self.int4_weight,
        quantize_activation=self.quantize_activation)
