"""Fusions either side of the quantized linear: gate+up of a gated MLP with its activation, and
concatenated projections that share one activation (q/k/v).

The reference issues one ``quantized_matmul`` per projection and leaves ``silu(gate) * up`` and the
operand sharing to XLA's fusion passes.  Here the two projections become ONE weight stream:

  ``interleave_gate_up``   stacks the K-minor weights of gate and up in groups of 16 rows (eight gate rows,
                           then the eight up rows of the same outputs) so that one output tile of the decode
                           kernels holds both halves of eight outputs.
  ``quantized_gate_up``    ``torch.ops.xla_b200.quantized_gate_up``: silu(x @ Wgate^T) * (x @ Wup^T) in one
                           kernel for decode batches (M <= 32), computed in fp32 from the fp32 accumulators;
                           larger batches run the stacked weight as one linear and apply the activation after.
  ``concat_projections``   row-concatenates K-minor weights (and their scales) of projections that read the
                           same activations; one call then produces all outputs, split by ``split_outputs``.

Per projection the arithmetic is the reference's (torch_xla/experimental/xla_quantized_matmul.py:152-170).
"""
import torch

from . import _capi
from . import quantized_matmul as _qm
from .packed import quantized_matmul_packed

LIB = torch.library.Library("xla_b200", "FRAGMENT")
try:
  getattr(torch.ops.xla_b200, "quantized_gate_up")
except (AttributeError, RuntimeError):
  LIB.define("quantized_gate_up(Tensor x, Tensor w, Tensor scale, int block_size=-1, bool int4_weight=False, "
             "bool weight_is_packed=False, ScalarType? out_dtype=None) -> Tensor")


def _interleave_rows(a, b, dim):
  """[.., N, ..] x2 -> [.., 2N, ..]: groups of eight rows of a, then the matching eight rows of b."""
  n = a.shape[dim]
  assert n % 8 == 0, f"out_features must be a multiple of 8 to interleave gate and up, got {n}"
  shape = list(a.shape)
  grouped = shape[:dim] + [n // 8, 8] + shape[dim + 1:]
  both = torch.stack((a.reshape(grouped), b.reshape(grouped)), dim=dim + 1)  # [.., N/8, 2, 8, ..]
  return both.reshape(shape[:dim] + [2 * n] + shape[dim + 1:]).contiguous()


def interleave_gate_up(w_gate, w_up, scale_gate, scale_up, block_size=-1):
  """K-minor weights [N,K] (int8) or [N,K/2] (packed) of gate and up -> the [2N, ..] weight and its scales in
  the row order ``quantized_gate_up`` expects.  Scales are [N] (per channel) or [K/bs, N] (blockwise)."""
  assert w_gate.shape == w_up.shape and w_gate.dtype == w_up.dtype
  assert scale_gate.shape == scale_up.shape
  w = _interleave_rows(w_gate, w_up, 0)
  s = _interleave_rows(scale_gate, scale_up, 0 if block_size == -1 else 1)
  return w, s


def _deinterleave(y):
  """[M, 2N] in interleaved column order -> (gate [M,N], up [M,N])."""
  m, n2 = y.shape
  g = y.reshape(m, n2 // 16, 2, 8)
  return g[:, :, 0, :].reshape(m, n2 // 2), g[:, :, 1, :].reshape(m, n2 // 2)


def quantized_gate_up(x, w, scaler, block_size=-1, int4_weight=False, weight_is_packed=False, out_dtype=None):
  _capi.require_cuda(x, w, scaler)
  K = x.shape[-1]
  assert w.dim() == 2 and w.shape[0] % 16 == 0, (
      f"interleaved gate/up weight is expected to be [2 * out_features, ...] with out_features % 8 == 0, got {list(w.shape)}")
  assert w.shape[1] * (2 if weight_is_packed else 1) == K, (
      f"Weight shape is expected to be [2 * output_dim, input_dim], input_dim: {K}, but got {list(w.shape)}.")
  if out_dtype is None:
    out_dtype = _qm._out_dtype(x, scaler, None)
  x2 = _qm._rows(x)
  M, N2 = x2.shape[0], w.shape[0]
  s32 = _qm._f32(scaler)
  wbits = 4 if weight_is_packed else 8
  fused = (1 <= M <= 32 and x2.dtype in (torch.bfloat16, torch.float16) and K % (512 // wbits) == 0 and
           (block_size == -1 or block_size % (512 // wbits) == 0) and _qm.current_variant() in ("auto", "mma"))
  if fused:
    expect = (N2,) if block_size == -1 else (K // block_size, N2)
    assert tuple(s32.shape) == expect, f"weight scaler shape is expect to be {list(expect)}, got {list(s32.shape)}."
    wc = w if w.is_contiguous() else w.contiguous()

    def run():
      out = torch.empty((M, N2 // 2), dtype=out_dtype, device=x.device)
      _capi.check(_capi.lib().qmm_gate_up_decode(wbits, x2.data_ptr(), _capi.dtype_code(x2.dtype), wc.data_ptr(),
                                                 s32.data_ptr(), out.data_ptr(), _capi.dtype_code(out_dtype), M, N2, K,
                                                 0 if block_size == -1 else block_size, _capi.stream_ptr(x.device)))
      return out

    out = _capi.on_device(x.device, run)
  else:
    out = None
    if (32 < M <= 1008 and x2.dtype in (torch.bfloat16, torch.float16, torch.float32) and K >= 128 and K % (128 // wbits) == 0 and
        (block_size == -1 or block_size == 128 or block_size % 256 == 0) and _qm.current_variant() in ("auto", "i8tc")):
      # larger batches: the split-activation tensor-core kernel applies silu(gate) * up in its drain
      expect = (N2,) if block_size == -1 else (K // block_size, N2)
      assert tuple(s32.shape) == expect, f"weight scaler shape is expect to be {list(expect)}, got {list(s32.shape)}."
      wc = w if w.is_contiguous() else w.contiguous()

      def run():
        ws, ws_bytes = _capi.workspace(x.device, M, K)
        if ws is None:  # a stream capture that began before the scratch existed
          return None
        res = torch.empty((M, N2 // 2), dtype=out_dtype, device=x.device)
        _capi.check(_capi.lib().qmm_gate_up(wbits, x2.data_ptr(), _capi.dtype_code(x2.dtype), wc.data_ptr(), s32.data_ptr(),
                                            res.data_ptr(), _capi.dtype_code(out_dtype), M, N2, K,
                                            0 if block_size == -1 else block_size, ws, ws_bytes, _capi.stream_ptr(x.device)))
        return res

      out = _capi.on_device(x.device, run)
  if out is None:
    y = quantized_matmul_packed(x2, w, s32, None, block_size=block_size, int4_weight=int4_weight,
                                weight_is_packed=weight_is_packed, out_dtype=torch.float32)
    g, u = _deinterleave(y)
    out = (torch.nn.functional.silu(g) * u).to(out_dtype)
  return out if x.dim() == 2 else out.reshape(x.shape[:-1] + (N2 // 2,))


def _meta(x, w, scaler, block_size=-1, int4_weight=False, weight_is_packed=False, out_dtype=None):
  if out_dtype is None:
    out_dtype = _qm._out_dtype(x, scaler, None)
  return torch.empty(x.shape[:-1] + (w.shape[0] // 2,), dtype=out_dtype, device=x.device)


LIB.impl("quantized_gate_up", quantized_gate_up, "CUDA")
LIB.impl("quantized_gate_up", _meta, "Meta")


def concat_projections(weights, scales, block_size=-1):
  """Row-concatenates K-minor weights ([N_i, K] or packed [N_i, K/2]) and their scales; returns (w, scale, sizes)."""
  w = torch.cat(list(weights), dim=0).contiguous()
  s = torch.cat(list(scales), dim=0 if block_size == -1 else 1).contiguous()
  return w, s, [int(t.shape[0]) for t in weights]


def split_outputs(y, sizes):
  """Splits the output of a concatenated projection back into its parts (views, no copy)."""
  return torch.split(y, sizes, dim=-1)
