"""ctypes front end of the CPU oracle (``qmm_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, by ``__graft_entry__.smoke`` and by the
CPU-baseline leg of ``bench.py``; never by the ``xla_b200`` package.

The functions mirror the reference's eager CPU kernel
(torch_xla/experimental/xla_quantized_matmul.py:56-73 and :139-183) and return CPU tensors.
Floating paths return float64 (the exact value of the reference's formula, optionally with the
reference's rounding of the dot product to the activation dtype re-applied); integer paths are
bit-exact restatements.
"""
import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libqmm_oracle.so")
_lib = None

ROUND_NONE, ROUND_BF16, ROUND_F16, ROUND_F32 = 0, 1, 2, 3
_ROUND_OF = {torch.bfloat16: ROUND_BF16, torch.float16: ROUND_F16, torch.float32: ROUND_F32}


def build(force=False):
  """Compiles qmm_oracle.c with the Makefile beside it (gcc only)."""
  src = os.path.join(_HERE, "qmm_oracle.c")
  if (not force and os.path.exists(_LIB_PATH) and
      os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
    return _LIB_PATH
  subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
  return _LIB_PATH


def lib():
  global _lib
  if _lib is None:
    if not os.path.exists(_LIB_PATH):
      build()
    L = ctypes.CDLL(_LIB_PATH)
    p, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    L.qo_set_threads.argtypes = [i32]
    L.qo_get_threads.restype = i32
    L.qo_quantize_act_bf16.argtypes = [p, i64, i64, p, p, i32]
    L.qo_quantize_act_f32.argtypes = [p, i64, i64, p, p, i32]
    L.qo_int8_gemm_i32.argtypes = [p, p, p, i64, i64, i64]
    L.qo_w8a8_epilogue_f32.argtypes = [p, p, p, p, p, p, i64, i64, i64]
    L.qo_perchannel.argtypes = [p, p, p, p, p, i64, i64, i64, i32]
    L.qo_blockwise.argtypes = [p, p, p, p, p, i64, i64, i64, i64, i32]
    L.qo_pack_int4_nk.argtypes = [p, p, i64, i64]
    L.qo_nk_to_sbn.argtypes = [p, p, i64, i64]
    _lib = L
  return _lib


def set_threads(n):
  lib().qo_set_threads(int(n))


def get_threads():
  return int(lib().qo_get_threads())


def _ptr(t):
  return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _c(t, dtype=None):
  t = t.detach().cpu()
  if dtype is not None:
    t = t.to(dtype)
  return t.contiguous()


def quantize_act(x, wrap=False):
  """``_quantize_tensor`` (xla_quantized_matmul.py:56-73) on the last dim.

  Returns (x_int8 [..., K], scale [..., 1] in x.dtype).  ``wrap=True`` reproduces the eager
  CPU conversion of a pre-cast value of +128 to -128; ``wrap=False`` saturates to 127.
  """
  assert x.dtype in (torch.bfloat16, torch.float32), x.dtype
  x = _c(x)
  K = x.shape[-1]
  M = x.numel() // K if K else 0
  xq = torch.empty(x.shape, dtype=torch.int8)
  scale = torch.empty(x.shape[:-1] + (1,), dtype=x.dtype)
  if x.numel():
    if x.dtype == torch.bfloat16:
      lib().qo_quantize_act_bf16(_ptr(x), M, K, _ptr(xq), _ptr(scale), int(wrap))
    else:
      lib().qo_quantize_act_f32(_ptr(x), M, K, _ptr(xq), _ptr(scale), int(wrap))
  return xq, scale


def int8_gemm_i32(xq, w):
  """acc[m,n] = sum_k xq[m,k]*w[n,k] in int32 (xla_quantized_matmul.py:153-158)."""
  xq, w = _c(xq, torch.int8), _c(w, torch.int8)
  K = xq.shape[-1]
  N = w.shape[0]
  M = xq.numel() // K if K else 0
  acc = torch.zeros(xq.shape[:-1] + (N,), dtype=torch.int32)
  if acc.numel() and K:
    lib().qo_int8_gemm_i32(_ptr(xq), _ptr(w), _ptr(acc), M, N, K)
  return acc


def w8a8_epilogue(acc, xq, w_scale, zero_point, x_scale):
  """fp32 dequant of the int32 accumulator in the reference's operation order (:159,:172-182)."""
  acc, xq = _c(acc, torch.int32), _c(xq, torch.int8)
  N = acc.shape[-1]
  K = xq.shape[-1]
  M = acc.numel() // N if N else 0
  ws = _c(w_scale, torch.float32)
  zp = _c(zero_point, torch.float32) if zero_point is not None else None
  xs = _c(x_scale, torch.float32).reshape(-1)
  out = torch.empty(acc.shape, dtype=torch.float32)
  if out.numel():
    lib().qo_w8a8_epilogue_f32(_ptr(acc), _ptr(xq), _ptr(ws), _ptr(zp), _ptr(xs), _ptr(out), M, N,
                               K)
  return out


def quantized_matmul(x,
                     w,
                     scaler,
                     zero_point=None,
                     block_size=-1,
                     int4_weight=False,
                     quantize_activation=False,
                     dot_round="x",
                     wrap=False):
  """The whole op (xla_quantized_matmul.py:139-183) on CPU tensors.

  ``dot_round``: "x" re-applies the reference's rounding of each dot product to x.dtype before
  the scale is applied; None returns the exact value of the formula.  Weight-only paths return
  float64; the W8A8 path returns the reference's own fp32 result (bit-exact restatement).
  ``int4_weight`` is accepted and ignored, like the reference's CPU kernel does.
  """
  del int4_weight
  lead = x.shape[:-1]
  K = x.shape[-1]
  if block_size == -1:
    N = w.shape[0]
    if quantize_activation:
      xq, xs = quantize_act(x.reshape(-1, K), wrap=wrap)
      acc = int8_gemm_i32(xq, w)
      out = w8a8_epilogue(acc, xq, scaler, zero_point, xs.float())
      return out.reshape(lead + (N,))
    mode = _ROUND_OF[x.dtype] if dot_round == "x" else ROUND_NONE
    xf = _c(x, torch.float32).reshape(-1, K)
    M = xf.shape[0]
    out = torch.zeros((M, N), dtype=torch.float64)
    ws = _c(scaler, torch.float32)
    zp = _c(zero_point, torch.float32) if zero_point is not None else None
    if out.numel():
      lib().qo_perchannel(_ptr(xf), _ptr(_c(w, torch.int8)), _ptr(ws), _ptr(zp), _ptr(out), M, N,
                          K, mode)
    return out.reshape(lead + (N,))
  assert not quantize_activation, "Blockwise quantization does not support activation quantization."
  N = w.shape[-1]
  mode = _ROUND_OF[x.dtype] if dot_round == "x" else ROUND_NONE
  xf = _c(x, torch.float32).reshape(-1, K)
  M = xf.shape[0]
  out = torch.zeros((M, N), dtype=torch.float64)
  ws = _c(scaler, torch.float32)
  zp = _c(zero_point, torch.float32) if zero_point is not None else None
  if out.numel():
    lib().qo_blockwise(_ptr(xf), _ptr(_c(w, torch.int8)), _ptr(ws), _ptr(zp), _ptr(out), M, N, K,
                       int(block_size), mode)
  return out.reshape(lead + (N,))


def pack_int4_nk(w_nk):
  """[N,K] int8 holding int4 values -> [N,K/2] uint8, low nibble = even k."""
  w_nk = _c(w_nk, torch.int8)
  N, K = w_nk.shape
  assert K % 2 == 0
  out = torch.empty((N, K // 2), dtype=torch.uint8)
  lib().qo_pack_int4_nk(_ptr(w_nk), _ptr(out), N, K)
  return out


def nk_to_sbn(w_nk, block_size):
  """[N,K] -> [K/bs, bs, N], the reference's blockwise layout (test_quantized_matmul.py:67-70)."""
  w_nk = _c(w_nk, torch.int8)
  N, K = w_nk.shape
  out = torch.empty((K // block_size, block_size, N), dtype=torch.int8)
  lib().qo_nk_to_sbn(_ptr(w_nk), _ptr(out), N, K)
  return out


def max_abs_rel(a, b):
  """max|a-b| / max|b|: the error measure the parity tests use for floating outputs."""
  a = a.detach().cpu().double()
  b = b.detach().cpu().double()
  denom = b.abs().max().item() if b.numel() else 1.0
  if denom == 0.0:
    denom = 1.0
  return (a - b).abs().max().item() / denom if a.numel() else 0.0
