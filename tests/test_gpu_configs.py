"""GPU parity at the benchmark configurations' own shapes, through the operators with the kernel choice left to AUTO,
against the CPU oracle (on a sample of token rows where the full product would take the oracle minutes).

Tolerances as everywhere: 1e-4 (max|a-b| / max|b|) for fp32 outputs against the exact value of the formula, 1e-2 for
16-bit outputs.  The shapes follow the reference's own test grid where one exists
(test/test_quantized_matmul_pallas_kernel.py:86-126 for the int8 operator without activation quantization).
"""
import pytest
import torch

import xla_b200
from oracle import qmm_oracle as qo
from tests import qmm_cases as qc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL_BF16 = 1e-2
TOL_F32 = 1e-4


def _rows_sample(M):
  return torch.tensor(sorted({0, M // 3, M // 2, M - 1}))


def test_config2_full_shape_all_batches():
  """W4A16 blockwise decode, w [14336, 4096] int4 packed, block 128, M in {1, 8, 32} (and 16, 64)."""
  g = qc.gen(0)
  N, K, bs = 14336, 4096, 128
  x = qc.activations(g, 64, K)
  w = qc.int4_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N)
  wp = xla_b200.pack_int4(w.to(DEV))
  exact = qo.quantized_matmul(x.float(), qc.to_sbn(w, bs), s, block_size=bs, dot_round=None)
  for M in (1, 8, 16, 32, 64):
    out = torch.ops.xla_b200.quantized_matmul_packed(x[:M].to(DEV), wp, s.to(DEV), block_size=bs, int4_weight=True,
                                                     weight_is_packed=True, out_dtype=torch.float32)
    assert qo.max_abs_rel(out, exact[:M]) < TOL_F32, M
    out16 = torch.ops.xla_b200.quantized_matmul_packed(x[:M].to(DEV), wp, s.to(DEV), block_size=bs, int4_weight=True,
                                                       weight_is_packed=True, out_dtype=torch.bfloat16)
    assert qo.max_abs_rel(out16, exact[:M]) < TOL_BF16, M


@pytest.mark.parametrize("M", [16, 32])
def test_config2_through_the_reference_layout_op(M):
  """torch.ops.xla.quantized_matmul(x, w[S,bs,N], scale[S,N], block_size=128): the reference's own call."""
  g = qc.gen(1)
  N, K, bs = 14336, 4096, 128
  x = qc.activations(g, M, K)
  w_sbn = qc.to_sbn(qc.int4_weight(g, N, K), bs)
  s = qc.blockwise_scale(g, K // bs, N)
  exact = qo.quantized_matmul(x.float(), w_sbn, s, block_size=bs, dot_round=None)
  wd, sd = w_sbn.to(DEV), s.to(DEV)
  for int4 in (True, False):   # packed int4 copy / transposed int8 copy behind the operator
    out = torch.ops.xla.quantized_matmul(x.to(DEV), wd, sd, block_size=bs, int4_weight=int4)
    assert out.dtype == torch.float32
    assert qo.max_abs_rel(out, exact) < TOL_F32, int4
  # a weight written in place is converted again
  wd.zero_()
  out = torch.ops.xla.quantized_matmul(x.to(DEV), wd, sd, block_size=bs, int4_weight=True)
  assert torch.all(out == 0)


LLAMA8B = [("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096), ("gate", 4096, 14336),
           ("up", 4096, 14336), ("down", 14336, 4096)]


@pytest.mark.parametrize("name,K,N", LLAMA8B)
def test_config4_every_linear(name, K, N):
  """int8 per-channel weight-only, M in {1, 16, 64, 512}, all seven linears of the layer."""
  g = qc.gen(K + N + len(name))
  w = qc.int8_weight(g, N, K)
  s = qc.per_channel_scale(g, N)
  x = qc.activations(g, 512, K)
  wd, sd = w.to(DEV), s.to(DEV)
  for M in (1, 16, 64, 512):
    rows = _rows_sample(M)
    out = torch.ops.xla.quantized_matmul(x[:M].to(DEV), wd, sd)
    assert out.dtype == torch.float32 and tuple(out.shape) == (M, N)
    exact = qo.quantized_matmul(x[rows].float(), w, s, dot_round=None)
    assert qo.max_abs_rel(out[rows.to(DEV)], exact) < TOL_F32, (name, M)


@pytest.mark.parametrize("name,K,N", [("gate", 8192, 28672), ("down", 28672, 8192)])
def test_config5_shapes_single_gpu(name, K, N):
  """W4A16 blockwise (block 128) at the 70B-shaped MLP's sizes, M in {1, 64, 512}, unsharded."""
  g = qc.gen(5 + len(name))
  bs = 128
  w = qc.int4_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N)
  x = qc.activations(g, 512, K)
  wp = xla_b200.pack_int4(w.to(DEV))
  sd = s.to(DEV)
  w_sbn = qc.to_sbn(w, bs)
  for M in (1, 64, 512):
    rows = _rows_sample(M)
    out = torch.ops.xla_b200.quantized_matmul_packed(x[:M].to(DEV), wp, sd, block_size=bs, int4_weight=True,
                                                     weight_is_packed=True, out_dtype=torch.float32)
    exact = qo.quantized_matmul(x[rows].float(), w_sbn, s, block_size=bs, dot_round=None)
    assert qo.max_abs_rel(out[rows.to(DEV)], exact) < TOL_F32, (name, M)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, TOL_BF16), (torch.float32, TOL_F32)])
@pytest.mark.parametrize("bs,n_in,n_out", [(128, 128, 128), (256, 256, 256), (512, 512, 512), (64, 64, 64), (192, 192, 192),
                                           (128, 512, 256), (512, 128, 192)])
def test_quantized_matmul_int8_without_activation_quantization(dtype, tol, bs, n_in, n_out):
  """The int8 operator's weight-only branch on the reference's grid of cube and ragged shapes."""
  g = qc.gen(bs + n_in + n_out)
  x = qc.activations(g, bs, n_in, dtype=dtype)
  w = qc.int8_weight(g, n_out, n_in)
  s = qc.per_channel_scale(g, n_out)
  out = torch.ops.xla.quantized_matmul_int8(x.to(DEV), w.to(DEV), s.to(DEV), quantize_activation=False)
  assert out.dtype == dtype and tuple(out.shape) == (bs, n_out)
  exact = qo.quantized_matmul(x.float(), w, s, dot_round=None)
  assert qo.max_abs_rel(out, exact) < tol
