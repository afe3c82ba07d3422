"""A restatement of the reference's eager CPU kernel with the same ATen operators it runs on.

TEST / BASELINE INFRASTRUCTURE ONLY (never imported by the ``xla_b200`` package).

The reference's CPU path (torch_xla/experimental/xla_quantized_matmul.py:139-183, dispatch key
CompositeExplicitAutograd) is a short chain of PyTorch CPU operators: F.linear on up-cast weights,
two einsums for the blockwise case, broadcasting multiplies for the scales.  Its speed on a host is
therefore the speed of libtorch's CPU GEMM/einsum.  This file re-expresses that chain so that the
CPU baseline can be timed on a machine where the reference checkout is not present.  It is pinned
against the reference's golden outputs by tests/test_oracle_golden.py.
"""
import torch
import torch.nn.functional as F


def quantize_rows(x):
  """Per-row symmetric int8 quantization, scale kept in x.dtype (reference :56-73)."""
  peak = x.abs().amax(dim=-1, keepdim=True)
  step = peak / 127
  return torch.round(x / step).to(torch.int8), step.to(x.dtype)


def quantized_matmul_cpu(x, w, scaler, zero_point=None, block_size=-1, quantize_activation=False):
  x_scale = None
  if block_size == -1:
    wt = w.to(x.dtype)
    if quantize_activation:
      x, x_scale = quantize_rows(x)
      x, wt = x.to(torch.int32), wt.to(torch.int32)
    y = F.linear(x, wt) * scaler
    if zero_point is not None:
      y = y - torch.einsum("...c,z->...z", x, zero_point)
  else:
    if quantize_activation:
      raise AssertionError("Blockwise quantization does not support activation quantization.")
    xb = x.reshape(*x.shape[:-1], x.shape[-1] // block_size, block_size)
    per_block = torch.einsum("scn,...sc->...sn", w.to(x.dtype), xb)
    y = torch.einsum("sn,...sn->...n", scaler, per_block)
    if zero_point is not None:
      y = y - torch.matmul(xb.sum(dim=-1), zero_point)
  if x_scale is not None:
    y = y * x_scale
  return y
