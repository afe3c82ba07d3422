"""Pins the CPU oracle (oracle/qmm_oracle.c) against outputs of the unmodified reference.

The golden arrays were produced by tests/golden/make_golden.py from
torch_xla/experimental/xla_quantized_matmul.py (eager CPU kernel :139-183, quantizer :56-73).
Integer results must match bit for bit.
"""
import numpy as np
import pytest
import torch

from oracle import qmm_oracle as qo


def test_quantize_bf16_bit_exact_with_wrap(golden):
  x = golden.t("quant_bf16/x", bf16=True)
  xq_ref = golden.t("quant_bf16/xq")
  s_ref = golden.t("quant_bf16/scale", bf16=True)
  xq, s = qo.quantize_act(x, wrap=True)
  assert torch.equal(s.view(torch.int16), s_ref.view(torch.int16))
  assert torch.equal(xq, xq_ref)


def test_quantize_bf16_saturating_differs_only_at_plus128(golden):
  x = golden.t("quant_bf16/x", bf16=True)
  xq_ref = golden.t("quant_bf16/xq")
  xq, _ = qo.quantize_act(x, wrap=False)
  diff = xq != xq_ref
  assert int(diff.sum()) == int(golden.np("quant_bf16/n_plus128")) > 0
  assert bool((xq[diff] == 127).all()) and bool((xq_ref[diff] == -128).all())


def test_quantize_f32_bit_exact(golden):
  x = golden.t("quant_f32/x")
  xq, s = qo.quantize_act(x, wrap=True)
  assert torch.equal(xq, golden.t("quant_f32/xq"))
  assert torch.equal(s, golden.t("quant_f32/scale"))
  assert int(xq.abs().max()) == 127


@pytest.mark.parametrize("tag", ["bf16", "f32"])
def test_w8a8_accumulator_and_output_bit_exact(golden, tag):
  bf = tag == "bf16"
  k = f"w8a8_{tag}"
  x = golden.t(k + "/x", bf16=bf)
  w, s, zp = golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp")
  xq, xs = qo.quantize_act(x, wrap=True)
  assert torch.equal(xq, golden.t(k + "/xq"))
  acc = qo.int8_gemm_i32(xq, w)
  assert acc.dtype == torch.int32 and torch.equal(acc, golden.t(k + "/acc"))
  out = qo.quantized_matmul(x, w, s, quantize_activation=True, wrap=True)
  assert out.dtype == torch.float32
  assert torch.equal(out, golden.t(k + "/out"))
  out_zp = qo.quantized_matmul(x, w, s, zp, quantize_activation=True, wrap=True)
  ref_zp = golden.t(k + "/out_zp")
  assert qo.max_abs_rel(out_zp, ref_zp) < 2e-6


@pytest.mark.parametrize("tag,tol", [("bf16", 4e-3), ("f32", 2e-6), ("f32b", 2e-6)])
def test_per_channel_weight_only(golden, tag, tol):
  bf = tag == "bf16"
  k = f"pc_{tag}"
  x = golden.t(k + "/x", bf16=bf)
  w, s, zp = golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp")
  assert qo.max_abs_rel(qo.quantized_matmul(x, w, s), golden.t(k + "/out")) < tol
  assert qo.max_abs_rel(qo.quantized_matmul(x, w, s, zp), golden.t(k + "/out_zp")) < tol
  # without re-applying the dot rounding the oracle is the exact value: bf16 resolution away
  assert qo.max_abs_rel(qo.quantized_matmul(x, w, s, dot_round=None), golden.t(k + "/out")) < 8e-3


@pytest.mark.parametrize("tag", ["kat", "b128"])
def test_blockwise(golden, tag):
  k = f"bw_{tag}"
  x, w, s, zp = (golden.t(k + "/x"), golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp"))
  bs = int(golden.np(k + "/block_size"))
  ref = golden.t(k + "/out")
  assert qo.max_abs_rel(qo.quantized_matmul(x, w, s, block_size=bs), ref) < 2e-6
  assert qo.max_abs_rel(qo.quantized_matmul(x, w, s, zp, block_size=bs), golden.t(k + "/out_zp")) < 2e-6
  # the eager kernel ignores int4_weight
  assert torch.equal(ref, golden.t(k + "/out_int4flag"))
  if tag == "kat":
    # the reference test's known answer: x @ dequantised weight (test_quantized_matmul.py:205-218)
    w_dq = (w.float() * s.unsqueeze(1)).reshape(x.shape[1], -1)
    assert qo.max_abs_rel(qo.quantized_matmul(x, w, s, block_size=bs), x @ w_dq) < 2e-6


def test_layout_helpers():
  g = torch.Generator().manual_seed(7)
  w = torch.randint(-8, 8, (6, 8), generator=g, dtype=torch.int8)
  p = qo.pack_int4_nk(w)
  lo = (p & 0xF).to(torch.int8)
  hi = (p >> 4).to(torch.int8)
  lo = torch.where(lo > 7, lo - 16, lo)
  hi = torch.where(hi > 7, hi - 16, hi)
  assert torch.equal(torch.stack([lo, hi], -1).reshape(6, 8), w)
  sbn = qo.nk_to_sbn(w, 4)
  assert torch.equal(sbn, w.reshape(6, 2, 4).permute(1, 2, 0).contiguous())


def test_empty_inputs():
  x = torch.zeros(0, 8, dtype=torch.bfloat16)
  w = torch.zeros(4, 8, dtype=torch.int8)
  s = torch.ones(4)
  assert qo.quantized_matmul(x, w, s).shape == (0, 4)
  assert qo.quantized_matmul(x, w, s, quantize_activation=True).shape == (0, 4)


def test_torch_port_matches_reference_outputs(golden):
  """oracle/torch_port.py (the timed CPU baseline) reproduces the reference's outputs exactly."""
  from oracle import torch_port as tp
  for tag in ("bf16", "f32"):
    k = f"w8a8_{tag}"
    x = golden.t(k + "/x", bf16=(tag == "bf16"))
    w, s, zp = golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp")
    assert torch.equal(tp.quantized_matmul_cpu(x, w, s, quantize_activation=True), golden.t(k + "/out"))
    assert torch.allclose(tp.quantized_matmul_cpu(x, w, s, zp, quantize_activation=True), golden.t(k + "/out_zp"),
                          rtol=1e-6, atol=1e-6)
  for tag in ("bf16", "f32", "f32b"):
    k = f"pc_{tag}"
    x = golden.t(k + "/x", bf16=(tag == "bf16"))
    w, s, zp = golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp")
    assert torch.allclose(tp.quantized_matmul_cpu(x, w, s), golden.t(k + "/out"), rtol=1e-5, atol=1e-5)
    assert torch.allclose(tp.quantized_matmul_cpu(x, w, s, zp), golden.t(k + "/out_zp"), rtol=1e-5, atol=1e-5)
  for tag in ("kat", "b128"):
    k = f"bw_{tag}"
    x, w, s, zp = golden.t(k + "/x"), golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp")
    bs = int(golden.np(k + "/block_size"))
    assert torch.allclose(tp.quantized_matmul_cpu(x, w, s, block_size=bs), golden.t(k + "/out"), rtol=1e-5, atol=1e-5)
    assert torch.allclose(tp.quantized_matmul_cpu(x, w, s, zp, block_size=bs), golden.t(k + "/out_zp"), rtol=1e-5,
                          atol=1e-5)
