"""Host-side mirror of the reference interface: schemas, validators, module, dispatch; no GPU."""
import pytest
import torch

import xla_b200
from xla_b200 import quantized_matmul as qm


def test_schemas_match_the_reference_byte_for_byte():
  # torch_xla/experimental/xla_quantized_matmul.py:7-9
  assert str(torch.ops.xla.quantized_matmul.default._schema) == (
      "xla::quantized_matmul(Tensor x, Tensor w, Tensor scale, Tensor? zero_point=None, int? block_size=-1, "
      "bool? int4_weight=False, bool? quantize_activation=False) -> Tensor")
  # torch_xla/experimental/custom_kernel.py:1742-1744
  assert str(torch.ops.xla.quantized_matmul_int8.default._schema) == (
      "xla::quantized_matmul_int8(Tensor x, Tensor w, Tensor scalar, Tensor? zero_point=None, "
      "Tensor? quant_block_size=None, bool quantize_activation=False, int? batch_block_size=None, "
      "int? out_block_size=None, int? in_block_size=None) -> Tensor")
  s = str(torch.ops.xla_b200.quantized_matmul_packed.default._schema)
  assert "weight_is_packed" in s and "block_size" in s and "quantize_activation" in s


def test_cpu_tensors_fail_loudly():
  x, w, s = torch.zeros(2, 8), torch.zeros(4, 8, dtype=torch.int8), torch.ones(4)
  with pytest.raises(NotImplementedError):
    torch.ops.xla.quantized_matmul(x, w, s)
  with pytest.raises(NotImplementedError):
    torch.ops.xla.quantized_matmul_int8(x, w, s)
  with pytest.raises(RuntimeError, match="no CPU path"):
    qm.quantized_matmul_cuda(x, w, s)


def test_meta_kernels_give_reference_shapes_and_dtypes():
  meta = lambda *s, dtype=torch.float32: torch.empty(*s, dtype=dtype, device="meta")
  x = meta(2, 3, 64, dtype=torch.bfloat16)
  w = meta(16, 64, dtype=torch.int8)
  assert torch.ops.xla.quantized_matmul(x, w, meta(16)).shape == (2, 3, 16)
  # type promotion decides the output dtype (bf16 activations, fp32 scaler -> fp32)
  assert torch.ops.xla.quantized_matmul(x, w, meta(16)).dtype == torch.float32
  assert torch.ops.xla.quantized_matmul(x, w, meta(16, dtype=torch.bfloat16)).dtype == torch.bfloat16
  wb = meta(4, 16, 24, dtype=torch.int8)
  assert torch.ops.xla.quantized_matmul(x, wb, meta(4, 24), block_size=16).shape == (2, 3, 24)
  # the Pallas-registry op always returns x.dtype
  x2 = meta(5, 64, dtype=torch.bfloat16)
  o = torch.ops.xla.quantized_matmul_int8(x2, w, meta(16), quantize_activation=True)
  assert o.shape == (5, 16) and o.dtype == torch.bfloat16
  o = torch.ops.xla_b200.quantized_matmul_packed(x, meta(16, 32, dtype=torch.uint8), meta(4, 16), block_size=16,
                                                int4_weight=True, weight_is_packed=True, out_dtype=torch.bfloat16)
  assert o.shape == (2, 3, 16) and o.dtype == torch.bfloat16


def test_validators_raise_assertion_errors_with_reference_text():
  w = torch.zeros(8, 5, dtype=torch.int8)
  s = torch.ones(8)
  qm._check_per_channel_quant_weight_dtype_shapes(5, 8, w, s, None)
  with pytest.raises(AssertionError, match="Weight dtype is expected to be torch.int8"):
    qm._check_per_channel_quant_weight_dtype_shapes(5, 8, w.float(), s, None)
  with pytest.raises(AssertionError, match="Weight tensor is expected to be 2D, got 3D"):
    qm._check_per_channel_quant_weight_dtype_shapes(5, 8, w[None], s, None)
  with pytest.raises(AssertionError, match=r"Weight shape is expected to be \[output_dim, input_dim\]"):
    qm._check_per_channel_quant_weight_dtype_shapes(6, 8, w, s, None)
  with pytest.raises(AssertionError, match="weight scaler shape is expect to be"):
    qm._check_per_channel_quant_weight_dtype_shapes(5, 8, w, torch.ones(7), None)
  wb = torch.zeros(3, 2, 8, dtype=torch.int8)
  sb = torch.ones(3, 8)
  qm._check_blockwise_quant_weight_dtype_shapes(6, 8, 2, wb, sb, sb)
  with pytest.raises(AssertionError, match="input_dim should be divisible by block_size"):
    qm._check_blockwise_quant_weight_dtype_shapes(7, 8, 2, wb, sb, None)
  with pytest.raises(AssertionError, match="Weight tensor is expected to be 3D"):
    qm._check_blockwise_quant_weight_dtype_shapes(6, 8, 2, wb[0], sb, None)
  with pytest.raises(AssertionError, match="weight scaler is expected to be 2D"):
    qm._check_blockwise_quant_weight_dtype_shapes(6, 8, 2, wb, sb[0], None)
  with pytest.raises(AssertionError, match="zero_point shape is expect to be"):
    qm._check_blockwise_quant_weight_dtype_shapes(6, 8, 2, wb, sb, torch.ones(2, 8))


def test_module_mirrors_reference_buffers(golden):
  sym = xla_b200.XlaQuantizedLinear(32, 16, is_symmetric=True)
  asym = xla_b200.XlaQuantizedLinear(32, 16)
  assert sorted(sym.state_dict().keys()) == list(golden.np("module/state_keys_sym"))
  assert sorted(asym.state_dict().keys()) == list(golden.np("module/state_keys_asym"))
  assert sym.weight.dtype == torch.int8 and tuple(sym.weight.shape) == (16, 32)
  assert sym.weight_scaler.shape == (16,) and sym.zero_point is None
  with pytest.raises(AssertionError):
    sym.load_quantized_weight(torch.zeros(16, 31, dtype=torch.int8), torch.ones(16))
  blk = xla_b200.XlaQuantizedLinear(32, 16, is_symmetric=True, block_size=8, int4_weight=True)
  blk.load_quantized_weight(torch.zeros(4, 8, 16, dtype=torch.int8), torch.ones(4, 16))
  assert tuple(blk.weight.shape) == (4, 8, 16)
  # state round trip keeps the reference's names
  sym2 = xla_b200.XlaQuantizedLinear(32, 16, is_symmetric=True)
  sym2.load_state_dict(sym.state_dict())


def test_blockwise_rejects_activation_quantization_before_touching_the_gpu():
  x = torch.zeros(2, 6, device="meta")
  with pytest.raises(Exception):
    qm.quantized_matmul_cuda(x, torch.zeros(3, 2, 8, dtype=torch.int8), torch.ones(3, 8), block_size=2,
                             quantize_activation=True)


def test_variant_heuristic_is_shape_only():
  L = xla_b200._capi.lib()
  assert L.qmm_variant_for(xla_b200._capi.OP_W8A16_PERCHANNEL, 1, 4096, 4096, 0, 0) == b"mma"
  assert L.qmm_variant_for(xla_b200._capi.OP_W8A16_PERCHANNEL, 1, 4096, 4096, 0, 1) == b"gemv"  # zero point
  assert L.qmm_variant_for(xla_b200._capi.OP_W8A16_PERCHANNEL, 512, 4096, 4096, 0, 0) == b"tcgen05"
  assert L.qmm_variant_for(xla_b200._capi.OP_W8A16_PERCHANNEL, 3, 8, 5, 0, 0) == b"generic"
  assert L.qmm_variant_for(xla_b200._capi.OP_W4A16_BLOCKWISE_PACKED, 1, 14336, 4096, 128, 0) == b"mma"
  assert L.qmm_variant_for(xla_b200._capi.OP_W4A16_BLOCKWISE_PACKED, 64, 14336, 4096, 128, 0) == b"tcgen05"
  assert L.qmm_variant_for(xla_b200._capi.OP_W8A8_PERCHANNEL, 2048, 4096, 4096, 0, 0) == b"tcgen05"


def test_tuned_table_lookup_and_auto_choice():
  """The measured table (the counterpart of the reference's tuned block sizes, quantized_matmul_kernel.py:326-555)
  answers every shape family it was generated for, nothing else; AUTO follows it and falls back to the shape rule."""
  import re
  from xla_b200 import tune
  L = xla_b200._capi.lib()
  known = {0, 3, 4, 6}  # no entry, tcgen05, mma, i8tc
  for (n, k) in tune.REFERENCE_SHAPES + tune.BENCH_SHAPES:
    for (wbits, bs) in tune.FORMATS:
      if (bs and k % bs) or (wbits == 4 and k % 32):
        continue
      for m in (1, 2, 3, 8, 16, 32, 33, 64):
        v = L.qmm_tuned_variant(wbits, m, n, k, bs)
        assert v in known and v != 0, (wbits, bs, n, k, m, v)
      assert L.qmm_tuned_variant(wbits, 65, n, k, bs) == 0   # beyond the last batch bucket
  assert L.qmm_tuned_variant(8, 1, 4097, 4096, 0) == 0     # a shape the tuner never saw
  # the committed table and the tuner agree on the row format
  rows = [l for l in open(tune.__file__.replace("tune.py", "csrc/tuned_table.inc")) if l.startswith("{")]
  assert len(rows) >= 100 and all(re.match(r"\{[48], \d+, \d+, \d+, \{(\d, ){6}\d\}\},", r) for r in rows)
  # AUTO: table first, shape rule on a miss; zero points rule the split-activation kernel out
  assert L.qmm_weight_only_variant_for(4, 1, 28672, 8192, 128, 0) == b"i8tc"
  assert L.qmm_weight_only_variant_for(4, 1, 14336, 4096, 128, 0) == b"mma"
  assert L.qmm_weight_only_variant_for(8, 512, 4097 * 2, 4096, 0, 0) == b"i8tc"   # shape rule: above 64 tokens
  assert L.qmm_weight_only_variant_for(8, 1, 4097 * 2, 4096, 0, 0) == b"mma"      # shape rule: a small weight at M = 1
  assert L.qmm_weight_only_variant_for(8, 1, 28672, 8192, 0, 1) != b"i8tc"


def test_rtn_quantizer_layouts_and_reconstruction():
  """quantize_rtn reproduces the reference test helper's layouts (test_quantized_matmul.py:25-74)."""
  from xla_b200 import weight_prep as wp
  g = torch.Generator().manual_seed(0)
  w = torch.randn(8, 12, generator=g)
  q, s, zp = wp.quantize_rtn(w, n_bits=8)
  assert q.dtype == torch.int8 and q.shape == (8, 12) and s.shape == (8,) and zp is None
  assert (q.float() * s[:, None] - w).abs().max() <= s.max() * 0.51
  q, s, zp = wp.quantize_rtn(w, n_bits=4, block_size=4, symmetric=False)
  assert q.shape == (3, 4, 8) and s.shape == (3, 8) and zp.shape == (3, 8)
  assert int(q.min()) >= -8 and int(q.max()) <= 7
  # dequantise: w[n, b*bs+c] ~ q[b,c,n]*s[b,n] - zp[b,n]   (zp is in scaled units)
  w_dq = (q.float() * s[:, None, :] - zp[:, None, :]).permute(2, 0, 1).reshape(8, 12)
  assert (w_dq - w).abs().max() <= s.max() * 0.51
  lin = torch.nn.Linear(12, 8, bias=False)
  m = wp.quantize_linear(lin, n_bits=8, block_size=4)
  assert tuple(m.weight.shape) == (3, 4, 8) and m.block_size == 4 and m.zero_point is None

  class Net(torch.nn.Module):

    def __init__(self):
      super().__init__()
      self.a = torch.nn.Linear(12, 8, bias=False)
      self.b = torch.nn.Sequential(torch.nn.Linear(8, 8, bias=True), torch.nn.Linear(8, 4, bias=False))

  net = wp.swap_linears(Net(), n_bits=8)
  assert isinstance(net.a, xla_b200.XlaQuantizedLinear) and isinstance(net.b[1], xla_b200.XlaQuantizedLinear)
  assert isinstance(net.b[0], torch.nn.Linear)  # has a bias: left alone


def test_gate_up_interleave_round_trip():
  """Row order of the stacked gate/up weight: eight gate rows, eight up rows, and back."""
  from xla_b200 import mlp
  n, k = 24, 6
  wg = torch.arange(n * k, dtype=torch.int32).reshape(n, k)
  wu = -wg - 1
  w, s = mlp.interleave_gate_up(wg, wu, torch.arange(n, dtype=torch.float32), -torch.arange(n, dtype=torch.float32) - 1)
  assert w.shape == (2 * n, k) and s.shape == (2 * n,)
  assert torch.equal(w[0:8], wg[0:8]) and torch.equal(w[8:16], wu[0:8]) and torch.equal(w[16:24], wg[8:16])
  # a [M, 2N] result in that column order splits back into gate and up
  y = torch.stack([s, 2 * s])
  g, u = mlp._deinterleave(y)
  assert torch.equal(g[0], torch.arange(n, dtype=torch.float32)) and torch.equal(u[0], -torch.arange(n, dtype=torch.float32) - 1)
  # blockwise scales [S, N] interleave along N
  sg, su = torch.zeros(3, n), torch.ones(3, n)
  _, s2 = mlp.interleave_gate_up(wg, wu, sg, su, block_size=2)
  assert s2.shape == (3, 2 * n) and torch.equal(s2[:, 0:8], sg[:, 0:8]) and torch.equal(s2[:, 8:16], su[:, 0:8])
  w3, s3, sizes = mlp.concat_projections([wg, wu[:8]], [sg[0], su[0, :8]])
  assert sizes == [n, 8] and w3.shape == (n + 8, k) and s3.shape == (n + 8,)
  parts = mlp.split_outputs(torch.zeros(2, n + 8), sizes)
  assert [p.shape[-1] for p in parts] == sizes
