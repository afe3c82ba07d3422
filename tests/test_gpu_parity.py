"""GPU parity: the CUDA kernels (through the ops and the C ABI) against the CPU oracle and against
the golden outputs of the unmodified reference.

Tolerances (max|a-b| / max|b|): 1e-2 when the reference itself rounds through bf16, 1e-4 for outputs
that are fp32-accumulated and compared with the exact value of the formula; integer results
(quantized activations, scales, int32 accumulators, the fp32 W8A8 output) bit for bit.
"""
import ctypes

import pytest
import torch

import xla_b200
from oracle import qmm_oracle as qo
from tests import qmm_cases as qc
from xla_b200 import _capi

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL_BF16 = 1e-2
TOL_F32 = 1e-4


def cu(t):
  return None if t is None else t.to(DEV)


def op(*args, variant="auto", **kw):
  with xla_b200.force_variant(variant):
    return torch.ops.xla.quantized_matmul(*args, **kw)


def packed_op(*args, variant="auto", **kw):
  with xla_b200.force_variant(variant):
    return torch.ops.xla_b200.quantized_matmul_packed(*args, **kw)


def test_library_is_loaded_and_device_healthy():
  L = _capi.lib()
  flag = torch.zeros(1, dtype=torch.int32)
  import ctypes
  f = ctypes.c_uint32(7)
  with torch.cuda.device(0):
    assert L.qmm_device_error_flag(ctypes.byref(f), _capi.stream_ptr()) == 0
  assert f.value == 0 and flag.item() == 0
  assert torch.cuda.get_device_capability(0)[0] == 10, "these kernels are built for sm_100a only"


# ---------------------------------------------------------------------------------------------
# golden vectors of the reference, replayed on the GPU
# ---------------------------------------------------------------------------------------------


@pytest.mark.parametrize("tag,tol", [("bf16", TOL_BF16), ("f32", 1e-5), ("f32b", 1e-5)])
def test_golden_per_channel(golden, tag, tol):
  k = f"pc_{tag}"
  x = golden.t(k + "/x", bf16=(tag == "bf16"))
  w, s, zp = golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp")
  out = op(cu(x), cu(w), cu(s))
  ref = golden.t(k + "/out")
  assert out.dtype == ref.dtype and out.shape == ref.shape
  assert qo.max_abs_rel(out, ref) < tol
  out_zp = op(cu(x), cu(w), cu(s), cu(zp))
  assert qo.max_abs_rel(out_zp, golden.t(k + "/out_zp")) < tol


@pytest.mark.parametrize("tag", ["kat", "b128"])
def test_golden_blockwise(golden, tag):
  k = f"bw_{tag}"
  x, w, s, zp = golden.t(k + "/x"), golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp")
  bs = int(golden.np(k + "/block_size"))
  out = op(cu(x), cu(w), cu(s), block_size=bs)
  assert out.dtype == torch.float32
  assert qo.max_abs_rel(out, golden.t(k + "/out")) < 1e-5
  out = op(cu(x), cu(w), cu(s), cu(zp), block_size=bs, int4_weight=True)
  assert qo.max_abs_rel(out, golden.t(k + "/out_zp")) < 1e-5


def test_golden_quantizer_bit_exact(golden):
  x = golden.t("quant_bf16/x", bf16=True)
  xq_ref, s_ref = golden.t("quant_bf16/xq"), golden.t("quant_bf16/scale", bf16=True)
  xq, s = xla_b200.quantize_tensor(cu(x), saturate=False)  # wrap like the eager reference
  assert torch.equal(s.cpu().view(torch.int16), s_ref.view(torch.int16))
  assert torch.equal(xq.cpu(), xq_ref)
  xq_sat, _ = xla_b200.quantize_tensor(cu(x), saturate=True)
  diff = xq_sat.cpu() != xq_ref
  assert int(diff.sum()) == int(golden.np("quant_bf16/n_plus128"))
  assert bool((xq_sat.cpu()[diff] == 127).all())
  x = golden.t("quant_f32/x")
  xq, s = xla_b200.quantize_tensor(cu(x), saturate=False)
  assert torch.equal(xq.cpu(), golden.t("quant_f32/xq")) and torch.equal(s.cpu(), golden.t("quant_f32/scale"))


@pytest.mark.parametrize("tag", ["bf16", "f32"])
@pytest.mark.parametrize("variant", ["generic", "tcgen05"])
def test_golden_w8a8_bit_exact(golden, tag, variant):
  k = f"w8a8_{tag}"
  x = golden.t(k + "/x", bf16=(tag == "bf16"))
  w, s, zp = golden.t(k + "/w"), golden.t(k + "/scale"), golden.t(k + "/zp")
  xla_b200.set_activation_saturation(False)  # the golden outputs come from the wrapping eager kernel
  try:
    out = op(cu(x), cu(w), cu(s), quantize_activation=True, variant=variant)
    out_zp = op(cu(x), cu(w), cu(s), cu(zp), quantize_activation=True, variant=variant)
  finally:
    xla_b200.set_activation_saturation(True)
  assert out.dtype == torch.float32
  assert torch.equal(out.cpu(), golden.t(k + "/out"))
  assert qo.max_abs_rel(out_zp, golden.t(k + "/out_zp")) < 2e-6
  # the int32 accumulator through the C ABI
  xq = cu(golden.t(k + "/xq"))
  M, K = xq.shape
  N = w.shape[0]
  acc = torch.empty((M, N), dtype=torch.int32, device=DEV)
  with torch.cuda.device(0):
    _capi.check(_capi.lib().qmm_w8a8_gemm(_capi.ptr(xq), _capi.ptr(cu(w)), None, None, None, None, _capi.ptr(acc),
                                         None, 0, M, N, K, _capi.VARIANTS[variant], _capi.stream_ptr()))
  assert torch.equal(acc.cpu(), golden.t(k + "/acc"))


def test_golden_module(golden):
  m = xla_b200.XlaQuantizedLinear(32, 16, is_symmetric=True)
  m.load_quantized_weight(cu(golden.t("module/w")), cu(golden.t("module/scale")))
  out = m(cu(golden.t("module/x")))
  ref = golden.t("module/out")
  assert out.shape == ref.shape and qo.max_abs_rel(out, ref) < 1e-5


# ---------------------------------------------------------------------------------------------
# per-channel W8A16 against the oracle (configuration: x [16,4096], w [4096,4096])
# ---------------------------------------------------------------------------------------------


@pytest.mark.parametrize("M,variant", [(1, "gemv"), (2, "gemv"), (3, "gemv"), (4, "gemv"), (8, "gemv"), (16, "generic"),
                                       (16, "auto"), (1, "generic"), (5, "auto")])
def test_w8a16_per_channel_vs_oracle(M, variant):
  g = qc.gen(0)
  N, K = 1024, 4096
  x = qc.activations(g, M, K)
  w = qc.int8_weight(g, N, K)
  s = qc.per_channel_scale(g, N)
  out = op(cu(x), cu(w), cu(s), variant=variant)
  assert out.dtype == torch.float32 and out.shape == (M, N)
  exact = qo.quantized_matmul(x, w, s, dot_round=None)
  refpath = qo.quantized_matmul(x, w, s, dot_round="x")
  assert qo.max_abs_rel(out, exact) < TOL_F32
  assert qo.max_abs_rel(out, refpath) < TOL_BF16
  # bf16 output (scaler given in bf16 -> promotion yields bf16)
  out_bf = op(cu(x), cu(w), cu(s.bfloat16()), variant=variant)
  assert out_bf.dtype == torch.bfloat16
  assert qo.max_abs_rel(out_bf, qo.quantized_matmul(x, w, s.bfloat16().float(), dot_round="x")) < TOL_BF16


@pytest.mark.parametrize("xdtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("variant", ["gemv", "generic"])
def test_w8a16_activation_dtypes_and_zero_point(xdtype, variant):
  g = qc.gen(1)
  M, N, K = 3, 520, 1024  # N is not a multiple of the 8-row CTA tile
  x = qc.activations(g, M, K, dtype=xdtype)
  w = qc.int8_weight(g, N, K)
  s = qc.per_channel_scale(g, N)
  zp = torch.randint(-8, 9, (N,), generator=g).float() * s
  tol = TOL_F32 if xdtype == torch.float32 else 2e-4
  out = op(cu(x), cu(w), cu(s), cu(zp), variant=variant)
  assert qo.max_abs_rel(out, qo.quantized_matmul(x, w, s, zp, dot_round=None)) < tol


def test_full_size_config1_all_paths_agree():
  """x [16,4096] bf16, w [4096,4096] int8, fp32 scaler, through the module like the reference test."""
  g = qc.gen(0)
  x = qc.activations(g, 16, 4096)
  w = qc.int8_weight(g, 4096, 4096)
  s = qc.per_channel_scale(g, 4096)
  m = xla_b200.XlaQuantizedLinear(4096, 4096, is_symmetric=True)
  m.load_quantized_weight(cu(w), cu(s))
  out = m(cu(x))
  exact = qo.quantized_matmul(x, w, s, dot_round=None)
  assert qo.max_abs_rel(out, exact) < TOL_F32
  with xla_b200.force_variant("generic"):
    out_g = m(cu(x))
  assert qo.max_abs_rel(out_g, exact) < TOL_F32


# ---------------------------------------------------------------------------------------------
# blockwise int4 (configuration: w [14336,4096] packed, block 128, M in {1,8,32})
# ---------------------------------------------------------------------------------------------


def _int4_case(g, M, N, K, bs):
  x = qc.activations(g, M, K)
  w_nk = qc.int4_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N)
  return x, w_nk, s


@pytest.mark.parametrize("M,variant", [(1, "gemv"), (8, "gemv"), (1, "generic"), (32, "generic"), (1, "auto"), (8, "auto"),
                                       (32, "auto")])
def test_w4a16_blockwise_packed_vs_oracle(M, variant):
  g = qc.gen(2)
  N, K, bs = 1536, 4096, 128
  x, w_nk, s = _int4_case(g, M, N, K, bs)
  w_sbn = qc.to_sbn(w_nk, bs)
  wp = xla_b200.pack_int4(cu(w_nk))
  assert torch.equal(wp.cpu(), qo.pack_int4_nk(w_nk))
  assert torch.equal(xla_b200.pack_int4(cu(w_sbn), layout="sbn").cpu(), wp.cpu())
  assert torch.equal(xla_b200.unpack_int4(wp).cpu(), w_nk)
  # the reference raises for bf16 x with an fp32 scaler; the oracle takes the exact upcast
  exact = qo.quantized_matmul(x.float(), w_sbn, s, block_size=bs, dot_round=None)
  out = packed_op(cu(x), wp, cu(s), block_size=bs, int4_weight=True, weight_is_packed=True, variant=variant)
  assert out.dtype == torch.float32 and out.shape == (M, N)
  assert qo.max_abs_rel(out, exact) < TOL_F32
  out_bf = packed_op(cu(x), wp, cu(s), block_size=bs, int4_weight=True, weight_is_packed=True,
                     out_dtype=torch.bfloat16, variant=variant)
  assert out_bf.dtype == torch.bfloat16 and qo.max_abs_rel(out_bf, exact) < TOL_BF16
  # same weights through the reference-layout op
  if M <= 8:
    out_ref_layout = op(cu(x), cu(w_sbn), cu(s), block_size=bs, int4_weight=True)
    assert qo.max_abs_rel(out_ref_layout, exact) < TOL_F32


def test_full_size_config2_decode():
  g = qc.gen(0)
  N, K, bs = 14336, 4096, 128
  x, w_nk, s = _int4_case(g, 8, N, K, bs)
  wp = xla_b200.pack_int4(cu(w_nk))
  exact = qo.quantized_matmul(x.float(), qc.to_sbn(w_nk, bs), s, block_size=bs, dot_round=None)
  for M in (1, 8):
    out = packed_op(cu(x[:M]), wp, cu(s), block_size=bs, int4_weight=True, weight_is_packed=True,
                    out_dtype=torch.bfloat16)
    assert qo.max_abs_rel(out, exact[:M]) < TOL_BF16


@pytest.mark.parametrize("variant", ["gemv", "generic"])
def test_w4a16_zero_point_and_per_channel_packed(variant):
  g = qc.gen(3)
  M, N, K, bs = 2, 264, 512, 64
  x, w_nk, s = _int4_case(g, M, N, K, bs)
  zp = torch.randint(-3, 4, (K // bs, N), generator=g).float() * s
  wp = xla_b200.pack_int4(cu(w_nk))
  out = packed_op(cu(x), wp, cu(s), cu(zp), block_size=bs, int4_weight=True, weight_is_packed=True, variant=variant)
  exact = qo.quantized_matmul(x.float(), qc.to_sbn(w_nk, bs), s, zp, block_size=bs, dot_round=None)
  assert qo.max_abs_rel(out, exact) < TOL_F32
  s1 = qc.per_channel_scale(g, N)
  z1 = torch.randint(-3, 4, (N,), generator=g).float() * s1
  out = packed_op(cu(x), wp, cu(s1), cu(z1), int4_weight=True, weight_is_packed=True, variant=variant)
  assert qo.max_abs_rel(out, qo.quantized_matmul(x, w_nk, s1, z1, dot_round=None)) < TOL_F32


def test_blockwise_module_prepacks_int4():
  g = qc.gen(4)
  M, N, K, bs = 4, 512, 1024, 128
  x, w_nk, s = _int4_case(g, M, N, K, bs)
  w_sbn = qc.to_sbn(w_nk, bs)
  m = xla_b200.XlaQuantizedLinear(K, N, is_symmetric=True, block_size=bs, int4_weight=True)
  m.load_quantized_weight(cu(w_sbn), cu(s))
  exact = qo.quantized_matmul(x.float(), w_sbn, s, block_size=bs, dot_round=None)
  out = m(cu(x))
  assert m._packed is not None and out.dtype == torch.float32
  assert qo.max_abs_rel(out, exact) < TOL_F32
  m2 = xla_b200.XlaQuantizedLinear(K, N, is_symmetric=True, block_size=bs, int4_weight=True, prepack=False)
  m2.load_quantized_weight(cu(w_sbn), cu(s))
  assert qo.max_abs_rel(m2(cu(x)), exact) < TOL_F32


# ---------------------------------------------------------------------------------------------
# W8A8 (configuration: x [2048,4096] with outliers, w [4096,4096])
# ---------------------------------------------------------------------------------------------


@pytest.mark.parametrize("variant", ["generic", "tcgen05"])
@pytest.mark.parametrize("M,N,K", [(256, 512, 4096), (130, 264, 144), (16, 4096, 4096), (1, 256, 128),
                                   (300, 37 * 256 + 40, 272), (512, 9472, 128)])
def test_w8a8_vs_oracle(variant, M, N, K):
  # the last two shapes have enough 256 x 256 tiles for the two-accumulator kernel (ragged and exact edges)
  g = qc.gen(5)
  x = qc.activations(g, M, K, outliers=True)
  w = qc.int8_weight(g, N, K)
  s = qc.per_channel_scale(g, N)
  xq_ref, xs_ref = qo.quantize_act(x, wrap=False)
  xq, xs = xla_b200.quantize_tensor(cu(x))
  assert torch.equal(xq.cpu(), xq_ref) and torch.equal(xs.cpu().view(torch.int16), xs_ref.view(torch.int16))
  acc_ref = qo.int8_gemm_i32(xq_ref, w)
  acc = torch.empty((M, N), dtype=torch.int32, device=DEV)
  with torch.cuda.device(0):
    _capi.check(_capi.lib().qmm_w8a8_gemm(_capi.ptr(xq), _capi.ptr(cu(w)), None, None, None, None, _capi.ptr(acc),
                                         None, 0, M, N, K, _capi.VARIANTS[variant], _capi.stream_ptr()))
  assert torch.equal(acc.cpu(), acc_ref), "int32 accumulator must be bit-exact"
  out = op(cu(x), cu(w), cu(s), quantize_activation=True, variant=variant)
  ref = qo.quantized_matmul(x, w, s, quantize_activation=True, wrap=False)
  assert torch.equal(out.cpu(), ref), "fp32 W8A8 output must be bit-exact"
  out_bf = torch.ops.xla.quantized_matmul_int8(cu(x), cu(w), cu(s), quantize_activation=True)
  assert out_bf.dtype == torch.bfloat16
  assert torch.equal(out_bf.cpu(), ref.bfloat16())


def test_full_size_config3_properties():
  """M=2048, K=N=4096: the tensor-core accumulator equals the CUDA-core one and a checksum in int64."""
  g = qc.gen(0)
  M, N, K = 2048, 4096, 4096
  x = cu(qc.activations(g, M, K, outliers=True))
  w = cu(qc.int8_weight(g, N, K))
  xq, xs = xla_b200.quantize_tensor(x)
  xq_ref, xs_ref = qo.quantize_act(x.cpu(), wrap=False)
  assert torch.equal(xq.cpu(), xq_ref) and torch.equal(xs.cpu().view(torch.int16), xs_ref.view(torch.int16))
  accs = {}
  for variant in ("tcgen05", "generic"):
    acc = torch.empty((M, N), dtype=torch.int32, device=DEV)
    with torch.cuda.device(0):
      _capi.check(_capi.lib().qmm_w8a8_gemm(_capi.ptr(xq), _capi.ptr(w), None, None, None, None, _capi.ptr(acc), None,
                                           0, M, N, K, _capi.VARIANTS[variant], _capi.stream_ptr()))
    accs[variant] = acc
  assert torch.equal(accs["tcgen05"], accs["generic"])
  # sum_n acc[m,n] == sum_k xq[m,k] * (sum_n w[n,k])
  lhs = accs["tcgen05"].to(torch.int64).sum(dim=1)
  rhs = (xq.to(torch.int64) * w.to(torch.int64).sum(dim=0)).sum(dim=1)
  assert torch.equal(lhs, rhs)
  # a slice against the CPU oracle
  sl = qo.int8_gemm_i32(xq_ref[100:132], w.cpu())
  assert torch.equal(accs["tcgen05"][100:132].cpu(), sl)


# ---------------------------------------------------------------------------------------------
# edge cases
# ---------------------------------------------------------------------------------------------


def test_empty_and_ragged_inputs():
  w = cu(torch.zeros(8, 16, dtype=torch.int8))
  s = cu(torch.ones(8))
  assert op(cu(torch.zeros(0, 16, dtype=torch.bfloat16)), w, s).shape == (0, 8)
  assert op(cu(torch.zeros(2, 0, 16)), w, s).shape == (2, 0, 8)
  assert op(cu(torch.zeros(0, 16)), w, s, quantize_activation=True).shape == (0, 8)
  g = qc.gen(6)
  # K not a multiple of 16: only the generic kernels take it
  x = torch.randn(3, 7, 37, generator=g)
  w = torch.randint(-127, 128, (11, 37), generator=g, dtype=torch.int8)
  s = qc.per_channel_scale(g, 11)
  out = op(cu(x), cu(w), cu(s))
  assert out.shape == (3, 7, 11)
  assert qo.max_abs_rel(out, qo.quantized_matmul(x, w, s, dot_round=None)) < 1e-5
  out = op(cu(x), cu(w), cu(s), quantize_activation=True)
  assert torch.equal(out.cpu(), qo.quantized_matmul(x, w, s, quantize_activation=True))
  # a non-contiguous activation view
  xt = torch.randn(37, 5, generator=g).t()
  assert qo.max_abs_rel(op(cu(xt), cu(w), cu(s)), qo.quantized_matmul(xt.contiguous(), w, s, dot_round=None)) < 1e-5
  # all-zero row: the reference divides by a zero scale; the kernel yields zeros, not NaN garbage
  xz = torch.zeros(2, 64, dtype=torch.bfloat16)
  xq, xs = xla_b200.quantize_tensor(cu(xz))
  assert int(xq.abs().max()) == 0 and float(xs.abs().max()) == 0.0


def test_errors_match_the_reference():
  x = cu(torch.zeros(2, 6))
  with pytest.raises(AssertionError, match="Blockwise quantization does not support activation quantization."):
    op(x, cu(torch.zeros(3, 2, 8, dtype=torch.int8)), cu(torch.ones(3, 8)), block_size=2, quantize_activation=True)
  with pytest.raises(AssertionError, match="Weight dtype is expected to be torch.int8"):
    op(x, cu(torch.zeros(8, 6)), cu(torch.ones(8)))
  with pytest.raises(AssertionError, match="Weight shape is expected to be"):
    op(x, cu(torch.zeros(8, 5, dtype=torch.int8)), cu(torch.ones(8)))
  with pytest.raises(AssertionError, match="zero_point is not supported"):
    torch.ops.xla.quantized_matmul_int8(x, cu(torch.zeros(8, 6, dtype=torch.int8)), cu(torch.ones(8)), cu(torch.ones(8)))
  with pytest.raises(NotImplementedError):  # a forced variant never silently becomes another one
    op(cu(torch.zeros(2, 37)), cu(torch.zeros(8, 37, dtype=torch.int8)), cu(torch.ones(8)), variant="gemv")


def test_llama_layer_shapes_decode():
  """q/o 4096->4096, k/v 4096->1024, gate/up 4096->14336, down 14336->4096 at M in {1,16}."""
  g = qc.gen(7)
  for (K, N) in ((4096, 1024), (4096, 14336), (14336, 4096)):
    w = qc.int8_weight(g, N, K)
    s = qc.per_channel_scale(g, N)
    x = qc.activations(g, 16, K)
    exact = qo.quantized_matmul(x, w, s, dot_round=None)
    wc, sc = cu(w), cu(s)
    for M in (1, 16):
      out = op(cu(x[:M]), wc, sc)
      assert qo.max_abs_rel(out, exact[:M]) < TOL_F32, (K, N, M)


# ---------------------------------------------------------------------------------------------
# weight-only tensor-core kernel (tcgen05 after shared-memory dequant), decode to prefill
# ---------------------------------------------------------------------------------------------


@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 5, 16, 33, 64, 100, 300])
def test_tc_w8a16_per_channel(M, xdtype):
  g = qc.gen(10)
  N, K = 1000, 2112  # N not a multiple of 128, K = 33 tiles of 64
  x = qc.activations(g, M, K, dtype=xdtype)
  w = qc.int8_weight(g, N, K)
  s = qc.per_channel_scale(g, N)
  out = op(cu(x), cu(w), cu(s), variant="tcgen05")
  assert out.dtype == torch.float32
  assert qo.max_abs_rel(out, qo.quantized_matmul(x, w, s, dot_round=None)) < TOL_F32


@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,bs", [(1, 128), (8, 128), (32, 128), (64, 64), (100, 256), (16, -1)])
def test_tc_w4a16_packed(M, bs, xdtype):
  g = qc.gen(11)
  N, K = 1160, 2048
  x = qc.activations(g, M, K, dtype=xdtype)
  w_nk = qc.int4_weight(g, N, K)
  wp = xla_b200.pack_int4(cu(w_nk))
  if bs == -1:
    s = qc.per_channel_scale(g, N)
    exact = qo.quantized_matmul(x, w_nk, s, dot_round=None)
  else:
    s = qc.blockwise_scale(g, K // bs, N)
    exact = qo.quantized_matmul(x.float(), qc.to_sbn(w_nk, bs), s, block_size=bs, dot_round=None)
  out = packed_op(cu(x), wp, cu(s), block_size=bs, int4_weight=True, weight_is_packed=True, variant="tcgen05")
  assert out.dtype == torch.float32 and out.shape == (M, N)
  assert qo.max_abs_rel(out, exact) < TOL_F32


def test_tc_kernel_is_deterministic_and_leaves_no_error():
  import ctypes
  g = qc.gen(12)
  M, N, K, bs = 32, 14336, 4096, 128
  x = cu(qc.activations(g, M, K))
  wp = cu(torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8))
  s = cu(qc.blockwise_scale(g, K // bs, N))
  outs = [packed_op(x, wp, s, block_size=bs, int4_weight=True, weight_is_packed=True, out_dtype=torch.bfloat16,
                    variant="tcgen05") for _ in range(20)]
  for o in outs[1:]:
    assert torch.equal(o, outs[0])
  f = ctypes.c_uint32(7)
  with torch.cuda.device(0):
    assert _capi.lib().qmm_device_error_flag(ctypes.byref(f), _capi.stream_ptr()) == 0
  assert f.value == 0
  # and it agrees with the CUDA-core kernel on the same inputs
  ref = packed_op(x[:8], wp, s, block_size=bs, int4_weight=True, weight_is_packed=True, variant="gemv")
  got = packed_op(x[:8], wp, s, block_size=bs, int4_weight=True, weight_is_packed=True, variant="tcgen05")
  assert qo.max_abs_rel(got, ref) < 1e-5


def test_prefill_llama_shapes_tc():
  """M=512 prefill on the layer's widest and deepest linears, against the oracle on a row sample."""
  g = qc.gen(13)
  for (K, N) in ((4096, 14336), (14336, 4096)):
    w = qc.int8_weight(g, N, K)
    s = qc.per_channel_scale(g, N)
    x = qc.activations(g, 512, K)
    out = op(cu(x), cu(w), cu(s), variant="tcgen05")
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 300, 511])
    exact = qo.quantized_matmul(x[rows], w, s, dot_round=None)
    assert qo.max_abs_rel(out[rows.to(DEV)], exact) < TOL_F32, (K, N)


# ---------------------------------------------------------------------------------------------
# decode kernel with register dequant into warp-level MMAs (M <= 32)
# ---------------------------------------------------------------------------------------------


@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,bs", [(1, 128), (7, 128), (8, 128), (9, 256), (16, 128), (17, 128), (32, 128), (4, -1), (24, -1)])
def test_mma_w4a16_packed(M, bs, xdtype):
  g = qc.gen(20)
  N, K = 1000, 2304  # N not a multiple of 16; K = 18 steps of 128
  x = qc.activations(g, M, K, dtype=xdtype)
  w_nk = qc.int4_weight(g, N, K)
  wp = xla_b200.pack_int4(cu(w_nk))
  if bs == -1:
    s = qc.per_channel_scale(g, N)
    exact = qo.quantized_matmul(x, w_nk, s, dot_round=None)
  else:
    s = qc.blockwise_scale(g, K // bs, N)
    exact = qo.quantized_matmul(x.float(), qc.to_sbn(w_nk, bs), s, block_size=bs, dot_round=None)
  out = packed_op(cu(x), wp, cu(s), block_size=bs, int4_weight=True, weight_is_packed=True, variant="mma")
  assert out.dtype == torch.float32 and out.shape == (M, N)
  assert qo.max_abs_rel(out, exact) < TOL_F32


@pytest.mark.parametrize("xdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 8, 13, 16, 32])
def test_mma_w8a16_per_channel(M, xdtype):
  g = qc.gen(21)
  N, K = 1000, 2112  # 33 steps of 64
  x = qc.activations(g, M, K, dtype=xdtype)
  w = qc.int8_weight(g, N, K)
  s = qc.per_channel_scale(g, N)
  out = op(cu(x), cu(w), cu(s), variant="mma")
  assert qo.max_abs_rel(out, qo.quantized_matmul(x, w, s, dot_round=None)) < TOL_F32
  with pytest.raises(NotImplementedError):
    op(cu(qc.activations(g, 33, K, dtype=xdtype)), cu(w), cu(s), variant="mma")


@pytest.mark.parametrize("N", [148 * 16 * 2 + 5, 148 * 16 * 3 + 40, 20000])
def test_mma_staged_tile_slots_and_rounds(N):
  """9..32 tokens: the per-SM kernel with 2, 4 and 8 row tiles per CTA, and more than one round of tiles."""
  g = qc.gen(22)
  K, bs, M = 1024, 128, 20
  x = qc.activations(g, M, K)
  w_nk = qc.int4_weight(g, N, K)
  wp = xla_b200.pack_int4(cu(w_nk))
  s = qc.blockwise_scale(g, K // bs, N)
  exact = qo.quantized_matmul(x.float(), qc.to_sbn(w_nk, bs), s, block_size=bs, dot_round=None)
  out = packed_op(cu(x), wp, cu(s), block_size=bs, int4_weight=True, weight_is_packed=True, variant="mma")
  assert qo.max_abs_rel(out, exact) < TOL_F32


# ---------------------------------------------------------------------------------------------
# decode kernel with the weight operand in tensor memory (tcgen05, M <= 32, cluster split-K)
# ---------------------------------------------------------------------------------------------


# ---------------------------------------------------------------------------------------------
# int8 blockwise weights stored K-minor (what the module keeps for the fast kernels)
# ---------------------------------------------------------------------------------------------


@pytest.mark.parametrize("M", [1, 8, 20, 64, 300])
@pytest.mark.parametrize("with_zp", [False, True])
def test_w8a16_blockwise_k_minor(M, with_zp):
  g = qc.gen(50)
  N, K, bs = 1000, 1024, 128
  x = qc.activations(g, M, K)
  w_nk = qc.int8_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N)
  zp = (qc.blockwise_scale(g, K // bs, N) - 0.02) if with_zp else None
  exact = qo.quantized_matmul(x.float(), qc.to_sbn(w_nk, bs), s, zp, block_size=bs, dot_round=None)
  out = packed_op(cu(x), cu(w_nk), cu(s), None if zp is None else cu(zp), block_size=bs)
  assert out.dtype == torch.float32 and out.shape == (M, N)
  assert qo.max_abs_rel(out, exact) < TOL_F32


def test_module_per_channel_int4_is_packed_once():
  """XlaQuantizedLinear(int4_weight=True), per channel: the int8 container is packed to half the bytes on first use."""
  g = qc.gen(52)
  N, K, M = 512, 1024, 4
  x = qc.activations(g, M, K)
  w = qc.int4_weight(g, N, K)
  s = qc.per_channel_scale(g, N)
  m = xla_b200.XlaQuantizedLinear(K, N, is_symmetric=True, int4_weight=True)
  m.load_quantized_weight(cu(w), cu(s))
  y = m(cu(x))
  wp, is_packed = m._packed_weight()
  assert is_packed and wp.shape == (N, K // 2) and wp.dtype == torch.uint8
  assert qo.max_abs_rel(y, qo.quantized_matmul(x, w, s, dot_round=None)) < TOL_F32
  assert torch.equal(xla_b200.unpack_int4(wp).cpu(), w)


def test_module_int8_blockwise_uses_k_minor_copy():
  """XlaQuantizedLinear(block_size>0, int8): reference layout in, K-minor copy built once, same results as the op."""
  g = qc.gen(51)
  N, K, bs, M = 512, 1024, 128, 4
  x = qc.activations(g, M, K)
  w_nk = qc.int8_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N)
  m = xla_b200.XlaQuantizedLinear(K, N, is_symmetric=True, block_size=bs)
  m.load_quantized_weight(cu(qc.to_sbn(w_nk, bs)), cu(s))
  y = m(cu(x))
  w_copy, is_packed = m._packed_weight()
  assert not is_packed and w_copy.shape == (N, K) and torch.equal(w_copy.cpu(), w_nk)
  exact = qo.quantized_matmul(x.float(), qc.to_sbn(w_nk, bs), s, block_size=bs, dot_round=None)
  assert qo.max_abs_rel(y, exact) < TOL_F32
  # the reference-layout operator gives the same numbers through the any-shape kernels
  y_ref = torch.ops.xla.quantized_matmul(cu(x), cu(qc.to_sbn(w_nk, bs)), cu(s), None, block_size=bs)
  assert qo.max_abs_rel(y_ref, exact) < TOL_F32


# ---------------------------------------------------------------------------------------------
# fused gate + up projection with silu(gate) * up, and concatenated projections
# ---------------------------------------------------------------------------------------------


def _silu_mul(g, u):
  g, u = g.double(), u.double()
  return g / (1 + torch.exp(-g)) * u


@pytest.mark.parametrize("M", [1, 8, 20, 32, 40])
@pytest.mark.parametrize("mode", ["w4_blockwise", "w8_per_channel"])
def test_gate_up_fused(M, mode):
  """One kernel for both projections and the activation (M <= 32); the stacked-linear path above that."""
  g = qc.gen(40)
  N, K, bs = 1000 - 1000 % 8, 1024, 128
  x = qc.activations(g, M, K)
  if mode == "w4_blockwise":
    wg, wu = qc.int4_weight(g, N, K), qc.int4_weight(g, N, K)
    sg, su = qc.blockwise_scale(g, K // bs, N), qc.blockwise_scale(g, K // bs, N)
    gate = qo.quantized_matmul(x.float(), qc.to_sbn(wg, bs), sg, block_size=bs, dot_round=None)
    up = qo.quantized_matmul(x.float(), qc.to_sbn(wu, bs), su, block_size=bs, dot_round=None)
    w, s = xla_b200.interleave_gate_up(xla_b200.pack_int4(cu(wg)), xla_b200.pack_int4(cu(wu)), cu(sg), cu(su), bs)
    out = torch.ops.xla_b200.quantized_gate_up(cu(x), w, s, block_size=bs, int4_weight=True, weight_is_packed=True)
  else:
    wg, wu = qc.int8_weight(g, N, K), qc.int8_weight(g, N, K)
    sg, su = qc.per_channel_scale(g, N), qc.per_channel_scale(g, N)
    gate = qo.quantized_matmul(x, wg, sg, dot_round=None)
    up = qo.quantized_matmul(x, wu, su, dot_round=None)
    w, s = xla_b200.interleave_gate_up(cu(wg), cu(wu), cu(sg), cu(su))
    out = torch.ops.xla_b200.quantized_gate_up(cu(x), w, s)
  assert out.shape == (M, N) and out.dtype == torch.float32
  assert qo.max_abs_rel(out, _silu_mul(gate, up)) < TOL_F32
  # bf16 output: one rounding of the fp32 result
  if mode == "w4_blockwise":
    out16 = torch.ops.xla_b200.quantized_gate_up(cu(x), w, s, block_size=bs, int4_weight=True, weight_is_packed=True,
                                                 out_dtype=torch.bfloat16)
    assert out16.dtype == torch.bfloat16
    assert qo.max_abs_rel(out16, _silu_mul(gate, up)) < TOL_BF16


@pytest.mark.parametrize("M", [33, 64, 100, 600])
@pytest.mark.parametrize("mode", ["w4_blockwise", "w8_per_channel"])
def test_gate_up_fused_large_batches(M, mode):
  """Above 32 tokens the split-activation kernel applies silu(gate) * up in its drain: one launch, no [M, 2N] round trip."""
  g = qc.gen(44)
  N, K, bs = 1000 - 1000 % 8, 1024, 128
  x = qc.activations(g, M, K)
  if mode == "w4_blockwise":
    wg, wu = qc.int4_weight(g, N, K), qc.int4_weight(g, N, K)
    sg, su = qc.blockwise_scale(g, K // bs, N), qc.blockwise_scale(g, K // bs, N)
    gate = qo.quantized_matmul(x.float(), qc.to_sbn(wg, bs), sg, block_size=bs, dot_round=None)
    up = qo.quantized_matmul(x.float(), qc.to_sbn(wu, bs), su, block_size=bs, dot_round=None)
    w, s = xla_b200.interleave_gate_up(xla_b200.pack_int4(cu(wg)), xla_b200.pack_int4(cu(wu)), cu(sg), cu(su), bs)
    kw = dict(block_size=bs, int4_weight=True, weight_is_packed=True)
  else:
    wg, wu = qc.int8_weight(g, N, K), qc.int8_weight(g, N, K)
    sg, su = qc.per_channel_scale(g, N), qc.per_channel_scale(g, N)
    gate = qo.quantized_matmul(x, wg, sg, dot_round=None)
    up = qo.quantized_matmul(x, wu, su, dot_round=None)
    w, s = xla_b200.interleave_gate_up(cu(wg), cu(wu), cu(sg), cu(su))
    kw = {}
  want = _silu_mul(gate, up)
  out = torch.ops.xla_b200.quantized_gate_up(cu(x), w, s, **kw)
  assert out.shape == (M, N) and out.dtype == torch.float32
  assert qo.max_abs_rel(out, want) < TOL_F32
  out16 = torch.ops.xla_b200.quantized_gate_up(cu(x), w, s, out_dtype=torch.bfloat16, **kw)
  assert out16.dtype == torch.bfloat16
  assert qo.max_abs_rel(out16, want) < TOL_BF16
  with xla_b200.force_variant("tcgen05"):  # the stacked-linear route computes the same thing
    ref = torch.ops.xla_b200.quantized_gate_up(cu(x), w, s, **kw)
  assert qo.max_abs_rel(out, ref.cpu()) < TOL_F32


def test_w8a8_outputs_at_odd_offsets():
  """fp32 `out` and int32 `acc_out` that are only 4-byte aligned (views one element into a buffer): the tensor-core
  epilogue must fall back from its 16-byte stores and give the same bits as with aligned outputs."""
  from xla_b200 import _capi
  L = _capi.lib()
  g = qc.gen(61)
  M, N, K = 256, 512, 1024
  xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).to(DEV)
  w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(DEV)
  ws = qc.per_channel_scale(g, N).to(DEV)
  xs = (torch.rand(M, generator=g) * 0.05 + 0.01).to(DEV)

  def run(out, acc):
    with torch.cuda.device(0):
      _capi.check(L.qmm_w8a8_gemm(_capi.ptr(xq), _capi.ptr(w), _capi.ptr(ws), None, _capi.ptr(xs), None, acc, out, _capi.F32,
                                  M, N, K, _capi.VARIANTS["tcgen05"], _capi.stream_ptr()))
      torch.cuda.synchronize()

  out_a = torch.empty(M * N, dtype=torch.float32, device=DEV)
  acc_a = torch.empty(M * N, dtype=torch.int32, device=DEV)
  run(out_a.data_ptr(), acc_a.data_ptr())
  out_b = torch.zeros(M * N + 1, dtype=torch.float32, device=DEV)
  acc_b = torch.zeros(M * N + 1, dtype=torch.int32, device=DEV)
  run(out_b.data_ptr() + 4, acc_b.data_ptr() + 4)
  assert torch.equal(out_b[1:], out_a) and torch.equal(acc_b[1:], acc_a)
  assert torch.equal(acc_a.view(M, N).cpu(), (xq.cpu().int() @ w.cpu().int().T))


def test_concat_projections_qkv():
  """q, k, v read the same activations: one weight stream, outputs split afterwards."""
  g = qc.gen(41)
  K, sizes = 1024, [512, 128, 128]
  x = qc.activations(g, 4, K)
  ws = [qc.int8_weight(g, n, K) for n in sizes]
  ss = [qc.per_channel_scale(g, n) for n in sizes]
  w, s, got_sizes = xla_b200.concat_projections([cu(t) for t in ws], [cu(t) for t in ss])
  assert got_sizes == sizes
  y = packed_op(cu(x), w, s)
  for part, wi, si in zip(xla_b200.split_outputs(y, sizes), ws, ss):
    assert qo.max_abs_rel(part, qo.quantized_matmul(x, wi, si, dot_round=None)) < TOL_F32


# ---------------------------------------------------------------------------------------------
# the reference's module-level tests, replayed on the GPU (test/quantized_ops/test_quantized_matmul.py)
# ---------------------------------------------------------------------------------------------


def _cos(a, b):
  a, b = a.flatten().double().cpu(), b.flatten().double().cpu()
  return float(torch.dot(a, b) / (a.norm() * b.norm()))


@pytest.mark.parametrize("quantize_activation", [False, True])
def test_reference_style_q_linear_module_per_channel(quantize_activation):
  # :112-126 -- fp Linear(5, 8) vs the quantized module, atol 0.01
  from xla_b200 import weight_prep as wp
  torch.manual_seed(123456)
  lin = torch.nn.Linear(5, 8, bias=False)
  x = torch.randn(3, 5)
  out_fp = lin(x)
  m = wp.quantize_linear(lin, quantize_activation=quantize_activation).to(DEV)
  out_q = m(x.to(DEV))
  assert torch.allclose(out_fp, out_q.cpu(), atol=0.02 if quantize_activation else 0.01)


@pytest.mark.parametrize("n_bits,block_size,symmetric,qa", [(4, -1, True, False), (8, 2, True, False), (4, 2, True, False),
                                                          (8, -1, False, False), (8, -1, False, True), (4, -1, False, False),
                                                          (8, 2, False, False)])
def test_reference_style_module_variants(n_bits, block_size, symmetric, qa):
  # :182-286 -- int4 per-channel, blockwise, asymmetric per-channel (with and without act-quant), asymmetric blockwise
  from xla_b200 import weight_prep as wp
  torch.manual_seed(123456)
  lin = torch.nn.Linear(6, 8, bias=False)
  x = torch.randn(3, 6)
  out_fp = lin(x)
  m = wp.quantize_linear(lin, n_bits=n_bits, block_size=block_size, symmetric=symmetric, quantize_activation=qa).to(DEV)
  out_q = m(x.to(DEV))
  assert _cos(out_fp, out_q) > (0.99 if n_bits == 8 else 0.95)
  # and against the oracle on the same quantized tensors
  ref = qo.quantized_matmul(x, m.weight.cpu(), m.weight_scaler.cpu(), None if m.zero_point is None else m.zero_point.cpu(),
                            block_size=block_size, quantize_activation=qa)
  assert qo.max_abs_rel(out_q, ref) < 1e-4


def test_torch_compile_default_backend():
  """The module and the two sibling operators under torch.compile with its default backend (the reference compiles
  its module with backend="openxla", test/quantized_ops/test_quantized_matmul.py:128-143): the operators are opaque
  custom ops with Meta kernels, so the compiled graphs call the same kernels and give the same bits."""
  g = qc.gen(31)
  K, N, bs = 1024, 512, 128
  x = cu(qc.activations(g, 4, K))
  m = xla_b200.XlaQuantizedLinear(K, N, is_symmetric=True)
  m.load_quantized_weight(cu(qc.int8_weight(g, N, K)), cu(qc.per_channel_scale(g, N)))
  assert torch.equal(torch.compile(m, fullgraph=True)(x), m(x))

  wp = xla_b200.pack_int4(cu(qc.int4_weight(g, N, K)))
  sb = cu(qc.blockwise_scale(g, K // bs, N))

  def packed(a):
    return torch.ops.xla_b200.quantized_matmul_packed(a, wp, sb, block_size=bs, int4_weight=True, weight_is_packed=True,
                                                      out_dtype=torch.bfloat16) * 2.0
  assert torch.equal(torch.compile(packed, fullgraph=True)(x), packed(x))

  wgu, sgu = xla_b200.interleave_gate_up(xla_b200.pack_int4(cu(qc.int4_weight(g, N, K))), xla_b200.pack_int4(cu(qc.int4_weight(g, N, K))),
                                         cu(qc.blockwise_scale(g, K // bs, N)), cu(qc.blockwise_scale(g, K // bs, N)), bs)

  def gate_up(a):
    return torch.ops.xla_b200.quantized_gate_up(a, wgu, sgu, block_size=bs, int4_weight=True, weight_is_packed=True)
  for xx in (x, cu(qc.activations(g, 48, K))):
    assert torch.equal(torch.compile(gate_up, fullgraph=True)(xx), gate_up(xx))


def test_torch_compile_and_cuda_graph_pass_through():
  # the op is an opaque custom op with a Meta kernel: Dynamo traces it, a CUDA graph captures it (:128-143)
  g = qc.gen(30)
  x = cu(qc.activations(g, 4, 1024))
  w = cu(qc.int8_weight(g, 512, 1024))
  s = cu(qc.per_channel_scale(g, 512))
  m = xla_b200.XlaQuantizedLinear(1024, 512, is_symmetric=True)
  m.load_quantized_weight(w, s)
  eager = m(x)
  compiled = torch.compile(m, backend="aot_eager", fullgraph=True)
  assert torch.equal(compiled(x), eager)
  st = torch.cuda.Stream()
  with torch.cuda.stream(st):
    m(x)
    st.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr, stream=st):
      y = m(x)
    gr.replay()
    st.synchronize()
  assert torch.equal(y, eager)


@pytest.mark.gpu
@pytest.mark.parametrize("packed,block_size", [(True, 128), (True, -1), (False, 128), (False, -1)])
def test_host_pipeline_matches_the_device_op(packed, block_size):
  """Host buffers in, host buffers out through one library call per linear: bit-identical to the device
  operator on the same inputs, for more calls than the pipeline has staging slots and for varying M."""
  import xla_b200
  dev = torch.device("cuda:0")
  g = torch.Generator().manual_seed(11)
  N, K = 1024, 512
  w = torch.randint(-8 if packed else -128, 8 if packed else 128, (N, K), generator=g, dtype=torch.int8)
  sshape = (N,) if block_size == -1 else (K // block_size, N)
  scale = (torch.rand(sshape, generator=g) * 0.04 + 0.01).to(dev)
  wd = w.to(dev)
  if packed:
    wd = xla_b200.pack_int4(wd)
  pipe = xla_b200.HostPipeline(max_M=32, K=K, N=N, depth=3, device=dev)
  lin = pipe.linear(wd, scale, block_size=block_size, weight_is_packed=packed)
  calls = []
  for i, M in enumerate([1, 8, 32, 5, 16, 32, 1, 9]):
    xh = torch.randn(M, K, generator=g).bfloat16().pin_memory()
    yh = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    lin(xh, yh)
    calls.append((xh, yh))
  pipe.synchronize()
  for xh, yh in calls:
    ref = torch.ops.xla_b200.quantized_matmul_packed(xh.to(dev), wd, scale, block_size=block_size, int4_weight=packed,
                                                     weight_is_packed=packed, out_dtype=torch.bfloat16)
    assert torch.equal(ref.cpu(), yh)
  with pytest.raises(Exception):
    lin(torch.zeros(64, K, dtype=torch.bfloat16).pin_memory(), torch.empty(64, N, dtype=torch.bfloat16).pin_memory())
  pipe.close()
