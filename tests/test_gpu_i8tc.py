"""GPU parity of the split-activation tensor-core kernel (variant "i8tc": unconverted int8/int4 weights into
tcgen05.mma.kind::i8, stream-K over all SMs) against the CPU oracle, through the operators and the C ABI.

The kernel's integer sums are exact and its fixed-point activations are exact for values within 2^-14 of the row
maximum, so fp32 outputs are held to 1e-4 (max|a-b| / max|b|) against the exact value of the formula and 16-bit
outputs to 1e-2, the tolerances of the other weight-only kernels.  Above 32 tokens a 16-bit output takes the two-limb
form of the activations (15 bits below the row maximum: with 1 % of the entries 20 times larger than the rest the
error is ~1e-3 of the output's scale); it is held to 3e-3 through f16 outputs.
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
TOL_TWO_LIMBS = 3e-3


def packed_op(*args, variant="i8tc", **kw):
  with xla_b200.force_variant(variant):
    return torch.ops.xla_b200.quantized_matmul_packed(*args, **kw)


def _exact(x, w_nk, s, bs):
  if bs > 0:
    return qo.quantized_matmul(x.float(), qc.to_sbn(w_nk, bs), s, block_size=bs, dot_round=None)
  return qo.quantized_matmul(x.float(), w_nk, s, dot_round=None)


def _run(x, w_nk, s, bs, wbits, out_dtype):
  wd = w_nk.to(DEV)
  if wbits == 4:
    wd = xla_b200.pack_int4(wd)
  return packed_op(x.to(DEV), wd, s.to(DEV), block_size=bs if bs > 0 else -1, int4_weight=wbits == 4,
                   weight_is_packed=wbits == 4, out_dtype=out_dtype)


# every token-count class of the kernel (limb columns 16, 32, 48, 96, one and two 42-token tiles) and the edges of each
@pytest.mark.parametrize("M", [1, 2, 5, 6, 10, 11, 16, 17, 32, 33, 42, 43, 64])
@pytest.mark.parametrize("wbits,bs", [(8, 0), (8, 128), (4, 128), (4, 0)])
def test_token_classes(M, wbits, bs):
  g = qc.gen(100 + M)
  N, K = 1536, 2048
  x = qc.activations(g, M, K)
  w = qc.int4_weight(g, N, K) if wbits == 4 else qc.int8_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N) if bs > 0 else qc.per_channel_scale(g, N)
  exact = _exact(x, w, s, bs)
  out = _run(x, w, s, bs, wbits, torch.float32)
  assert out.dtype == torch.float32 and tuple(out.shape) == (M, N)
  assert qo.max_abs_rel(out, exact) < TOL_F32
  out16 = _run(x, w, s, bs, wbits, torch.bfloat16)
  assert qo.max_abs_rel(out16, exact) < TOL_BF16


# ragged N (last tile partly empty), K tails (not a multiple of the 128-value stage), few tiles with a long K
# (every tile is shared by many CTAs), many tiles with a short K
@pytest.mark.parametrize("N,K,wbits,bs", [
    (1000, 4096, 8, 0), (1000, 4096 + 16, 8, 0), (130, 8192, 8, 0), (3001, 256, 8, 128), (256, 28672, 4, 128),
    (1000, 4096 + 32, 4, 0), (1111, 4096 + 96, 4, 0), (8192, 128, 8, 128), (77, 1024, 4, 256), (512, 3072, 8, 512),
    (640, 2304, 4, 128),
])
@pytest.mark.parametrize("M", [3, 24])
def test_ragged_shapes(N, K, wbits, bs, M):
  g = qc.gen(N + K + M)
  x = qc.activations(g, M, K)
  w = qc.int4_weight(g, N, K) if wbits == 4 else qc.int8_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N) if bs > 0 else qc.per_channel_scale(g, N)
  out = _run(x, w, s, bs, wbits, torch.float32)
  assert qo.max_abs_rel(out, _exact(x, w, s, bs)) < TOL_F32


# larger batches run as (weight tile, token tile) items with 42 tokens per tile; 1008 tokens per launch
@pytest.mark.parametrize("M", [65, 84, 85, 126, 127, 300, 512, 1008, 1009, 1100])
@pytest.mark.parametrize("wbits,bs", [(8, 0), (4, 128), (8, 128), (4, 0), (8, 512)])
def test_large_batches(M, wbits, bs):
  g = qc.gen(300 + M)
  N, K = 900, 1536
  x = qc.activations(g, M, K, outliers=True)
  w = qc.int4_weight(g, N, K) if wbits == 4 else qc.int8_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N) if bs > 0 else qc.per_channel_scale(g, N)
  exact = _exact(x, w, s, bs)
  out = _run(x, w, s, bs, wbits, torch.float32)
  assert tuple(out.shape) == (M, N)
  assert qo.max_abs_rel(out, exact) < TOL_F32
  if M in (127, 512):
    out16 = _run(x, w, s, bs, wbits, torch.bfloat16)
    assert qo.max_abs_rel(out16, exact) < TOL_BF16


# 16-bit outputs above 32 tokens: two limbs per token, 64 tokens per tile; stream-K up to 64 tokens, items above,
# chunks of 1024 tokens
@pytest.mark.parametrize("M", [33, 63, 64, 65, 128, 129, 300, 1024, 1025, 1100])
@pytest.mark.parametrize("wbits,bs", [(8, 0), (4, 128), (8, 128), (4, 0), (4, 256)])
def test_two_limb_batches(M, wbits, bs):
  g = qc.gen(500 + M)
  N, K = 900, 1536
  x = qc.activations(g, M, K, outliers=True)
  x[M // 2] *= 1e-3
  x[M - 1, 5] = 127.5  # a largest value just under a power of two (mantissa all ones): the narrower scaling
  w = qc.int4_weight(g, N, K) if wbits == 4 else qc.int8_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N) if bs > 0 else qc.per_channel_scale(g, N)
  exact = _exact(x, w, s, bs)
  out = _run(x, w, s, bs, wbits, torch.float16).cpu()
  assert out.dtype == torch.float16 and tuple(out.shape) == (M, N)
  for m in {0, M // 2, M - 1, min(M - 1, 63), min(M - 1, 64)}:
    assert qo.max_abs_rel(out[m], exact[m]) < TOL_TWO_LIMBS, m
  assert qo.max_abs_rel(out, exact) < TOL_TWO_LIMBS
  out16 = _run(x, w, s, bs, wbits, torch.bfloat16)
  assert qo.max_abs_rel(out16, exact) < TOL_BF16


def test_two_limb_stream_k_is_deterministic():
  g = qc.gen(12)
  M, N, K = 64, 384, 8192   # three weight tiles over all SMs: every tile is summed from many partial tiles
  x, w, s = qc.activations(g, M, K), qc.int8_weight(g, N, K), qc.blockwise_scale(g, K // 128, N)
  outs = [_run(x, w, s, 128, 8, torch.bfloat16) for _ in range(10)]
  for o in outs[1:]:
    assert torch.equal(o, outs[0])
  assert qo.max_abs_rel(outs[0], _exact(x, w, s, 128)) < TOL_BF16


def _abi_int4(x, wp, s, bs, out_dtype, ws_bytes):
  """qmm_weight_only(4, ...) through the C ABI with a zeroed workspace of exactly ws_bytes."""
  from xla_b200 import _capi
  L = _capi.lib()
  M, K = x.shape
  N = wp.shape[0]
  out = torch.empty((M, N), dtype=out_dtype, device=DEV)
  ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
  with torch.cuda.device(0):
    _capi.check(L.qmm_weight_only(4, _capi.ptr(x), _capi.dtype_code(x.dtype), _capi.ptr(wp), _capi.ptr(s), None, _capi.ptr(out),
                                  _capi.dtype_code(out_dtype), M, N, K, bs, _capi.VARIANTS["i8tc"], _capi.ptr(ws), ws_bytes,
                                  _capi.stream_ptr()))
    torch.cuda.synchronize()
  return out


# long int4 batches (384 tokens per channel, 512 with scale blocks): the weights are expanded to int8 once when the
# workspace has room (all of them, or slices of rows), per tile inside the kernel otherwise; the three routes add the
# same integers in the same order
@pytest.mark.parametrize("M,out_dtype", [(400, torch.float32), (512, torch.bfloat16), (800, torch.bfloat16), (1100, torch.bfloat16),
                                         (1100, torch.float32)])
@pytest.mark.parametrize("bs", [0, 128])
def test_int4_widened_once_matches_in_kernel_expansion(M, out_dtype, bs):
  from xla_b200 import _capi
  L = _capi.lib()
  g = qc.gen(700 + M)
  N, K = 9000, 512
  x = qc.activations(g, M, K, outliers=True).to(DEV)
  w = qc.int4_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N) if bs > 0 else qc.per_channel_scale(g, N)
  wp = xla_b200.pack_int4(w.to(DEV))
  sd = s.to(DEV)
  base = L.qmm_weight_only_workspace_size(M, K)
  full = L.qmm_weight_only_workspace_size_for(4, M, N, K)
  assert full >= base + N * K
  direct = _abi_int4(x, wp, sd, bs, out_dtype, base)
  whole = _abi_int4(x, wp, sd, bs, out_dtype, full)
  sliced = _abi_int4(x, wp, sd, bs, out_dtype, base + 256 + 7168 * K)
  assert torch.equal(whole, direct) and torch.equal(sliced, direct)
  tol = TOL_F32 if out_dtype == torch.float32 else TOL_BF16
  assert qo.max_abs_rel(direct, _exact(x.cpu(), w, s, bs)) < tol


# 160 items (20 weight tiles x 8 token tiles) on 148 SMs: the partly filled second round is avoided by dealing the
# (item, K unit) space in equal shares; items that span two CTAs go through the partial-tile exchange
@pytest.mark.parametrize("bs", [128, 0])
def test_items_dealt_in_equal_shares(bs):
  from xla_b200 import _capi
  g = qc.gen(900 + bs)
  M, N, K = 512, 2560, 8192
  x = qc.activations(g, M, K, outliers=True)
  w = qc.int4_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N) if bs > 0 else qc.per_channel_scale(g, N)
  wp = xla_b200.pack_int4(w.to(DEV))
  base = _capi.lib().qmm_weight_only_workspace_size(M, K)   # no room to widen: the int4 instance runs
  outs = [_abi_int4(x.to(DEV), wp, s.to(DEV), bs, torch.bfloat16, base) for _ in range(3)]
  assert torch.equal(outs[1], outs[0]) and torch.equal(outs[2], outs[0])
  rows = torch.cat([torch.arange(0, 6), torch.arange(60, 70), torch.arange(250, 260), torch.arange(505, 512)])
  exact = _exact(x[rows], w, s, bs)
  assert qo.max_abs_rel(outs[0][rows], exact) < TOL_BF16
  out32 = _abi_int4(x.to(DEV), wp, s.to(DEV), bs, torch.float32, base)   # three limbs: 13 token tiles
  assert qo.max_abs_rel(out32[rows], exact) < TOL_F32


# one 64-token tile over more weight tiles than SMs: a round of whole tiles, the rest split along K
@pytest.mark.parametrize("K", [1024, 8192])
def test_single_wide_tile_over_many_weight_tiles(K):
  g = qc.gen(950 + K)
  M, N, bs = 64, 20000, 128
  x = qc.activations(g, M, K)
  w = qc.int4_weight(g, N, K)
  s = qc.blockwise_scale(g, K // bs, N)
  outs = [_run(x, w, s, bs, 4, torch.bfloat16) for _ in range(3)]
  assert torch.equal(outs[1], outs[0]) and torch.equal(outs[2], outs[0])
  rows = torch.tensor([0, 1, 31, 32, 62, 63])
  assert qo.max_abs_rel(outs[0][rows], _exact(x[rows], w, s, bs)) < TOL_BF16


@pytest.mark.parametrize("xdt", [torch.float32, torch.float16, torch.bfloat16])
def test_activation_dtypes_and_ranges(xdt):
  g = qc.gen(7)
  M, N, K = 8, 512, 1024
  x = qc.activations(g, M, K, dtype=torch.float32, outliers=True)
  x[1] *= 1e-3   # rows of very different magnitude: the exponent is per row
  x[2] *= 250.0
  x[3] = 0.0     # an all-zero row
  x[4, ::2] = 0.0
  x = x.to(xdt)
  w = qc.int8_weight(g, N, K)
  s = qc.per_channel_scale(g, N)
  exact = _exact(x, w, s, 0)
  out = _run(x, w, s, 0, 8, torch.float32).cpu()
  assert torch.all(out[3] == 0)
  for m in range(M):
    if m != 3:
      assert qo.max_abs_rel(out[m], exact[m]) < TOL_F32, m


def test_largest_int8_products_do_not_overflow():
  # every limb of row 0 at -128 (top limb -63) against weights of -127 over the longest supported accumulation
  M, N, K = 2, 128, 65536
  X = -(63 * 65536 + 128 * 256 + 128)
  x = torch.full((M, K), X * 2.0 ** -21, dtype=torch.float32)  # exact in fp32, exponent 0
  x[1, ::2] = 255.0 / 256.0
  w = torch.full((N, K), -127, dtype=torch.int8)
  w[:, 1::2] = 127
  w[0] = -127
  s = torch.ones(N)
  out = _run(x, w, s, 0, 8, torch.float32)
  assert qo.max_abs_rel(out, _exact(x, w, s, 0)) < 1e-6


def test_deterministic_and_workspace_left_clean():
  g = qc.gen(11)
  M, N, K = 16, 384, 8192   # three tiles over all SMs: every tile is summed from many partial tiles
  x, w, s = qc.activations(g, M, K), qc.int8_weight(g, N, K), qc.per_channel_scale(g, N)
  # (other work between the runs shifts the timing of the partial tiles; the sums must not depend on when they land)
  outs = []
  for i in range(30):
    outs.append(_run(x, w, s, 0, 8, torch.float32))
    if i % 3 == 0:
      torch.zeros(1 << 22, device=DEV).sum()
  for o in outs[1:]:
    assert torch.equal(o, outs[0])
  assert qo.max_abs_rel(outs[0], _exact(x, w, s, 0)) < TOL_F32


def test_auto_picks_it_and_reference_op_reaches_it():
  from xla_b200 import _capi
  g = qc.gen(3)
  M, N, K = 16, 4096, 4096   # the W8A16 per-channel configuration
  x, w, s = qc.activations(g, M, K), qc.int8_weight(g, N, K), qc.per_channel_scale(g, N)
  out = torch.ops.xla.quantized_matmul(x.to(DEV), w.to(DEV), s.to(DEV))
  assert out.dtype == torch.float32
  assert qo.max_abs_rel(out, _exact(x, w, s, 0)) < TOL_F32
  assert _capi.lib().qmm_weight_only_workspace_size(16, 4096) > 0
