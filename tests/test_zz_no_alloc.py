"""The no-allocation entry point, qmm_w8a8_perchannel_static, against qmm_w8a8_perchannel.

Some hosts of this library cannot give it scratch memory: the GPU's memory belongs to their
framework's allocator, or their rules forbid allocating once the service is up.  For them the W8A8
op keeps its scratch in a fixed array inside the library.  This test calls that entry point through
the C ABI, twice in a row on different inputs (the array keeps the first call's contents, which the
second call must not see), and expects bit-identical results to the workspace-taking entry point.

Collected last on purpose (file name), so a failure here cannot hide the other tests' results.
"""
import ctypes

import pytest
import torch

from xla_b200 import _capi

pytestmark = pytest.mark.gpu

STATIC_BYTES = 8 * 1024 * 1024 + 64 * 1024


def _inputs(seed, M, N, K, dev):
  g = torch.Generator().manual_seed(seed)
  x = torch.randn(M, K, generator=g)
  x = torch.where(torch.rand(M, K, generator=g) < 0.01, x * 20.0, x).bfloat16().to(dev)
  w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(dev)
  s = (torch.rand(N, generator=g) * 0.019 + 0.001).to(dev)
  zp = (torch.randint(-8, 9, (N,), generator=g).float()).to(dev) * s
  return x, w, s, zp


def _with_workspace(L, x, w, s, zp, out, M, N, K, variant):
  nbytes = L.qmm_workspace_size(_capi.OP_W8A8_PERCHANNEL, M, N, K)
  ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
  _capi.check(L.qmm_w8a8_perchannel(_capi.ptr(x), _capi.BF16, _capi.ptr(w), _capi.ptr(s), _capi.ptr(zp), _capi.ptr(out),
                                    _capi.F32, M, N, K, 1, variant, _capi.ptr(ws), nbytes, _capi.stream_ptr()))


def _static(L, x, w, s, zp, out, M, N, K, variant):
  return L.qmm_w8a8_perchannel_static(_capi.ptr(x), _capi.BF16, _capi.ptr(w), _capi.ptr(s), _capi.ptr(zp), _capi.ptr(out),
                                      _capi.F32, M, N, K, 1, variant, _capi.stream_ptr())


@pytest.mark.parametrize("variant", [_capi.AUTO, _capi.GENERIC])
def test_static_scratch_matches_workspace_entry_point_twice(variant):
  L = _capi.lib()
  dev = torch.device("cuda", 0)
  with torch.cuda.device(dev):
    # first call: a large shape that fills most of the array; second: a small one with a zero point
    for seed, (M, N, K), use_zp in ((1, (1024, 512, 4096), False), (2, (48, 264, 272), True)):
      x, w, s, zp = _inputs(seed, M, N, K, dev)
      zp = zp if use_zp else None
      ref = torch.empty((M, N), dtype=torch.float32, device=dev)
      got = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
      _with_workspace(L, x, w, s, zp, ref, M, N, K, variant)
      _capi.check(_static(L, x, w, s, zp, got, M, N, K, variant))
      torch.cuda.synchronize()
      assert torch.equal(got, ref), f"static-scratch result differs for shape {(M, N, K)}"


def test_static_scratch_refuses_oversized_shapes_and_takes_the_largest_that_fits():
  L = _capi.lib()
  dev = torch.device("cuda", 0)
  with torch.cuda.device(dev):
    # 2048 x 4096 activations (the W8A8 prefill configuration) is the documented size that fits
    assert L.qmm_workspace_size(_capi.OP_W8A8_PERCHANNEL, 2048, 64, 4096) <= STATIC_BYTES
    x, w, s, _ = _inputs(3, 2048, 64, 4096, dev)
    ref = torch.empty((2048, 64), dtype=torch.float32, device=dev)
    got = torch.empty_like(ref)
    _with_workspace(L, x, w, s, None, ref, 2048, 64, 4096, _capi.AUTO)
    _capi.check(_static(L, x, w, s, None, got, 2048, 64, 4096, _capi.AUTO))
    torch.cuda.synchronize()
    assert torch.equal(got, ref)
    # one row more does not fit: refused with a status and a message, nothing launched
    assert L.qmm_workspace_size(_capi.OP_W8A8_PERCHANNEL, 2100, 64, 4096) > STATIC_BYTES
    rc = L.qmm_w8a8_perchannel_static(None, _capi.BF16, None, None, None, None, _capi.F32, 2100, 64, 4096, 1, 0, None)
    assert rc == 5
    msg = L.qmm_last_error_string().decode()
    assert "built-in" in msg and "qmm_w8a8_perchannel" in msg
    # empty problems succeed without touching the GPU
    assert L.qmm_w8a8_perchannel_static(None, _capi.BF16, None, None, None, None, _capi.F32, 0, 64, 4096, 1, 0, None) == 0
