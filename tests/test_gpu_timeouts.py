"""The bounded device-side waits, made to run out on purpose - on the host's terms: a flag word that nothing ever
sets and a wait limit of a few milliseconds.  The kernel must return, fill its result with NaN, leave the code of the
wait in the device error word, and the context must stay usable.  Nothing here faults or hangs a GPU.

The waits are the ones of the two kernels that wait for another GPU (one-shot all-reduce over peer memory, row-parallel
decode with the exchange in its epilogue); on one GPU the "peer" is a second buffer of the same device whose flag
stays zero.
"""
import ctypes

import pytest
import torch

import xla_b200
from tests import qmm_cases as qc
from xla_b200 import _capi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture
def short_wait():
  L = _capi.lib()
  assert _capi.device_error(DEV) == 0, "the device error word was set before this test"
  _capi.check(L.qmm_set_peer_wait_limit(0.005))
  yield L
  _capi.check(L.qmm_set_peer_wait_limit(1.0))
  _capi.device_error(DEV)  # leave the word clear for whoever runs next


def _ptr_array(tensors):
  return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def test_allreduce_gives_up_when_a_peer_never_signals(short_wait):
  L = short_wait
  n = 4096
  data = [torch.ones(n, device=DEV), torch.ones(n, device=DEV)]
  flags = [torch.zeros(16, dtype=torch.int32, device=DEV) for _ in range(2)]
  out = torch.zeros(n, device=DEV)
  with torch.cuda.device(0):
    rc = L.qmm_allreduce_oneshot(_ptr_array(data), _ptr_array(flags), 0, 2, 1, out.data_ptr(), _capi.F32, n,
                                 _capi.stream_ptr(DEV))
  assert rc == 0
  torch.cuda.synchronize()           # returns: the wait was bounded
  assert torch.isnan(out).all()      # not stale memory
  word = ctypes.c_uint32(0)
  with torch.cuda.device(0):
    rc = L.qmm_device_error_flag(ctypes.byref(word), _capi.stream_ptr(DEV))
  assert rc == 8, "QMM_ERR_TIMEOUT"
  assert word.value & 0xff == 7 and word.value >> 8 == 1, hex(word.value)   # all-reduce wait, peer rank 1
  assert _capi.device_error(DEV) == 0                                      # reading cleared it
  # the context is alive and the same call works once the "peer" has signalled (its flag word for this epoch)
  flags[0][1] = 2
  with torch.cuda.device(0):
    _capi.check(L.qmm_allreduce_oneshot(_ptr_array(data), _ptr_array(flags), 0, 2, 2, out.data_ptr(), _capi.F32, n,
                                        _capi.stream_ptr(DEV)))
  torch.cuda.synchronize()
  assert torch.all(out == 2.0)
  with pytest.raises(TimeoutError):
    flags[0][1] = 0
    with torch.cuda.device(0):
      L.qmm_allreduce_oneshot(_ptr_array(data), _ptr_array(flags), 0, 2, 3, out.data_ptr(), _capi.F32, n, _capi.stream_ptr(DEV))
    _capi.check_device(DEV)


def test_fused_rowparallel_decode_gives_up_when_a_peer_never_signals(short_wait):
  L = short_wait
  g = qc.gen(9)
  M, N, K = 2, 256, 512
  x = qc.activations(g, M, K).to(DEV)
  w = qc.int8_weight(g, N, K).to(DEV)
  s = qc.per_channel_scale(g, N).to(DEV)
  nbytes = L.qmm_rowparallel_buffer_bytes(8, N, 2)
  bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(2)]
  out = torch.zeros(M, N, device=DEV)
  with torch.cuda.device(0):
    rc = L.qmm_rowparallel_decode(8, x.data_ptr(), _capi.BF16, w.data_ptr(), s.data_ptr(), out.data_ptr(), _capi.F32, M, N, K, 0,
                                  _ptr_array(bufs), 0, 2, 8 * N, _capi.stream_ptr(DEV))
  assert rc == 0
  torch.cuda.synchronize()
  assert torch.isnan(out).all()
  word = _capi.device_error(DEV)
  assert word & 0xff == 8 and word >> 8 == 1, hex(word)   # fused exchange wait, peer rank 1
  # the library still works on this device
  y = torch.ops.xla.quantized_matmul(x, w, s)
  assert torch.isfinite(y).all()
