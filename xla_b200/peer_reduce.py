"""One-shot all-reduce over peer memory for the row-parallel quantized linear (GPUs of one box).

Each rank keeps the fp32 partial result of its K slice in a buffer that the other ranks map through CUDA
IPC; one kernel per GPU signals, waits (bounded) and sums the G partials in rank order
(``qmm_allreduce_oneshot``, xla_b200/csrc/peer_reduce.cu).  For decode-sized results (a few KB) this replaces
the latency of a library all-reduce; large results should stay on NCCL (``max_elems`` bounds what goes here).

The reference has no collective attached to the quantized linear (under SPMD, XLA inserts the all-reduce:
torch_xla/csrc/cross_replica_reduces.cpp:154).
"""
import ctypes

import torch
import torch.distributed as dist

from . import _capi


class _Span:
  """Device memory span exposed through the CUDA array interface (zero-copy view for torch.as_tensor)."""

  def __init__(self, ptr, n_floats):
    self.__cuda_array_interface__ = {"shape": (n_floats,), "typestr": "<f4", "data": (ptr, False), "version": 3,
                                     "strides": None}


class PeerAllReduce:
  """Peer-mapped partial-result buffers of one process group (one process per GPU, same box).

  ``partial_view(M, N)`` is where the next call's fp32 partial goes; ``reduce(M, N, out_dtype)`` then returns
  the sum over ranks.  Every rank must make the same calls in the same order.
  """

  FLAG_BYTES = 256

  def __init__(self, max_elems, group=None):
    assert dist.is_initialized(), "PeerAllReduce needs an initialised process group"
    self.group = group
    self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
    assert self.world <= 8, "at most 8 ranks"
    self.max_elems = (int(max_elems) + 3) // 4 * 4
    self.device = torch.device("cuda", torch.cuda.current_device())
    L = _capi.lib()
    self._slot_bytes = self.max_elems * 4
    nbytes = 2 * self._slot_bytes + self.FLAG_BYTES
    own = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    _capi.check(L.qmm_peer_buffer_create(nbytes, ctypes.byref(own), handle))
    self._own = own.value
    handles = [None] * self.world
    dist.all_gather_object(handles, bytes(handle.raw), group=group)
    self._ptrs = []
    for r, h in enumerate(handles):
      if r == self.rank:
        self._ptrs.append(self._own)
      else:
        p = ctypes.c_void_p()
        _capi.check(L.qmm_peer_buffer_open(h, ctypes.byref(p)))
        self._ptrs.append(p.value)
    arr = ctypes.c_void_p * self.world
    self._data = [arr(*[p + s * self._slot_bytes for p in self._ptrs]) for s in range(2)]
    self._flags = arr(*[p + 2 * self._slot_bytes for p in self._ptrs])
    self._views = [torch.as_tensor(_Span(self._own + s * self._slot_bytes, self.max_elems), device=self.device)
                   for s in range(2)]
    self.epoch = 0
    dist.barrier(group=group)  # every rank has mapped every buffer before anyone signals

  def partial_view(self, M, N):
    """fp32 [M, N] view of the slot the NEXT reduce() reads on this rank."""
    n = M * N
    assert n <= self.max_elems, f"{M}x{N} exceeds the peer buffer ({self.max_elems} elements)"
    return self._views[(self.epoch + 1) % 2][:n].view(M, N)

  def fits(self, M, N):
    return M * N <= self.max_elems and (M * N) % 4 == 0

  def reduce(self, M, N, out_dtype):
    self.epoch += 1
    out = torch.empty((M, N), dtype=out_dtype, device=self.device)
    # epoch 0: the kernel keeps the call number in device memory, so a launch captured in a CUDA graph stays
    # valid on replay (capture an even number of calls per graph: the two data slots must keep alternating)
    _capi.check(_capi.lib().qmm_allreduce_oneshot(self._data[self.epoch % 2], self._flags, self.rank, self.world, 0,
                                                  out.data_ptr(), _capi.dtype_code(out_dtype), M * N,
                                                  _capi.stream_ptr(self.device)))
    return out

  def close(self):
    """Unmaps the peers' buffers and frees this rank's (collective: every rank must call it)."""
    if self._own is None:
      return
    torch.cuda.synchronize(self.device)
    dist.barrier(group=self.group)
    L = _capi.lib()
    for r, p in enumerate(self._ptrs):
      if r != self.rank:
        _capi.check(L.qmm_peer_buffer_close(p))
    dist.barrier(group=self.group)
    self._views = None
    _capi.check(L.qmm_peer_buffer_destroy(self._own))
    self._own = None
