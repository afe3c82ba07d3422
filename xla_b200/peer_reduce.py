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


def _create_and_exchange(nbytes, rank, world, group):
  """cudaMalloc's an IPC-shareable buffer on this rank, swaps handles, maps the peers'.  Returns (own, ptrs)."""
  L = _capi.lib()
  own = ctypes.c_void_p()
  handle = ctypes.create_string_buffer(64)
  _capi.check(L.qmm_peer_buffer_create(nbytes, ctypes.byref(own), handle))
  handles = [None] * world
  dist.all_gather_object(handles, bytes(handle.raw), group=group)
  ptrs = []
  for r, h in enumerate(handles):
    if r == rank:
      ptrs.append(own.value)
    else:
      p = ctypes.c_void_p()
      _capi.check(L.qmm_peer_buffer_open(h, ctypes.byref(p)))
      ptrs.append(p.value)
  return own.value, ptrs


class FusedRowParallelDecode:
  """Exchange buffers for ``qmm_rowparallel_decode``: the K-sharded decode linear whose kernel also sums the
  partial results of all ranks (M <= 8).  One instance serves one out_features ``N``; every rank must make the
  same calls in the same order."""

  def __init__(self, N, max_M=8, group=None):
    assert dist.is_initialized()
    self.group, self.N, self.max_M = group, int(N), int(max_M)
    self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
    self.device = torch.device("cuda", torch.cuda.current_device())
    nbytes = _capi.lib().qmm_rowparallel_buffer_bytes(self.max_M, self.N, self.world)
    self._own, self._ptrs = _create_and_exchange(nbytes, self.rank, self.world, group)
    self._arr = (ctypes.c_void_p * self.world)(*self._ptrs)
    dist.barrier(group=group)

  def fits(self, M, N):
    return N == self.N and 1 <= M <= min(self.max_M, 8)

  def __call__(self, x_local, w, scaler, block_size=-1, weight_is_packed=False, out_dtype=torch.float32):
    K = x_local.shape[-1]
    x2 = x_local.reshape(-1, K)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    M = x2.shape[0]
    assert self.fits(M, w.shape[0]), f"M={M}, N={w.shape[0]} do not fit this exchange buffer (N={self.N}, M<={self.max_M})"
    s32 = scaler if scaler.dtype == torch.float32 else scaler.float()
    out = torch.empty((M, self.N), dtype=out_dtype, device=self.device)
    _capi.check(_capi.lib().qmm_rowparallel_decode(
        4 if weight_is_packed else 8, x2.data_ptr(), _capi.dtype_code(x2.dtype), w.data_ptr(), s32.contiguous().data_ptr(),
        out.data_ptr(), _capi.dtype_code(out_dtype), M, self.N, K, 0 if block_size == -1 else block_size, self._arr,
        self.rank, self.world, self.max_M * self.N, _capi.stream_ptr(self.device)))
    return out.reshape(x_local.shape[:-1] + (self.N,))

  def check(self):
    """Raises TimeoutError if a kernel on this device gave up waiting for a peer's tile since the last check (the
    affected outputs are NaN).  Synchronises the current stream; call it wherever a step's results are consumed."""
    _capi.check_device(self.device)

  def close(self):
    if self._own is None:
      return
    torch.cuda.synchronize(self.device)
    word = _capi.device_error(self.device)
    if word:
      import warnings
      warnings.warn(f"xla_b200: a peer exchange on {self.device} gave up a wait (code {word & 0xff}, rank {word >> 8}); "
                    "results of that call were NaN")
    dist.barrier(group=self.group)
    L = _capi.lib()
    for r, p in enumerate(self._ptrs):
      if r != self.rank:
        _capi.check(L.qmm_peer_buffer_close(p))
    dist.barrier(group=self.group)
    _capi.check(L.qmm_peer_buffer_destroy(self._own))
    self._own = None


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

  def check(self):
    """Raises TimeoutError if an exchange on this device gave up waiting for a peer since the last check (the
    affected result is NaN).  Synchronises the current stream; call it wherever a step's results are consumed."""
    _capi.check_device(self.device)

  def close(self):
    """Unmaps the peers' buffers and frees this rank's (collective: every rank must call it)."""
    if self._own is None:
      return
    torch.cuda.synchronize(self.device)
    word = _capi.device_error(self.device)
    if word:
      import warnings
      warnings.warn(f"xla_b200: a peer exchange on {self.device} gave up a wait (code {word & 0xff}, rank {word >> 8}); "
                    "results of that call were NaN")
    dist.barrier(group=self.group)
    L = _capi.lib()
    for r, p in enumerate(self._ptrs):
      if r != self.rank:
        _capi.check(L.qmm_peer_buffer_close(p))
    dist.barrier(group=self.group)
    self._views = None
    _capi.check(L.qmm_peer_buffer_destroy(self._own))
    self._own = None
