"""Host-buffer front end: activations in (page-locked) host memory in, result in host memory out.

A user of the reference moves the activation to the device, calls ``torch.ops.xla.quantized_matmul``
(torch_xla/experimental/xla_quantized_matmul.py:79-114, :133-170) and reads the result back.  ``HostPipeline``
does that round trip with ONE call into the library per linear: copy-in, kernel and copy-out run on three
streams of the pipeline's own, so the copies of neighbouring calls overlap the kernel, and the Python side
enqueues one call instead of six.

  pipe = HostPipeline(max_M=32, K=4096, N=14336, device="cuda:0")
  lin = pipe.linear(w_packed, scale, block_size=128, weight_is_packed=True)   # weights stay on the device
  lin(x_host, out_host)          # enqueue; returns at once
  pipe.synchronize()             # out_host now holds x_host @ W^T

``linear()`` orders the pipeline after whatever torch's current stream holds at that moment (so a weight packed
just before is complete when the first linear reads it); ``x_host`` must not be modified until ``synchronize()``.
"""
import ctypes

import torch

from . import _capi

LAYOUT_W4_BLOCKWISE_PACKED = 0
LAYOUT_W4_PERCHANNEL_PACKED = 1
LAYOUT_W8_PERCHANNEL = 2
LAYOUT_W8_BLOCKWISE_KMINOR = 3


class HostLinear:
  """One weight bound to a pipeline; calling it enqueues ``out_host = x_host @ W^T`` (see HostPipeline.linear)."""

  def __init__(self, pipe, layout, w, scale, zero_point, N, K, block_size, variant):
    self.pipe, self.layout, self.N, self.K, self.block_size = pipe, layout, N, K, block_size
    self._keep = (w, scale, zero_point)  # the device tensors must outlive the calls
    self._w, self._s = w.data_ptr(), scale.data_ptr()
    self._zp = zero_point.data_ptr() if zero_point is not None else None
    self._variant = variant
    self._fn = _capi.lib().qmm_host_weight_only

  def __call__(self, x_host, out_host):
    assert x_host.device.type == "cpu" and out_host.device.type == "cpu", "HostLinear takes host tensors"
    assert x_host.dim() == 2 and x_host.shape[1] == self.K and x_host.is_contiguous(), (
        f"x_host is expected to be a contiguous [M, {self.K}] tensor, got {list(x_host.shape)}")
    M = x_host.shape[0]
    assert tuple(out_host.shape) == (M, self.N) and out_host.is_contiguous(), (
        f"out_host is expected to be a contiguous [{M}, {self.N}] tensor, got {list(out_host.shape)}")
    _capi.check(self._fn(self.pipe._handle, self.layout, x_host.data_ptr(), _capi.dtype_code(x_host.dtype), self._w, self._s,
                         self._zp, out_host.data_ptr(), _capi.dtype_code(out_host.dtype), M, self.N, self.K, self.block_size,
                         self._variant))
    return out_host


class HostPipeline:
  """Device staging slots, streams and events for host-to-host linears on one GPU (created once, reused)."""

  def __init__(self, max_M, K, N, depth=8, device=None, x_dtype=torch.bfloat16, out_dtype=torch.bfloat16):
    self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    assert self.device.type == "cuda", "HostPipeline needs a CUDA device"
    xb = max_M * K * torch.empty((), dtype=x_dtype).element_size()
    ob = max_M * N * torch.empty((), dtype=out_dtype).element_size()
    handle = ctypes.c_void_p()

    def make():
      _capi.check(_capi.lib().qmm_host_pipeline_create(xb, ob, depth, ctypes.byref(handle)))

    _capi.on_device(self.device, make)
    self._handle = handle.value

  def linear(self, w, scale, zero_point=None, block_size=-1, weight_is_packed=False, variant="auto"):
    """Binds a device-resident K-minor weight: int8 [N,K], or packed int4 uint8 [N,K/2] with
    ``weight_is_packed``; ``scale`` / ``zero_point`` f32 [N] (per channel) or [K/block_size, N] (blockwise)."""
    _capi.require_cuda(w, scale)
    assert w.dim() == 2 and w.is_contiguous(), "the weight is expected K-minor and contiguous"
    N, K = w.shape[0], w.shape[1] * (2 if weight_is_packed else 1)
    blockwise = block_size != -1
    expect = (K // block_size, N) if blockwise else (N,)
    assert tuple(scale.shape) == expect and scale.dtype == torch.float32 and scale.is_contiguous(), (
        f"weight scaler is expected to be a contiguous f32 {list(expect)} tensor, got {scale.dtype} {list(scale.shape)}")
    if zero_point is not None:
      assert tuple(zero_point.shape) == expect and zero_point.dtype == torch.float32 and zero_point.is_contiguous()
    if weight_is_packed:
      assert w.dtype == torch.uint8
      layout = LAYOUT_W4_BLOCKWISE_PACKED if blockwise else LAYOUT_W4_PERCHANNEL_PACKED
    else:
      assert w.dtype == torch.int8
      layout = LAYOUT_W8_BLOCKWISE_KMINOR if blockwise else LAYOUT_W8_PERCHANNEL
    # the weight may still be in the making on torch's current stream (a pack kernel, an upload): the pipeline's
    # kernel stream is private and non-blocking, so it is ordered after that work here, once per binding
    _capi.on_device(self.device, lambda: _capi.check(
        _capi.lib().qmm_host_pipeline_wait_stream(self._handle, _capi.stream_ptr(self.device))))
    return HostLinear(self, layout, w, scale, zero_point, N, K, block_size if blockwise else 0, _capi.VARIANTS[variant])

  def synchronize(self):
    _capi.check(_capi.lib().qmm_host_pipeline_sync(self._handle))

  def close(self):
    if self._handle:
      _capi.check(_capi.lib().qmm_host_pipeline_destroy(self._handle))
      self._handle = None

  def __del__(self):
    try:
      self.close()
    except Exception:
      pass
