"""ctypes binding of libqmm_b200.so (the C ABI declared in include/qmm_b200.h).

The library is loaded from ``xla_b200/lib``; if it is missing, importing this module fails with a
message that says how to build it.  There is no fallback implementation.
"""
import ctypes
import os

import torch

from . import _build

F32, BF16, F16 = 0, 1, 2
AUTO, GENERIC, GEMV, TCGEN05, MMA, I8TC = 0, 1, 2, 3, 4, 6
OP_W8A16_PERCHANNEL, OP_BLOCKWISE_SBN, OP_W4A16_BLOCKWISE_PACKED, OP_W8A8_PERCHANNEL, OP_W4A16_PERCHANNEL_PACKED = range(5)

VARIANTS = {"auto": AUTO, "generic": GENERIC, "gemv": GEMV, "tcgen05": TCGEN05, "mma": MMA, "i8tc": I8TC}

_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_STATUS_EXC = {1: AssertionError, 2: NotImplementedError, 3: ValueError, 5: ValueError, 6: ValueError}

# name -> (restype, argtypes); every symbol include/qmm_b200.h declares
_p, _i, _i64, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
SIGNATURES = {
    "qmm_abi_version": (_i, []),
    "qmm_status_string": (ctypes.c_char_p, [_i]),
    "qmm_last_error_string": (ctypes.c_char_p, []),
    "qmm_w8a16_perchannel": (_i, [_p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i, _p]),
    "qmm_w4a16_perchannel_packed": (_i, [_p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i, _p]),
    "qmm_w8a16_blockwise": (_i, [_p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _i, _p]),
    "qmm_weight_only_workspace_size": (_sz, [_i64, _i64]),
    "qmm_weight_only_workspace_size_for": (_sz, [ctypes.c_int, _i64, _i64, _i64]),
    "qmm_tuned_variant": (_i, [_i, _i64, _i64, _i64, _i64]),
    "qmm_weight_only_variant_for": (ctypes.c_char_p, [_i, _i64, _i64, _i64, _i64, _i]),
    "qmm_weight_only": (_i, [_i, _p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _i, _p, _sz, _p]),
    "qmm_host_pipeline_create": (_i, [_sz, _sz, _i, ctypes.POINTER(ctypes.c_void_p)]),
    "qmm_host_weight_only": (_i, [_p, _i, _p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _i]),
    "qmm_host_pipeline_wait_stream": (_i, [_p, _p]),
    "qmm_host_pipeline_sync": (_i, [_p]),
    "qmm_host_pipeline_destroy": (_i, [_p]),
    "qmm_peer_buffer_create": (_i, [_sz, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]),
    "qmm_peer_buffer_open": (_i, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "qmm_peer_buffer_close": (_i, [_p]),
    "qmm_peer_buffer_destroy": (_i, [_p]),
    "qmm_allreduce_oneshot": (_i, [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), _i, _i, ctypes.c_uint32,
                                  _p, _i, _i64, _p]),
    "qmm_rowparallel_buffer_bytes": (_sz, [_i64, _i64, _i]),
    "qmm_rowparallel_decode": (_i, [_i, _p, _i, _p, _p, _p, _i, _i64, _i64, _i64, _i64, ctypes.POINTER(ctypes.c_void_p), _i, _i,
                                   _i64, _p]),
    "qmm_gate_up_decode": (_i, [_i, _p, _i, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _p]),
    "qmm_blockwise_sbn": (_i, [_p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _i, _p]),
    "qmm_w4a16_blockwise_packed": (_i, [_p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i64, _i, _p]),
    "qmm_quantize_activation": (_i, [_p, _i, _p, _p, _p, _i64, _i64, _i, _p]),
    "qmm_w8a8_gemm": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i, _p]),
    "qmm_w8a8_perchannel": (_i, [_p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i, _i, _p, _sz, _p]),
    "qmm_w8a8_perchannel_static": (_i, [_p, _i, _p, _p, _p, _p, _i, _i64, _i64, _i64, _i, _i, _p]),
    "qmm_workspace_size": (_sz, [_i, _i64, _i64, _i64]),
    "qmm_pack_int4_nk": (_i, [_p, _p, _i64, _i64, _p]),
    "qmm_pack_int4_sbn": (_i, [_p, _p, _i64, _i64, _i64, _p]),
    "qmm_unpack_int4_nk": (_i, [_p, _p, _i64, _i64, _p]),
    "qmm_device_error_flag": (_i, [_p, _p]),
    "qmm_gate_up": (_i, [ctypes.c_int, _p, ctypes.c_int, _p, _p, _p, ctypes.c_int, _i64, _i64, _i64, _i64, _p, _sz, _p]),
    "qmm_set_peer_wait_limit": (_i, [ctypes.c_double]),
    "qmm_set_activation_limbs": (_i, [ctypes.c_int]),
    "qmm_stream_read": (_i, [_p, _sz, _p, _p]),
    "qmm_variant_for": (ctypes.c_char_p, [_i, _i64, _i64, _i64, _i64, _i]),
}

_lib = None


def lib_path():
  return _build.LIB_PATH


def lib():
  """The loaded library; raises if it has not been built."""
  global _lib
  if _lib is None:
    path = lib_path()
    if not os.path.exists(path):
      raise ImportError(
          f"{path} is missing: build it with `python -m xla_b200._build` (needs nvcc). "
          "xla_b200 has no CPU or PyTorch fallback for its kernels.")
    L = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
      fn = getattr(L, name)
      fn.restype, fn.argtypes = res, args
    _lib = L
  return _lib


def dtype_code(dt):
  try:
    return _DTYPES[dt]
  except KeyError:
    raise TypeError(f"xla_b200: unsupported floating dtype {dt}") from None


def ptr(t):
  """Device address as a plain int (ctypes converts it for a void* parameter); None stays None."""
  return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device=None):
  """Handle of torch's current stream on `device` (an int usable as cudaStream_t)."""
  if _raw_stream is not None:
    if device is None:
      idx = None
    elif isinstance(device, int):
      idx = device
    else:
      idx = torch.device(device).index  # accepts torch.device and strings like "cuda:0"
    return _raw_stream(torch.cuda.current_device() if idx is None else idx)
  return torch.cuda.current_stream(device).cuda_stream


def on_device(device, fn):
  """Runs fn() with `device` current; skips the context switch when it already is."""
  if device.index is None or device.index == torch.cuda.current_device():
    return fn()
  with torch.cuda.device(device):
    return fn()


_workspaces = {}


def workspace(device, max_M, K, N=0, wbits=8):
  """Scratch for ``qmm_weight_only`` on torch's current stream of `device`: (pointer, bytes), or (None, 0) when no
  variant needs one; with N and wbits, including the room that lets a long int4 batch expand its weights to int8
  once.  One buffer per (device, stream), zero-filled when created (the kernels keep its flag words
  zero) and grown on demand; a stream capture in progress never allocates - it gets the existing buffer or none."""
  need = lib().qmm_weight_only_workspace_size_for(wbits, max_M, N, K) if N else lib().qmm_weight_only_workspace_size(max_M, K)
  if need == 0:
    return None, 0
  idx = device.index if device.index is not None else torch.cuda.current_device()
  key = (idx, stream_ptr(idx))
  buf = _workspaces.get(key)
  if buf is None or buf.numel() < need:
    if torch.cuda.is_current_stream_capturing():
      return (None, 0) if buf is None else (buf.data_ptr(), buf.numel())
    size = max(need, 16 << 20) if buf is None else max(need, 2 * buf.numel())
    buf = torch.zeros(size, dtype=torch.uint8, device=torch.device("cuda", idx))
    _workspaces[key] = buf
  return buf.data_ptr(), buf.numel()


def check(status):
  """Turns a non-zero qmm_status into the Python exception the reference would raise."""
  if status == 0:
    return
  L = lib()
  msg = L.qmm_last_error_string().decode() or L.qmm_status_string(status).decode()
  raise _STATUS_EXC.get(status, RuntimeError)(f"qmm_b200[{L.qmm_status_string(status).decode()}]: {msg}")


def device_error(device=None):
  """Reads and clears the device error word of `device` (synchronises torch's current stream there); returns the
  raw word, 0 when healthy.  Bits 0-7: which bounded wait gave up, bits 8 and up: the CTA or the peer rank."""
  dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
  word = ctypes.c_uint32(0)

  def read():
    lib().qmm_device_error_flag(ctypes.byref(word), stream_ptr(dev))

  on_device(dev, read)
  return word.value


def check_device(device=None):
  """Raises TimeoutError if a kernel on `device` gave up a bounded wait since the last check."""
  word = device_error(device)
  if word:
    raise TimeoutError(f"qmm_b200: a device-side wait gave up (code {word & 0xff}, unit {word >> 8}); results of the "
                       "affected call are NaN or undefined")


def require_cuda(*tensors):
  for t in tensors:
    if t is not None and not t.is_cuda:
      raise RuntimeError("xla_b200 kernels run on CUDA tensors only; there is no CPU path "
                         f"(got a tensor on {t.device})")
