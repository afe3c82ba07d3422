"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from xla_b200 import _build, _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
  text = open(os.path.join(ROOT, "include", "qmm_b200.h")).read()
  return sorted(set(re.findall(r"QMM_API\s+[\w\s\*]+?\b(qmm_\w+)\s*\(", text)))


def test_library_is_built_in_tree():
  assert os.path.exists(_build.LIB_PATH), "run `python -m xla_b200._build`"
  assert _build.LIB_PATH.startswith(ROOT)


def test_every_declared_symbol_is_exported_and_bound():
  names = declared_symbols()
  assert len(names) >= 16
  L = ctypes.CDLL(_build.LIB_PATH)
  for n in names:
    assert hasattr(L, n), f"{n} declared in include/qmm_b200.h but not exported"
  assert set(names) == set(_capi.SIGNATURES), "ctypes table and header disagree"


def test_version_and_status_strings():
  L = _capi.lib()
  assert L.qmm_abi_version() == 1
  assert L.qmm_status_string(0) == b"ok"
  assert L.qmm_status_string(2) == b"unsupported"
  assert L.qmm_status_string(99) == b"unknown status"


def test_argument_errors_need_no_gpu():
  L = _capi.lib()
  # negative dimension
  assert L.qmm_w8a16_perchannel(None, 1, None, None, None, None, 1, -1, 4, 4, 0, None) == 1
  assert b"negative" in L.qmm_last_error_string()
  # bad dtype code
  assert L.qmm_w8a16_perchannel(None, 7, None, None, None, None, 1, 1, 4, 4, 0, None) == 2
  # NULL output with work to do
  assert L.qmm_w8a16_perchannel(None, 1, None, None, None, None, 1, 1, 4, 4, 0, None) == 6
  # empty problem is a no-op success
  assert L.qmm_w8a16_perchannel(None, 1, None, None, None, None, 1, 0, 4, 4, 0, None) == 0
  # block size must divide K
  assert L.qmm_blockwise_sbn(None, 1, None, None, None, None, 1, 0, 4, 6, 4, 0, None) == 1
  assert b"divisible by block_size" in L.qmm_last_error_string()
  # workspace size: xq + scales + row sums, 256-byte granules
  assert L.qmm_workspace_size(_capi.OP_W8A8_PERCHANNEL, 2048, 4096, 4096) == 2048 * 4096 + 2 * 8192
  assert L.qmm_workspace_size(_capi.OP_W8A16_PERCHANNEL, 16, 4096, 4096) == 0
  # fused gate/up: the interleaved weight has a multiple of 16 rows
  assert L.qmm_gate_up_decode(4, 1, 1, 1, 1, 1, 1, 1, 24, 128, 0, None) == 1
  assert b"multiple of 16" in L.qmm_last_error_string()
  assert L.qmm_gate_up(4, 1, 1, 1, 1, 1, 1, 64, 24, 128, 0, None, 0, None) == 1
  assert b"multiple of 16" in L.qmm_last_error_string()
  # scratch of the weight-only entry point: grows with the batch, never shrinks; the int4 form adds room for the
  # weights as int8 from 384 tokens
  sizes = [L.qmm_weight_only_workspace_size(m, 4096) for m in (1, 16, 32, 33, 64, 65, 512, 1008, 1024, 4096)]
  assert all(a <= b for a, b in zip(sizes, sizes[1:])) and sizes[0] > 0
  assert L.qmm_weight_only_workspace_size_for(8, 512, 14336, 4096) == L.qmm_weight_only_workspace_size(512, 4096)
  assert L.qmm_weight_only_workspace_size_for(4, 64, 14336, 4096) == L.qmm_weight_only_workspace_size(64, 4096)
  assert L.qmm_weight_only_workspace_size_for(4, 512, 14336, 4096) >= L.qmm_weight_only_workspace_size(512, 4096) + 14336 * 4096
  # limbs per activation: by output type (0) or three everywhere (3)
  assert L.qmm_set_activation_limbs(3) == 0 and L.qmm_set_activation_limbs(0) == 0
  assert L.qmm_set_activation_limbs(2) == 1
  # exchange buffers of the fused row-parallel kernel: two slots of `world` regions, one flag word per rank and tile
  world, max_m, n = 8, 8, 8192
  want = 2 * world * max_m * n * 4 + (world * (n // 16) + 2) * 4
  assert L.qmm_rowparallel_buffer_bytes(max_m, n, world) == (want + 255) // 256 * 256
  assert L.qmm_rowparallel_buffer_bytes(0, n, world) == 0
  # one-shot all-reduce: whole float4 vectors only, at most 8 ranks
  ptrs = (ctypes.c_void_p * 2)(16, 32)
  assert L.qmm_allreduce_oneshot(ptrs, ptrs, 0, 2, 1, 64, 0, 6, None) == 1
  assert L.qmm_allreduce_oneshot(ptrs, ptrs, 0, 9, 1, 64, 0, 8, None) == 1
  # host pipeline: argument checks come before any CUDA call
  handle = ctypes.c_void_p()
  assert L.qmm_host_pipeline_create(0, 16, 2, ctypes.byref(handle)) == 1
  assert L.qmm_host_pipeline_create(16, 16, 65, ctypes.byref(handle)) == 1
  assert L.qmm_host_pipeline_create(16, 16, 2, None) == 6
  assert L.qmm_host_weight_only(None, 0, 16, 1, 16, 16, None, 16, 1, 1, 4, 128, 128, 0) == 6
  assert L.qmm_host_pipeline_sync(None) == 6
  assert L.qmm_host_pipeline_destroy(None) == 0
  with pytest.raises(AssertionError):
    _capi.check(1)
  with pytest.raises(NotImplementedError):
    _capi.check(2)
