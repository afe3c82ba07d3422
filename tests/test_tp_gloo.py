"""Tensor-parallel sharding arithmetic on CPU: two gloo ranks, the CPU oracle as the local matmul.

Column-parallel shards must concatenate to, and row-parallel shards must all-reduce to, the unsharded
oracle result (the only pin the reference offers for sharded runs: equality with the unsharded op).
"""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _unpack(wp):
  lo = (wp & 0xF).to(torch.int8)
  hi = (wp >> 4).to(torch.int8)
  lo = torch.where(lo > 7, lo - 16, lo)
  hi = torch.where(hi > 7, hi - 16, hi)
  return torch.stack([lo, hi], -1).reshape(wp.shape[0], -1)


def _oracle_local_op(x, w, scaler, zero_point, block_size, int4_weight, weight_is_packed, out_dtype):
  from oracle import qmm_oracle as qo
  w_nk = _unpack(w) if weight_is_packed else w
  if block_size == -1:
    y = qo.quantized_matmul(x, w_nk, scaler, zero_point, dot_round=None)
  else:
    w_sbn = qo.nk_to_sbn(w_nk, block_size)
    y = qo.quantized_matmul(x.float(), w_sbn, scaler, zero_point, block_size=block_size, dot_round=None)
  return y.to(out_dtype or torch.float32)


def _worker(rank, world, port, results):
  sys.path.insert(0, ROOT)
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    from oracle import qmm_oracle as qo
    from xla_b200 import tensor_parallel as tp
    g = torch.Generator().manual_seed(0)
    M, K, N, bs = 3, 512, 64, 128
    x = torch.randn(M, K, generator=g).bfloat16()
    w4 = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)
    wp = qo.pack_int4_nk(w4)
    sb = torch.rand(K // bs, N, generator=g) * 0.045 + 0.005
    full_bw = qo.quantized_matmul(x.float(), qo.nk_to_sbn(w4, bs), sb, block_size=bs, dot_round=None).float()
    w8 = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    sc = torch.rand(N, generator=g) * 0.019 + 0.001
    zp = torch.randint(-8, 9, (N,), generator=g).float() * sc
    full_pc = qo.quantized_matmul(x, w8, sc, zp, dot_round=None).float()

    ok = True
    # column-parallel, blockwise packed int4: shards concatenate to the full result
    col = tp.ColumnParallelQuantizedLinear(wp, sb, block_size=bs, int4_weight=True, weight_is_packed=True,
                                           local_op=_oracle_local_op)
    assert tuple(col.weight.shape) == (N // world, K // 2) and tuple(col.weight_scaler.shape) == (K // bs, N // world)
    y = col(x)
    assert y.shape == (M, N // world)
    ok &= torch.allclose(y, full_bw[:, rank * N // world:(rank + 1) * N // world], rtol=1e-5, atol=1e-5)
    ok &= torch.allclose(col(x, gather=True), full_bw, rtol=1e-5, atol=1e-5)
    # row-parallel, blockwise packed int4: partials all-reduce to the full result
    row = tp.RowParallelQuantizedLinear(wp, sb, block_size=bs, int4_weight=True, weight_is_packed=True,
                                        local_op=_oracle_local_op)
    assert tuple(row.weight.shape) == (N, K // 2 // world) and tuple(row.weight_scaler.shape) == (K // bs // world, N)
    ok &= torch.allclose(row(row.local_slice(x)), full_bw, rtol=1e-5, atol=1e-5)
    # row-parallel, per-channel int8 with a zero point: scale and zero point stay on every rank
    rowpc = tp.RowParallelQuantizedLinear(w8, sc, zp, local_op=_oracle_local_op)
    ok &= torch.allclose(rowpc(rowpc.local_slice(x)), full_pc, rtol=1e-5, atol=1e-5)
    # bf16 partials (the all-reduce payload the configuration names): within bf16 resolution
    rowbf = tp.RowParallelQuantizedLinear(w8, sc, reduce_dtype=torch.bfloat16, out_dtype=torch.bfloat16,
                                          local_op=_oracle_local_op)
    ref = qo.quantized_matmul(x, w8, sc, dot_round=None)
    ok &= qo.max_abs_rel(rowbf(rowbf.local_slice(x)), ref) < 1e-2
    # shapes that do not shard are refused
    try:
      tp.shard_row(wp, sb, None, rank, world, K, block_size=512, weight_is_packed=True)
      ok = False
    except AssertionError:
      pass
    results[rank] = bool(ok)
  finally:
    dist.destroy_process_group()


def test_column_and_row_parallel_match_unsharded_oracle():
  world = 2
  ctx = mp.get_context("spawn")
  results = ctx.Manager().dict()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
  for p in procs:
    p.start()
  for p in procs:
    p.join(timeout=120)
    assert p.exitcode == 0, f"rank exited with {p.exitcode}"
  assert dict(results) == {0: True, 1: True}


def test_single_process_defaults_to_world_one():
  from xla_b200 import tensor_parallel as tp
  w = torch.zeros(8, 16, dtype=torch.int8)
  wl, sl, _ = tp.shard_column(w, torch.ones(8), None, 0, 1)
  assert wl.shape == w.shape and sl.shape == (8,)
  wl, sl, _ = tp.shard_row(w, torch.ones(8), None, 1, 2, 16)
  assert wl.shape == (8, 8)
  with pytest.raises(AssertionError):
    tp.shard_column(w, torch.ones(8), None, 0, 3)
