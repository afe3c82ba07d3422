"""Tensor-parallel quantized linear on real GPUs: two NCCL ranks, column- and row-sharded weights, the
row-parallel output all-reduced, compared with the unsharded kernel and with the CPU oracle.
Skipped on boxes with fewer than two GPUs (the sharding arithmetic itself is covered on CPU with gloo).
"""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _worker(rank, world, port, results):
  sys.path.insert(0, ROOT)
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  import torch.distributed as dist
  torch.cuda.set_device(rank)
  dev = torch.device("cuda", rank)
  dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
  try:
    import xla_b200
    from oracle import qmm_oracle as qo
    from xla_b200 import tensor_parallel as tp
    from xla_b200 import _capi, peer_reduce
    import ctypes
    g = torch.Generator().manual_seed(0)  # same seed on every rank: identical full tensors
    H, F, bs = 1024, 2048, 128
    ok = True
    peers = peer_reduce.PeerAllReduce(max_elems=64 * H)
    fused = peer_reduce.FusedRowParallelDecode(N=H, max_M=8)
    for M in (1, 8, 64):
      x = torch.randn(M, H, generator=g).bfloat16()
      w_up = torch.randint(-8, 8, (F, H), generator=g, dtype=torch.int8)
      s_up = torch.rand(H // bs, F, generator=g) * 0.045 + 0.005
      w_dn = torch.randint(-8, 8, (H, F), generator=g, dtype=torch.int8)
      s_dn = torch.rand(F // bs, H, generator=g) * 0.045 + 0.005
      wp_up, wp_dn = xla_b200.pack_int4(w_up.to(dev)), xla_b200.pack_int4(w_dn.to(dev))
      col = tp.ColumnParallelQuantizedLinear(wp_up, s_up.to(dev), block_size=bs, int4_weight=True,
                                             weight_is_packed=True, out_dtype=torch.bfloat16)
      row = tp.RowParallelQuantizedLinear(wp_dn, s_dn.to(dev), block_size=bs, int4_weight=True,
                                          weight_is_packed=True, out_dtype=torch.bfloat16)
      h_local = col(x.to(dev))                      # [M, F/world], stays sharded
      y = row(h_local)                              # the column shard is exactly this rank's K slice
      # unsharded kernels on this rank
      op = torch.ops.xla_b200.quantized_matmul_packed
      h_full = op(x.to(dev), wp_up, s_up.to(dev), block_size=bs, int4_weight=True, weight_is_packed=True,
                  out_dtype=torch.bfloat16)
      y_full = op(h_full, wp_dn, s_dn.to(dev), block_size=bs, int4_weight=True, weight_is_packed=True,
                  out_dtype=torch.bfloat16)
      ok &= torch.equal(h_local, h_full[:, rank * F // world:(rank + 1) * F // world])
      ok &= qo.max_abs_rel(y, y_full) < 1e-2
      # the same row-parallel linear with the one-shot peer-memory all-reduce, twice (both buffer slots)
      row_p = tp.RowParallelQuantizedLinear(wp_dn, s_dn.to(dev), block_size=bs, int4_weight=True, weight_is_packed=True,
                                            out_dtype=torch.bfloat16, peer_reduce=peers)
      for _ in range(2):
        y_p = row_p(h_local)
        ok &= y_p.shape == y.shape and y_p.dtype == y.dtype
        ok &= qo.max_abs_rel(y_p, y_full) < 1e-2
        ok &= qo.max_abs_rel(y_p, y) < 1e-2
      # every rank summed the same partials in the same order: identical bits everywhere
      gathered = [torch.empty_like(y_p) for _ in range(world)]
      dist.all_gather(gathered, y_p)
      ok &= all(torch.equal(t, gathered[0]) for t in gathered)
      if M <= 8:
        # and with the exchange fused into the decode kernel itself, three calls (both slots, counter wrap of the slots)
        row_f = tp.RowParallelQuantizedLinear(wp_dn, s_dn.to(dev), block_size=bs, int4_weight=True, weight_is_packed=True,
                                              out_dtype=torch.bfloat16, fused_decode=fused)
        for _ in range(3):
          y_f = row_f(h_local)
          ok &= y_f.shape == y.shape and y_f.dtype == y.dtype
          # same order of addition over the ranks; inside a tile the two paths may split K over a different number
          # of warps (the exchange kernel always uses four), so the partial sums agree to fp32 rounding only
          ok &= qo.max_abs_rel(y_f, y_p) < 1e-2 and qo.max_abs_rel(y_f, y_full) < 1e-2
        gathered = [torch.empty_like(y_f) for _ in range(world)]
        dist.all_gather(gathered, y_f)
        ok &= all(torch.equal(t, gathered[0]) for t in gathered)
      # and the oracle for the first linear
      exact = qo.quantized_matmul(x.float(), qo.nk_to_sbn(w_up, bs), s_up, block_size=bs, dot_round=None)
      ok &= qo.max_abs_rel(col(x.to(dev), gather=True), exact) < 1e-2
    flag = ctypes.c_uint32(7)
    ok &= _capi.lib().qmm_device_error_flag(ctypes.byref(flag), _capi.stream_ptr(dev)) == 0 and flag.value == 0
    peers.close()
    fused.close()
    results[rank] = bool(ok)
  finally:
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_mlp_two_ranks_nccl():
  world = 2
  ctx = mp.get_context("spawn")
  results = ctx.Manager().dict()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
  for p in procs:
    p.start()
  for p in procs:
    p.join(timeout=300)
    assert p.exitcode == 0, f"rank exited with {p.exitcode}"
  assert dict(results) == {0: True, 1: True}
