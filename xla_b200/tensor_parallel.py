"""Tensor-parallel use of the quantized linear: column- and row-sharded weights across the GPUs of a box.

The reference attaches no collective to this operator; under SPMD it would mark the weight sharded
(torch_xla/distributed/spmd/xla_sharding.py:685 ``mark_sharding``) and let XLA insert the all-reduce
(torch_xla/csrc/cross_replica_reduces.cpp:154).  Here the sharding is explicit, one process per GPU:

  column-parallel  rank r holds output rows [r*N/G, (r+1)*N/G); x is replicated; the output stays
                   sharded along N; no communication.
  row-parallel     rank r holds the K slice [r*K/G, (r+1)*K/G) of every weight row and the matching
                   slice of the activations; each rank produces a partial [M, N]; one all-reduce (sum)
                   over NCCL finishes it.  Per-channel scales are applied on every rank before the sum
                   (they distribute over it); blockwise scales are sliced with their K blocks.

``local_op`` is the function that runs the local quantized matmul.  On GPUs it is the packed sibling
operator; the CPU tests of the sharding arithmetic pass the CPU oracle instead.
"""
import torch
import torch.distributed as dist


def _world(group=None):
  if dist.is_available() and dist.is_initialized():
    return dist.get_rank(group), dist.get_world_size(group)
  return 0, 1


def _default_local_op(x, w, scaler, zero_point, block_size, int4_weight, weight_is_packed, out_dtype, out=None):
  from . import packed
  return packed.quantized_matmul_packed(x, w, scaler, zero_point, block_size=block_size, int4_weight=int4_weight,
                                        weight_is_packed=weight_is_packed, out_dtype=out_dtype, out=out)


def shard_column(w, scaler, zero_point, rank, world, block_size=-1):
  """Rows [r*N/G, (r+1)*N/G) of a K-minor weight ([N,K] int8 or [N,K/2] packed) and their scales."""
  n = w.shape[0]
  assert n % world == 0, f"out_features {n} must divide evenly over {world} ranks"
  lo, hi = rank * n // world, (rank + 1) * n // world
  pick = (lambda t: None if t is None else t[lo:hi].contiguous()) if block_size == -1 else (
      lambda t: None if t is None else t[:, lo:hi].contiguous())
  return w[lo:hi].contiguous(), pick(scaler), pick(zero_point)


def shard_row(w, scaler, zero_point, rank, world, in_features, block_size=-1, weight_is_packed=False):
  """K slice [r*K/G, (r+1)*K/G) of every weight row; blockwise scales are sliced with their blocks."""
  k = in_features
  assert k % world == 0, f"in_features {k} must divide evenly over {world} ranks"
  kl = k // world
  if block_size != -1:
    assert kl % block_size == 0, f"each rank's K slice ({kl}) must hold whole blocks of {block_size}"
  if weight_is_packed:
    assert kl % 2 == 0
    wl = w[:, rank * kl // 2:(rank + 1) * kl // 2].contiguous()
  else:
    wl = w[:, rank * kl:(rank + 1) * kl].contiguous()
  if block_size == -1:
    return wl, scaler, zero_point  # per-channel scale/zero point apply to every rank's partial
  sl = kl // block_size
  pick = lambda t: None if t is None else t[rank * sl:(rank + 1) * sl].contiguous()
  return wl, pick(scaler), pick(zero_point)


class ColumnParallelQuantizedLinear(torch.nn.Module):
  """out[:, r*N/G:(r+1)*N/G] = quantized_matmul(x, local weight); no communication."""

  def __init__(self, w, scaler, zero_point=None, block_size=-1, int4_weight=False, weight_is_packed=False,
               out_dtype=None, group=None, local_op=None):
    super().__init__()
    self.group = group
    rank, world = _world(group)
    wl, sl, zl = shard_column(w, scaler, zero_point, rank, world, block_size)
    self.register_buffer("weight", wl)
    self.register_buffer("weight_scaler", sl)
    self.zero_point = zl
    self.block_size, self.int4_weight, self.weight_is_packed = block_size, int4_weight, weight_is_packed
    self.out_dtype = out_dtype
    self.local_op = local_op or _default_local_op

  def forward(self, x, gather=False):
    y = self.local_op(x, self.weight, self.weight_scaler, self.zero_point, self.block_size, self.int4_weight,
                      self.weight_is_packed, self.out_dtype)
    _, world = _world(self.group)
    if gather and world > 1:
      parts = [torch.empty_like(y) for _ in range(world)]
      dist.all_gather(parts, y.contiguous(), group=self.group)
      y = torch.cat(parts, dim=-1)
    return y


class RowParallelQuantizedLinear(torch.nn.Module):
  """out = all_reduce_sum_r quantized_matmul(x[:, K slice r], local weight)."""

  def __init__(self, w, scaler, zero_point=None, in_features=None, block_size=-1, int4_weight=False,
               weight_is_packed=False, out_dtype=None, reduce_dtype=torch.float32, group=None, local_op=None,
               peer_reduce=None, fused_decode=None):
    super().__init__()
    self.group = group
    # a xla_b200.peer_reduce.FusedRowParallelDecode: decode batches (M <= 8, symmetric weights) run the kernel
    # that also sums over the ranks
    self.fused_decode = fused_decode
    # a xla_b200.peer_reduce.PeerAllReduce: results that fit its buffers are summed by the one-shot
    # peer-memory kernel instead of the process group's all-reduce
    self.peer_reduce = peer_reduce
    rank, world = _world(group)
    k = in_features if in_features is not None else (w.shape[1] * (2 if weight_is_packed else 1))
    wl, sl, zl = shard_row(w, scaler, zero_point, rank, world, k, block_size, weight_is_packed)
    self.register_buffer("weight", wl)
    self.register_buffer("weight_scaler", sl)
    # a per-channel zero point is a term -(sum_k x) * zp over the FULL K: every rank subtracts its own
    # K slice's share, so it stays on every rank unchanged
    self.zero_point = zl
    self.block_size, self.int4_weight, self.weight_is_packed = block_size, int4_weight, weight_is_packed
    self.out_dtype, self.reduce_dtype = out_dtype, reduce_dtype
    self.in_features_local = k // world
    self.local_op = local_op or _default_local_op

  def local_slice(self, x_full):
    """The K slice of replicated activations that belongs to this rank."""
    rank, _ = _world(self.group)
    kl = self.in_features_local
    return x_full[..., rank * kl:(rank + 1) * kl]

  def forward(self, x_local):
    _, world = _world(self.group)
    pr, fd = self.peer_reduce, self.fused_decode
    if fd is not None and world > 1 and self.zero_point is None and self.local_op is _default_local_op:
      M = x_local.numel() // x_local.shape[-1]
      if fd.fits(M, self.weight.shape[0]) and x_local.dtype in (torch.bfloat16, torch.float16):
        return fd(x_local, self.weight, self.weight_scaler, self.block_size, self.weight_is_packed,
                  self.out_dtype if self.out_dtype is not None else torch.float32)
    if pr is not None and world > 1 and self.local_op is _default_local_op:
      M = x_local.numel() // x_local.shape[-1]
      N = self.weight.shape[0]
      if pr.fits(M, N):
        out_dtype = self.out_dtype if self.out_dtype is not None else torch.float32
        self.local_op(x_local.reshape(M, -1), self.weight, self.weight_scaler, self.zero_point, self.block_size,
                      self.int4_weight, self.weight_is_packed, torch.float32, out=pr.partial_view(M, N))
        return pr.reduce(M, N, out_dtype).reshape(x_local.shape[:-1] + (N,))
    part_dtype = self.reduce_dtype if world > 1 else self.out_dtype
    y = self.local_op(x_local, self.weight, self.weight_scaler, self.zero_point, self.block_size, self.int4_weight,
                      self.weight_is_packed, part_dtype)
    if world > 1:
      dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
    if self.out_dtype is not None and y.dtype != self.out_dtype:
      y = y.to(self.out_dtype)
    return y
