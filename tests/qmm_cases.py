"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Everything is generated on the CPU from ``torch.Generator().manual_seed(seed)`` so that the oracle
and the CUDA kernels see identical bits.
"""
import torch


def gen(seed=0):
  return torch.Generator().manual_seed(seed)


def activations(g, m, k, dtype=torch.bfloat16, outliers=False):
  x = torch.randn(m, k, generator=g)
  if outliers:  # 1 % of the entries multiplied by 20 (W8A8 prefill configuration)
    mask = torch.rand(m, k, generator=g) < 0.01
    x = torch.where(mask, x * 20.0, x)
  return x.to(dtype)


def int8_weight(g, n, k):
  return torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)


def int4_weight(g, n, k):
  """int4 values in an int8 container, [N,K]."""
  return torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)


def per_channel_scale(g, n):
  return torch.rand(n, generator=g) * 0.019 + 0.001


def blockwise_scale(g, s, n):
  return torch.rand(s, n, generator=g) * 0.045 + 0.005


def to_sbn(w_nk, block_size):
  """[N,K] -> [K/bs, bs, N], the reference's blockwise layout."""
  n, k = w_nk.shape
  return w_nk.reshape(n, k // block_size, block_size).permute(1, 2, 0).contiguous()
