"""Generates tests/golden/qmm_golden.npz from the UNMODIFIED reference implementation.

Run where a pytorch/xla checkout is available (it is not needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/pytorch-xla

The reference file torch_xla/experimental/xla_quantized_matmul.py is loaded by path after
pre-seeding ``sys.modules`` with stand-ins for ``torch_xla`` and
``torch_xla.core.xla_model`` (the latter only has to provide ``XLA_LIB``); its eager CPU
kernel (dispatch key CompositeExplicitAutograd, :139-183) and ``_quantize_tensor`` (:56-73)
then run as they are.  Each case stores the inputs and the reference's outputs, so that the
CPU oracle and the CUDA kernels can be pinned against them without the reference present.
"""
import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch


def load_reference(root):
  if "torch_xla" not in sys.modules:
    tx = types.ModuleType("torch_xla")
    core = types.ModuleType("torch_xla.core")
    xm = types.ModuleType("torch_xla.core.xla_model")
    xm.XLA_LIB = torch.library.Library("xla", "DEF")
    tx.core, core.xla_model = core, xm
    sys.modules.update({"torch_xla": tx, "torch_xla.core": core, "torch_xla.core.xla_model": xm})
  path = os.path.join(root, "torch_xla", "experimental", "xla_quantized_matmul.py")
  spec = importlib.util.spec_from_file_location("reference_xla_quantized_matmul", path)
  mod = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(mod)
  return mod


def bits(t):
  """numpy view that keeps every bit: bf16 as uint16, everything else as is."""
  t = t.detach().cpu().contiguous()
  if t.dtype == torch.bfloat16:
    return t.view(torch.int16).numpy().view(np.uint16)
  return t.numpy()


def outlier_activations(gen, m, k, dtype):
  """N(0,1) with 1% of the entries multiplied by 20 (the W8A8 prefill distribution)."""
  x = torch.randn(m, k, generator=gen)
  mask = torch.rand(m, k, generator=gen) < 0.01
  x = torch.where(mask, x * 20.0, x)
  return x.to(dtype)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--reference", required=True, help="checkout of the reference project (pytorch/xla)")
  ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                 "qmm_golden.npz"))
  args = ap.parse_args()
  ref = load_reference(args.reference)
  op = torch.ops.xla.quantized_matmul
  out = {}
  torch.set_num_threads(1)

  # --- _quantize_tensor on bf16 activations, including rows whose pre-cast value hits +128 ---
  gen = torch.Generator().manual_seed(0)
  x = outlier_activations(gen, 48, 2048, torch.bfloat16)
  xq, xs = ref._quantize_tensor(x)
  pre = torch.round(x / (torch.amax(torch.abs(x), dim=-1, keepdim=True) / 127))
  out["quant_bf16/x"] = bits(x)
  out["quant_bf16/xq"] = bits(xq)
  out["quant_bf16/scale"] = bits(xs)
  out["quant_bf16/n_plus128"] = np.array(int((pre.float() == 128.0).sum()))
  print("quant_bf16: +128 positions:", int((pre.float() == 128.0).sum()), "of", x.numel())

  gen = torch.Generator().manual_seed(1)
  x = outlier_activations(gen, 8, 512, torch.float32)
  xq, xs = ref._quantize_tensor(x)
  out["quant_f32/x"], out["quant_f32/xq"], out["quant_f32/scale"] = bits(x), bits(xq), bits(xs)

  # --- W8A8 per-channel: int32 accumulator and the op's fp32 output, with and without zp ---
  for tag, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
    gen = torch.Generator().manual_seed(2)
    x = outlier_activations(gen, 16, 256, dt)
    w = torch.randint(-127, 128, (64, 256), generator=gen, dtype=torch.int8)
    s = torch.rand(64, generator=gen) * 0.019 + 0.001
    zp = torch.randint(-8, 9, (64,), generator=gen).float() * s
    xq, xs = ref._quantize_tensor(x)
    acc = torch.nn.functional.linear(xq.to(torch.int32), w.to(torch.int32))
    k = f"w8a8_{tag}"
    out[k + "/x"], out[k + "/w"], out[k + "/scale"], out[k + "/zp"] = bits(x), bits(w), bits(s), bits(zp)
    out[k + "/xq"], out[k + "/x_scale"], out[k + "/acc"] = bits(xq), bits(xs), bits(acc)
    out[k + "/out"] = bits(op(x, w, s, quantize_activation=True))
    out[k + "/out_zp"] = bits(op(x, w, s, zp, quantize_activation=True))

  # --- weight-only per-channel (bf16 and fp32 activations; reference test shape 3x5 -> 8) ---
  for tag, dt, (m, kk, n) in (("bf16", torch.bfloat16, (5, 64, 24)), ("f32", torch.float32, (3, 5, 8)),
                              ("f32b", torch.float32, (4, 128, 32))):
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(m, kk, generator=gen).to(dt)
    w = torch.randint(-127, 128, (n, kk), generator=gen, dtype=torch.int8)
    s = torch.rand(n, generator=gen) * 0.019 + 0.001
    zp = torch.randint(-8, 9, (n,), generator=gen).float() * s
    k = f"pc_{tag}"
    out[k + "/x"], out[k + "/w"], out[k + "/scale"], out[k + "/zp"] = bits(x), bits(w), bits(s), bits(zp)
    out[k + "/out"] = bits(op(x, w, s))
    out[k + "/out_zp"] = bits(op(x, w, s, zp))

  # --- blockwise (layout [S, bs, N]); first case is the reference's own known-answer shape ---
  for tag, (m, kk, n, bs) in (("kat", (3, 6, 8, 2)), ("b128", (4, 256, 16, 128))):
    gen = torch.Generator().manual_seed(4)
    x = torch.rand(m, kk, generator=gen)
    w = torch.randint(-8, 8, (kk // bs, bs, n), generator=gen, dtype=torch.int8)
    s = (torch.ones(kk // bs, n) if tag == "kat" else
         torch.rand(kk // bs, n, generator=gen) * 0.045 + 0.005)
    zp = torch.randint(-3, 4, (kk // bs, n), generator=gen).float() * s
    k = f"bw_{tag}"
    out[k + "/x"], out[k + "/w"], out[k + "/scale"], out[k + "/zp"] = bits(x), bits(w), bits(s), bits(zp)
    out[k + "/block_size"] = np.array(bs)
    out[k + "/out"] = bits(op(x, w, s, block_size=bs))
    out[k + "/out_zp"] = bits(op(x, w, s, zp, block_size=bs))
    out[k + "/out_int4flag"] = bits(op(x, w, s, block_size=bs, int4_weight=True))

  # --- the module: buffer names and forward, per-channel symmetric ---
  gen = torch.Generator().manual_seed(5)
  m = ref.XlaQuantizedLinear(32, 16, is_symmetric=True)
  out["module/state_keys_sym"] = np.array(sorted(m.state_dict().keys()))
  out["module/state_keys_asym"] = np.array(sorted(ref.XlaQuantizedLinear(32, 16).state_dict().keys()))
  w = torch.randint(-127, 128, (16, 32), generator=gen, dtype=torch.int8)
  s = torch.rand(16, generator=gen) * 0.019 + 0.001
  x = torch.randn(2, 3, 32, generator=gen)
  m.load_quantized_weight(w, s)
  out["module/x"], out["module/w"], out["module/scale"] = bits(x), bits(w), bits(s)
  out["module/out"] = bits(m(x))

  np.savez_compressed(args.out, **out)
  print("wrote", args.out, os.path.getsize(args.out), "bytes,", len(out), "arrays")


if __name__ == "__main__":
  main()
