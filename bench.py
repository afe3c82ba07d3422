"""Benchmark of the weight-quantized linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (every N, including 1): the tensor-parallel configuration - a Llama-3-70B-shaped MLP, W4A16 blockwise int4
(block 128): gate and up [28672, 8192] column-sharded over the N GPUs (no communication), down [8192, 28672]
row-sharded with one sum exchange of the partial outputs; x bf16 [M, 8192] for M in {1, 64, 512}, bf16 output.
Total work is fixed as N grows ("scaling": "strong").  One STEP = `--reps` passes of the three linears + exchange for
each M.  Weights rotate through a pool of copies larger than L2 wherever one copy of a GPU's shards would fit in L2.

  value      tokens/s with inputs resident in HBM: CUDA events around the K steps, max over ranks.  M = 1 and 64 are
             CUDA-graph replays (launch-bound otherwise); M = 512 is launched eagerly with events around every
             linear, which is where the roofline's per-launch duration comes from.
  roofline   the dominant kernel (largest share of the step): algorithmic flops per launch / its average launch
             duration inside the timed region, against the measured peak (MEASURED_PEAKS.json).
  e2e        the same metric with HOST activations through the public operator and sharding helpers: every pass
             copies x in from pinned host memory and the result out to pinned host memory inside the timed region.
  tp.checked before anything is timed: the sharded result against the unsharded operator on the same seeded inputs,
             bit-identity across ranks, the device error word.
  cpu_baseline / --impl reference: the reference's CPU path (oracle/torch_port.py, the same ATen operators) on the
             host cores, on a bounded sample of the same workload.

`other_configs` (N = 1 only) carries kernel timings of the remaining benchmark configurations.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      d = json.load(f)
    return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
            "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
  return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
  """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
  QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self, index):
    self.index, self.rows, self.proc = index, [], None

  def start(self):
    try:
      self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                    "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                   stderr=subprocess.DEVNULL, text=True)
      self.thread = threading.Thread(target=self._read, daemon=True)
      self.thread.start()
    except OSError:
      self.proc = None

  def _read(self):
    for line in self.proc.stdout:
      self.rows.append([c.strip() for c in line.split(",")])

  def stop(self):
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    time.sleep(0.15)
    self.proc.terminate()
    try:
      self.proc.wait(timeout=2)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    sm = sorted(float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit())
    mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
    return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None, "reasons": reasons,
            "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# the workload
# ------------------------------------------------------------------------------------------------

H, F, BS = 8192, 28672, 128
MS = (1, 64, 512)
WORKLOAD = ("Llama-3-70B-shaped MLP, W4A16 blockwise int4 (block 128): gate/up int4 [28672,8192] column-sharded, down int4 "
            "[8192,28672] row-sharded + sum exchange; x bf16 [M,8192] ~N(0,1), M in {1,64,512}; bf16 out")
DTYPE = "bf16 activations x int4 weights, fp32 accumulate"


def config_dict(world, reps):
  """The same dictionary for both arms."""
  return {"workload": WORKLOAD, "reps_per_M": reps, "parallelism": f"tp{world}" if world > 1 else "single GPU",
          "flush": "GPU arm: every pass streams more weight bytes than L2 holds, or rotates through a pool of weight "
                   "copies larger than L2 where one GPU's shards would fit; CPU arm: n/a"}


def algorithmic_bytes(m, world):
  """Compulsory HBM bytes per GPU of one MLP pass: every weight, scale, activation and output once."""
  fl = F // world
  w = 3 * (fl * H // 2)
  sc = 4 * (2 * (H // BS) * fl + (fl // BS) * H)
  act = 2 * m * (H + H + fl) + 2 * m * (fl + fl + H)
  return w + sc + act


class TPMlp:
  """This rank's shards of the MLP, `copies` times over, and the three exchange forms of the down projection."""

  def __init__(self, dev, rank, world, seed, want_check=True):
    from xla_b200 import tensor_parallel as tp
    self.dev, self.rank, self.world = dev, rank, world
    self.fl = F // world
    g = torch.Generator(device=dev).manual_seed(seed)  # the same seed on every rank: identical full weights
    per_copy = 3 * (self.fl * H // 2) + 4 * (2 * (H // BS) * self.fl + (self.fl // BS) * H)
    self.copies = max(1, -(-2 * L2_BYTES // per_copy)) if per_copy < 2 * L2_BYTES else 1
    self.sets = []
    self.full0 = None
    for c in range(self.copies):
      mk = lambda n, k: torch.randint(0, 256, (n, k // 2), generator=g, device=dev, dtype=torch.uint8)
      mks = lambda k, n: torch.rand(k // BS, n, generator=g, device=dev) * 0.045 + 0.005
      gw, gs = mk(F, H), mks(H, F)
      uw, us = mk(F, H), mks(H, F)
      dw, ds = mk(H, F), mks(F, H)
      if c == 0 and want_check and world > 1:
        self.full0 = (gw, gs, uw, us, dw, ds)
      sh = (tp.shard_column(gw, gs, None, rank, world, BS)[:2] + tp.shard_column(uw, us, None, rank, world, BS)[:2] +
            tp.shard_row(dw, ds, None, rank, world, F, BS, weight_is_packed=True)[:2])
      self.sets.append(sh)
      del gw, gs, uw, us, dw, ds
    self.x = {m: torch.randn(m, H, generator=g, device=dev).bfloat16() for m in MS}
    self.peers = self.fused = None
    if world > 1:
      try:
        from xla_b200 import peer_reduce
        self.peers = peer_reduce.PeerAllReduce(max_elems=64 * H)
        self.fused = peer_reduce.FusedRowParallelDecode(N=H, max_M=8)
      except Exception as e:  # no peer access between these GPUs: NCCL serves every batch
        print(f"[bench] peer-memory exchange unavailable ({type(e).__name__}: {e})", file=sys.stderr)
    self._i = 0
    self.chosen = {}

  def lin(self, x, w, s, out_dtype=torch.bfloat16, out=None):
    from xla_b200 import packed
    return packed.quantized_matmul_packed(x, w, s, block_size=BS, int4_weight=True, weight_is_packed=True, out_dtype=out_dtype,
                                          out=out)

  def exchange_options(self, m):
    """The sum exchanges that can serve a batch of m tokens on this set-up."""
    if self.world == 1:
      return ["none"]
    opts = ["nccl"]
    if self.peers is not None and self.peers.fits(m, H):
      opts.append("peer")
    if self.fused is not None and self.fused.fits(m, H):
      opts.append("fused")
    return opts

  def exchange_for(self, m):
    """The exchange used for a batch of m tokens: the fastest of the available forms as measured by choose_exchanges()
    (NCCL until then)."""
    return self.chosen.get(m, "none" if self.world == 1 else "nccl")

  def choose_exchanges(self, stream, ms):
    """Times one MLP pass per available exchange form and batch size (CUDA-graph replays, max over ranks) and keeps
    the fastest; every rank sees the same numbers, so every rank makes the same choice."""
    import torch.distributed as dist
    table = {}
    for m in ms:
      if m not in self.x:
        self.x[m] = self.x[64][:m].contiguous()
      row = {}
      for ex in self.exchange_options(m):
        if ex == "none":
          continue
        try:
          us = time_graph(lambda i: self.forward(m, exchange=ex), stream, reps=4, iters=3)
        except Exception as e:
          torch.cuda.synchronize(self.dev)
          print(f"[bench] exchange {ex} at M={m} not measured ({type(e).__name__}: {e})", file=sys.stderr)
          us = float("inf")
        t = torch.tensor([us], dtype=torch.float64, device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        row[ex] = float(t.item())
      if row:
        self.chosen[m] = min(row, key=row.get)
        table[f"M{m}"] = {k: (v if v != float("inf") else "not measured") for k, v in row.items()}
    return table

  def forward(self, m, x=None, exchange=None, events=None):
    """One MLP pass on the next weight copy; `events` collects (start, end) pairs around the three linears."""
    import torch.distributed as dist
    i = self._i = (self._i + 1) % self.copies
    gw, gs, uw, us, dw, ds = self.sets[i]
    x = self.x[m] if x is None else x
    ex = exchange or self.exchange_for(m)

    def timed(fn):
      if events is None:
        return fn()
      e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      e0.record()
      r = fn()
      e1.record()
      events.append((e0, e1))
      return r

    a = timed(lambda: self.lin(x, gw, gs))
    b = timed(lambda: self.lin(x, uw, us))
    del a  # silu(gate) * up is not part of the configuration: the three linears and the exchange are
    if ex == "fused":
      return timed(lambda: self.fused(b, dw, ds, block_size=BS, weight_is_packed=True, out_dtype=torch.bfloat16))
    if ex == "peer":
      timed(lambda: self.lin(b, dw, ds, out_dtype=torch.float32, out=self.peers.partial_view(m, H)))
      return self.peers.reduce(m, H, torch.bfloat16)
    y = timed(lambda: self.lin(b, dw, ds))
    if ex == "nccl":
      dist.all_reduce(y)
    return y

  def check(self):
    """Sharded against unsharded on the same inputs, identity across ranks, the device error word."""
    import torch.distributed as dist
    from xla_b200 import _capi
    if self.world == 1:
      return {"note": "single GPU: nothing is sharded; parity with the CPU oracle is covered by the test suite"}
    gw, gs, uw, us, dw, ds = self.full0
    res = {}
    worst, identical = 0.0, True
    for m in (1, 8, 64):
      x = self.x[64][:m].contiguous()
      b_full = self.lin(x, uw, us)
      ref = self.lin(b_full, dw, ds, out_dtype=torch.float32)
      for ex in ("nccl", "peer", "fused"):
        if (ex == "fused" and (self.fused is None or not self.fused.fits(m, H))) or (
            ex == "peer" and (self.peers is None or not self.peers.fits(m, H))):
          continue
        self._i = -1  # weight copy 0 is the one whose full tensors were kept
        y = self.forward(m, x=x, exchange=ex).float()
        err = float((y - ref).abs().max() / ref.abs().max())
        worst = max(worst, err)
        parts = [torch.empty_like(y) for _ in range(self.world)]
        dist.all_gather(parts, y.contiguous())
        same = all(torch.equal(parts[0], q) for q in parts[1:])
        identical = identical and (same or ex == "nccl")  # only the peer-memory forms add in rank order everywhere
        res[f"M{m}_{ex}"] = {"max_abs_rel_vs_unsharded": err, "identical_across_ranks": same}
    self.full0 = None
    word = _capi.device_error(self.dev)
    t = torch.tensor([worst, 0.0 if identical else 1.0, float(word)], dtype=torch.float64, device=self.dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    worst, not_identical, word = t.tolist()
    out = {"max_abs_rel": worst, "identical_across_ranks": not_identical == 0.0, "error_word": int(word), "cases": res,
           "tolerance": 1e-2}
    if worst > 1e-2 or word != 0 or not_identical:
      raise RuntimeError(f"tensor-parallel check failed: {out}")
    return out

  def close(self):
    for o in (self.peers, self.fused):
      if o is not None:
        o.close()


# ------------------------------------------------------------------------------------------------
# CPU baseline (reference CPU path restated with the same ATen operators)
# ------------------------------------------------------------------------------------------------


def cpu_sample(seed):
  """tokens/s of the unsharded MLP on the host cores from a bounded sample: the gate projection in the reference's own
  layout ([64,128,28672] int8, fp32 activations) at M = 1 and 64, and at M = 512 on one eighth of the output rows; the
  three projections of the MLP cost the same flops and bytes each."""
  from oracle import torch_port as tp
  cores = os.cpu_count() or 1
  torch.set_num_threads(cores)
  g = torch.Generator().manual_seed(seed)
  S = H // BS
  w = torch.randint(-8, 8, (S, BS, F), generator=g, dtype=torch.int8)
  sc = torch.rand(S, F, generator=g) * 0.045 + 0.005
  n8 = F // 8
  w8, sc8 = w[:, :, :n8].contiguous(), sc[:, :n8].contiguous()
  t0 = time.perf_counter()
  per = {}
  for m in MS:
    x = torch.randn(m, H, generator=g)
    a = time.perf_counter()
    if m == 512:
      tp.quantized_matmul_cpu(x, w8, sc8, block_size=BS)
      per[m] = (time.perf_counter() - a) * (F / n8)
    else:
      tp.quantized_matmul_cpu(x, w, sc, block_size=BS)
      per[m] = time.perf_counter() - a
  dt = time.perf_counter() - t0
  value = sum(MS) / (3.0 * sum(per.values()))
  return {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "threads": torch.get_num_threads(),
          "sample": f"gate projection [64,128,28672] int8, fp32 activations: M=1 {per[1]:.2f} s, M=64 {per[64]:.2f} s, M=512 "
                    f"{per[512]:.2f} s (one eighth of the output rows, scaled by 8); an MLP pass = 3 such projections; "
                    f"{dt:.1f} s wall"}


def run_reference(args, rank, world):
  if rank != 0:
    return
  t0 = time.perf_counter()
  vals, base = [], None
  for i in range(args.warmup + args.steps):
    base = cpu_sample(args.seed)
    if i >= args.warmup:
      vals.append(base["value"])
  value = sum(vals) / len(vals)
  base["value"] = value
  line = {"impl": "reference", "metric": "qlinear_tp_mlp_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
          "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * (time.perf_counter() - t0) / max(1, args.steps + args.warmup),
          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 activations x int8-held int4",
          "data": "synthetic", "config": config_dict(world, args.reps), "cpu_baseline": base,
          "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
  print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# kernel timings of the other benchmark configurations (N = 1)
# ------------------------------------------------------------------------------------------------


def time_graph(fn, stream, reps=10, iters=5, warm=2):
  """us per call of fn(i): `reps` calls captured in one CUDA graph, replayed `iters` times."""
  with torch.cuda.stream(stream):
    for i in range(warm):
      fn(i)
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
      for i in range(reps):
        fn(i)
    g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
      g.replay()
    e1.record(stream)
    stream.synchronize()
  return e0.elapsed_time(e1) * 1e3 / (iters * reps)


def _rand_i8(gen, dev, n, k):
  return torch.randint(-127, 128, (n, k), generator=gen, device=dev, dtype=torch.int8)


def _variant_name(wbits, M, N, K, bs):
  from xla_b200 import _capi
  L = _capi.lib()
  name = L.qmm_weight_only_variant_for(wbits, M, N, K, bs, 0).decode()
  return name + (" (tuned table)" if L.qmm_tuned_variant(wbits, M, N, K, bs) else " (shape rule)")


def other_configs(dev, stream, peaks, seed):
  """W4A16 decode (configuration 2, with a plain streamed read of the same bytes beside it and the reference-layout
  operator), W8A16 decode (configuration 1), W8A8 prefill (configuration 3), the Llama-3-8B-shaped layer
  (configuration 4)."""
  import xla_b200
  from xla_b200 import _capi
  g = torch.Generator(device=dev).manual_seed(seed + 100)
  qmm = torch.ops.xla.quantized_matmul
  packed = torch.ops.xla_b200.quantized_matmul_packed
  out = {}
  hbm = peaks["hbm_gbs"]

  # ---- configuration 2: W4A16 blockwise decode, w [14336,4096] int4 packed, block 128, M in {1,8,32} ----
  N, K, bs = 14336, 4096, 128
  S = K // bs
  copies = 10
  wp = [torch.randint(0, 256, (N, K // 2), generator=g, device=dev, dtype=torch.uint8) for _ in range(copies)]
  sc = [torch.rand(S, N, generator=g, device=dev) * 0.045 + 0.005 for _ in range(copies)]
  c2 = {}
  for M in (1, 8, 32):
    x = torch.randn(M, K, generator=g, device=dev).bfloat16()
    us = time_graph(lambda i: packed(x, wp[i % copies], sc[i % copies], block_size=bs, int4_weight=True, weight_is_packed=True,
                                     out_dtype=torch.bfloat16), stream, reps=20)
    byt = N * K // 2 + 4 * S * N + 2 * M * K + 2 * M * N
    c2[f"M{M}"] = {"us": us, "gb_per_s": byt / us / 1e3, "frac_of_hbm_peak": byt / us / 1e3 / hbm, "algorithmic_bytes": byt,
                   "kernel": _variant_name(4, M, N, K, bs)}
  # a plain read of one weight copy, launched back to back the same way: what a kernel of this size can reach at all
  sink = torch.zeros(1, dtype=torch.int32, device=dev)
  Lq = _capi.lib()
  us_read = time_graph(lambda i: _capi.check(Lq.qmm_stream_read(wp[i % copies].data_ptr(), N * K // 2, sink.data_ptr(),
                                                                _capi.stream_ptr(dev))), stream, reps=20)
  c2["streamed_read_of_the_same_weight_bytes"] = {"us": us_read, "gb_per_s": N * K // 2 / us_read / 1e3,
                                                  "how": "qmm_stream_read over one weight copy, launched back to back like the linears"}
  # the same weights through the reference's own call: torch.ops.xla.quantized_matmul on the [S, bs, N] layout
  w_sbn = [xla_b200.unpack_int4(wp[i]).reshape(N, S, bs).permute(1, 2, 0).contiguous() for i in range(4)]
  for M in (1, 8, 32):
    x = torch.randn(M, K, generator=g, device=dev).bfloat16()
    for i in range(4):
      qmm(x, w_sbn[i], sc[i], block_size=bs, int4_weight=True)  # first use converts and caches the K-minor copy
    us = time_graph(lambda i: qmm(x, w_sbn[i % 4], sc[i % 4], block_size=bs, int4_weight=True), stream, reps=16)
    c2[f"M{M}"]["us_reference_layout_op_steady_state"] = us
  out["c2_w4a16_decode_14336x4096"] = c2
  del wp, sc, w_sbn

  # ---- configuration 1: W8A16 per-channel, x [16,4096], w [4096,4096] int8, module path ----
  N = K = 4096
  copies = 16
  mods = []
  for _ in range(copies):
    m = xla_b200.XlaQuantizedLinear(K, N, is_symmetric=True)
    m.load_quantized_weight(_rand_i8(g, dev, N, K), torch.rand(N, generator=g, device=dev) * 0.019 + 0.001)
    mods.append(m)
  x = torch.randn(16, K, generator=g, device=dev).bfloat16()
  us = time_graph(lambda i: mods[i % copies](x), stream, reps=16)
  byt = N * K + 4 * N + 2 * 16 * K + 4 * 16 * N
  out["c1_w8a16_M16_4096x4096"] = {"us": us, "gb_per_s": byt / us / 1e3, "frac_of_hbm_peak": byt / us / 1e3 / hbm,
                                   "kernel": _variant_name(8, 16, N, K, 0), "out": "f32 (type promotion of bf16 x and f32 scaler)"}
  del mods

  # ---- configuration 3: W8A8, x [2048,4096] with 1% outliers x20, w [4096,4096] ----
  M = 2048
  xs = torch.randn(M, K, generator=g, device=dev)
  xs = torch.where(torch.rand(M, K, generator=g, device=dev) < 0.01, xs * 20.0, xs).bfloat16()
  ws = [_rand_i8(g, dev, N, K) for _ in range(8)]
  sc = torch.rand(N, generator=g, device=dev) * 0.019 + 0.001
  us_op = time_graph(lambda i: torch.ops.xla.quantized_matmul_int8(xs, ws[i % 8], sc, quantize_activation=True), stream, reps=8)
  L = _capi.lib()
  xq = torch.empty((M, K), dtype=torch.int8, device=dev)
  xsc = torch.empty((M,), dtype=torch.float32, device=dev)
  y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)

  def quant(i):
    _capi.check(L.qmm_quantize_activation(_capi.ptr(xs), _capi.BF16, _capi.ptr(xq), _capi.ptr(xsc), None, M, K, 1,
                                          _capi.stream_ptr(dev)))

  def gemm(i):
    _capi.check(L.qmm_w8a8_gemm(_capi.ptr(xq), _capi.ptr(ws[i % 8]), _capi.ptr(sc), None, _capi.ptr(xsc), None, None,
                                _capi.ptr(y), _capi.BF16, M, N, K, _capi.TCGEN05, _capi.stream_ptr(dev)))

  us_q = time_graph(quant, stream, reps=8)
  us_g = time_graph(gemm, stream, reps=8)
  ops = 2.0 * M * N * K
  calib = {}
  try:  # the vendor's int8 GEMM (int32 out, no dequant epilogue) on the same shape and harness, and at 8192^3 as a peak
    us_same = time_graph(lambda i: torch._int_mm(xq, ws[i % 8].t()), stream, reps=8)
    big = 8192
    a8 = torch.randint(-127, 128, (big, big), generator=g, device=dev, dtype=torch.int8)
    b8 = torch.randint(-127, 128, (big, big), generator=g, device=dev, dtype=torch.int8)
    us_big = time_graph(lambda i: torch._int_mm(a8, b8.t()), stream, reps=2, iters=3)
    calib = {"int8_peak_tops": 2.0 * big ** 3 / us_big / 1e6, "vendor_gemm_us_same_shape": us_same,
             "vendor_gemm_tops_same_shape": ops / us_same / 1e6, "how": "cuBLASLt through torch._int_mm, CUDA-graph replays"}
    del a8, b8
  except Exception as e:
    torch.cuda.synchronize(dev)
    calib = {"int8_peak_tops": None, "how": f"torch._int_mm unavailable ({type(e).__name__})"}
  out["c3_w8a8_M2048_4096x4096"] = {
      "us_op": us_op, "us_quantize": us_q, "us_gemm": us_g, "gemm_tops": ops / us_g / 1e6,
      "gemm_frac_of_int8_peak": (ops / us_g / 1e6 / calib["int8_peak_tops"]) if calib.get("int8_peak_tops") else None,
      "gemm_frac_of_2x_bf16_burst_peak": ops / us_g / 1e6 / (2 * peaks["bf16_tflops"]), "int8_calibration": calib,
      "op_tokens_per_s": M / (us_op * 1e-6),
      "note": "int8 dense peak is not in MEASURED_PEAKS.json; it is calibrated here with the vendor GEMM"}
  del ws, xq, y

  # ---- configuration 4: one Llama-3-8B-shaped layer, int8 per-channel, bf16 out, M in {1,16,64,512} ----
  shapes = [(4096, 4096), (4096, 1024), (4096, 1024), (4096, 4096), (4096, 14336), (4096, 14336), (14336, 4096)]  # (K, N)
  layers = []
  for _ in range(2):  # two copies: 437 MB, so no weight is found in L2 again
    layers.append([(_rand_i8(g, dev, n, k), (torch.rand(n, generator=g, device=dev) * 0.019 + 0.001).bfloat16())
                   for (k, n) in shapes])
  res4 = {}
  for M in (1, 16, 64, 512):
    xk = {k: torch.randn(M, k, generator=g, device=dev).bfloat16() for k in (4096, 14336)}

    def layer(i):
      for (w, s_) in layers[i % 2]:
        qmm(xk[w.shape[1]], w, s_)  # bf16 scaler -> bf16 output

    us = time_graph(layer, stream, reps=4, iters=3)
    byt = sum(n * k + 4 * n + 2 * M * k + 2 * M * n for (k, n) in shapes)
    fl = sum(2.0 * M * n * k for (k, n) in shapes)
    res4[f"M{M}"] = {"us_per_layer": us, "layer_tokens_per_s": M / (us * 1e-6), "gb_per_s": byt / us / 1e3,
                     "frac_of_hbm_peak": byt / us / 1e3 / hbm, "tflops": fl / us / 1e6,
                     "frac_of_bf16_sustained_peak": fl / us / 1e6 / peaks["bf16_tflops_sustained"]}
  out["c4_llama8b_layer_w8a16"] = res4
  return out


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------


def run_ours(args, rank, world, local_rank):
  import torch.distributed as dist
  import xla_b200  # noqa: F401  (registers the ops; raises if the CUDA library is missing)
  from xla_b200 import _capi
  if not torch.cuda.is_available():
    raise RuntimeError("bench.py needs a CUDA device: xla_b200 has no CPU path")
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)
  peaks = measured_peaks()
  reps = args.reps
  stream = torch.cuda.Stream(device=dev)

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize(dev)

  with torch.cuda.stream(stream):
    wl = TPMlp(dev, rank, world, args.seed)
    checked = wl.check()
    barrier()
    exchange_table = wl.choose_exchanges(stream, (1, 8, 64, 512)) if world > 1 else None
    barrier()
    # M = 1 and 64: one CUDA graph of `reps` passes each (eager launches if the exchange refuses capture)
    graphs, how = {}, {}
    gph = None
    for m in MS:
      for _ in range(3):
        wl.forward(m)
    stream.synchronize()
    for m in (1, 64):
      try:
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gph, stream=stream):
          for _ in range(reps):
            wl.forward(m)
        graphs[m], how[m] = gph, "cuda graph"
      except Exception as e:
        torch.cuda.synchronize(dev)
        graphs[m], how[m] = None, f"eager launches ({type(e).__name__} during capture)"
    how[512] = "eager launches, events around every linear"
    launches_per_pass = {m: 3 + (1 if wl.exchange_for(m) in ("nccl", "peer") else 0) + (3 if m <= 64 else 0) for m in MS}

    def step(group_ev=None, lin_ev=None):
      for m in MS:
        if group_ev is not None:
          e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
          e0.record(stream)
        if graphs.get(m) is not None:
          graphs[m].replay()
        else:
          for _ in range(reps):
            wl.forward(m, events=lin_ev if m == 512 else None)
        if group_ev is not None:
          e1.record(stream)
          group_ev[m].append((e0, e1))

    for _ in range(args.warmup):
      step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
      sampler.start()
    group_ev = {m: [] for m in MS}
    lin_ev = []
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for _ in range(args.steps):
      step(group_ev, lin_ev)
    t_end.record(stream)
    barrier()
    total_ms = t_start.elapsed_time(t_end)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: host activations in, host result out, every pass ----
    hx = {m: torch.randn(m, H).bfloat16().pin_memory() for m in MS}
    hy = {m: torch.empty(m, H, dtype=torch.bfloat16).pin_memory() for m in MS}
    e2e_reps = max(1, min(reps, 4))

    # With several GPUs the host link is the scarce resource: every rank needs the whole batch, but only a 1/N
    # slice of it has to cross that rank's PCIe link - the ranks gather the slices over NVLink - and the result, which
    # is identical on all ranks after the exchange, is read by rank 0 alone.  (Bytes per step below are rank 0's.)
    def sliced(m):
      return world > 1 and m % world == 0

    def copy_in(m, dst=None):
      if not sliced(m):
        if dst is None:
          return hx[m].to(dev, non_blocking=True)
        dst.copy_(hx[m], non_blocking=True)
        return dst
      rows = m // world
      part = hx[m][rank * rows:(rank + 1) * rows].to(dev, non_blocking=True)
      full = torch.empty(m, H, dtype=torch.bfloat16, device=dev) if dst is None else dst
      dist.all_gather_into_tensor(full, part)
      return full

    def copy_out(m, y):
      if rank == 0 or not sliced(m):
        hy[m].copy_(y, non_blocking=True)

    def e2e_pass(m):
      y = wl.forward(m, x=copy_in(m))
      copy_out(m, y)

    # the small batches are launch-bound from Python: their passes (copy in, three linears, exchange, copy out) are
    # captured once and replayed, which any user of the operators can do; M = 512 is launched eagerly
    e2e_graphs = {}
    for m in (1, 64):
      try:
        for _ in range(2):
          e2e_pass(m)
        stream.synchronize()
        eg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(eg, stream=stream):
          for _ in range(e2e_reps):
            e2e_pass(m)
        e2e_graphs[m] = eg
        eg = None  # the dict holds the only reference: teardown has to be able to drop every graph
      except Exception as e:
        torch.cuda.synchronize(dev)
        print(f"[bench] end-to-end pass at M={m} not captured ({type(e).__name__}: {e}); launched eagerly", file=sys.stderr)

    # Eagerly launched passes (M = 512) move their copies to two side streams: the activations of pass r + 1 come in
    # while pass r computes, its result goes out under pass r + 1 - what a serving loop over the operators does.
    cp_in, cp_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    xin = {m: [torch.empty(m, H, dtype=torch.bfloat16, device=dev) for _ in range(2)] for m in MS if m not in e2e_graphs}
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_out_done = torch.cuda.Event()

    def e2e_passes_overlapped(m):
      for r in range(e2e_reps):
        b = r & 1
        if sliced(m):
          # the gather is a collective: it stays on the compute stream, in program order with the exchange
          with torch.cuda.stream(cp_in):
            part = hx[m][rank * (m // world):(rank + 1) * (m // world)].to(dev, non_blocking=True)
            ev_in[b].record(cp_in)
          stream.wait_event(ev_in[b])
          dist.all_gather_into_tensor(xin[m][b], part)
          part.record_stream(stream)
        else:
          with torch.cuda.stream(cp_in):
            if r >= 2:
              cp_in.wait_event(ev_free[b])  # the pass that read this buffer has finished with it
            xin[m][b].copy_(hx[m], non_blocking=True)
            ev_in[b].record(cp_in)
          stream.wait_event(ev_in[b])
        y = wl.forward(m, x=xin[m][b])
        ev_free[b].record(stream)
        ev_y = torch.cuda.Event()
        ev_y.record(stream)
        if rank == 0 or not sliced(m):
          with torch.cuda.stream(cp_out):
            cp_out.wait_event(ev_y)
            hy[m].copy_(y, non_blocking=True)
            y.record_stream(cp_out)
      ev_out_done.record(cp_out)
      stream.wait_event(ev_out_done)

    def e2e_step():
      for m in MS:
        if m in e2e_graphs:
          e2e_graphs[m].replay()
        else:
          e2e_passes_overlapped(m)
      stream.synchronize()  # every result of the step is in its host buffer

    for _ in range(3):
      e2e_step()
    barrier()
    w0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    e2e_steps = max(3, args.steps // 2)
    for _ in range(e2e_steps):
      e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), 1e3 * (time.perf_counter() - w0))
    word = _capi.device_error(dev)
    if word:
      raise RuntimeError(f"device error word {word:#x} after the timed region")

    # ---- per-batch exchange variants (N > 1) and the other configurations (N = 1) ----
    extras = {}
    if not args.headline_only:
      if world > 1:
        extras["tp_exchange_us_per_mlp"] = exchange_table
      else:
        extras["other_configs"] = other_configs(dev, stream, peaks, args.seed)

  times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
  if world > 1:
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
  total_ms, e2e_ms = times.tolist()

  if rank == 0:
    tokens = args.steps * reps * sum(MS)
    value = tokens / (total_ms * 1e-3)
    fl = F // world
    per_m = []
    for m in MS:
      ms = sum(a.elapsed_time(b) for a, b in group_ev[m]) / (len(group_ev[m]) * reps)
      byt = algorithmic_bytes(m, world)
      flops = 3 * 2.0 * m * fl * H
      per_m.append({"M": m, "us_per_mlp": ms * 1e3, "exchange": wl.exchange_for(m), "timing": how[m],
                    "kernel": _variant_name(4, m, fl, H, BS), "gb_per_s_per_gpu": byt / ms / 1e6,
                    "frac_of_hbm_peak": byt / ms / 1e6 / peaks["hbm_gbs"], "tflops_per_gpu": flops / ms / 1e9,
                    "frac_of_bf16_sustained_peak": flops / ms / 1e9 / peaks["bf16_tflops_sustained"]})
    tot = sum(r["us_per_mlp"] for r in per_m)
    for r in per_m:
      r["share_of_step"] = r["us_per_mlp"] / tot
    # the dominant kernel: the M = 512 gate / up projections, timed one by one inside the timed region
    lin_us = [a.elapsed_time(b) * 1e3 for a, b in lin_ev]
    gate_up_us = [t for i, t in enumerate(lin_us) if i % 3 != 2]
    dom_us = sum(gate_up_us) / max(1, len(gate_up_us))
    dom_flops = 2.0 * 512 * fl * H
    achieved = dom_flops / dom_us / 1e6
    e2e_tokens = e2e_steps * e2e_reps * sum(MS)
    line = {
        "metric": "qlinear_tp_mlp_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": config_dict(world, reps),
        "weight_copies_in_rotation": wl.copies,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": None,
                     "traffic_note": "DRAM bytes of this kernel: see profiles/ (ncu); not re-measured per run",
                     "peak_source": peaks["source"] + " (sustained bf16: the kernel runs inside a long step)",
                     "kernel": f"{_variant_name(4, 512, fl, H, BS)}: gate/up projection [{fl},{H}] int4 at M=512, "
                               f"{dom_us:.1f} us per launch, {len(gate_up_us)} launches timed",
                     "algorithmic_flops_per_launch": dom_flops},
        "per_batch": per_m,
        "e2e": {"value": e2e_tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": e2e_reps * sum(2 * (m // world if world > 1 and m % world == 0 else m) * H for m in MS),
                "d2h_bytes_per_step": e2e_reps * sum(2 * m * H for m in MS),
                "how": "pinned host activations in, pinned host result out, every pass; with N GPUs each rank copies in a 1/N "
                       "slice of the batch and the ranks all-gather it over NVLink, rank 0 reads the result (bytes are rank 0's)"},
        "gpu_launches": args.steps * reps * sum(launches_per_pass.values()),
        "clocks": clocks,
        "tp": {"G": world, "checked": checked},
    }
    line.update(extras)
    if not args.no_cpu_baseline and world == 1:
      line["cpu_baseline"] = cpu_sample(args.seed)
    print(json.dumps(line), flush=True)
  # The line is out.  Teardown of the process group has blocked before when something still held a captured
  # communicator; a rank that cannot finish it within half a minute leaves anyway.
  if world > 1:
    sys.stdout.flush()
    watchdog = threading.Timer(30.0, lambda: os._exit(0))
    watchdog.daemon = True
    watchdog.start()
  # captured graphs hold the communicator and the peer buffers: they go first
  graphs.clear()
  e2e_graphs.clear()
  del gph
  import gc
  gc.collect()
  torch.cuda.synchronize(dev)
  wl.close()
  if world > 1:
    dist.destroy_process_group()


def _claim_stdout():
  """Keeps stdout for the one JSON line: everything else that libraries write to fd 1 (NCCL's version
  banner, for one) goes to stderr.  Returns a file object bound to the real stdout."""
  sys.stdout.flush()
  real = os.fdopen(os.dup(1), "w")
  os.dup2(2, 1)
  return real


def main():
  global print
  real_stdout = _claim_stdout()
  _print = print

  def print(*a, **k):  # noqa: A001 - the JSON line is the only thing this program prints
    k.setdefault("file", real_stdout)
    _print(*a, **k)
    real_stdout.flush()

  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=5)
  ap.add_argument("--reps", type=int, default=8, help="MLP passes per M per step")
  ap.add_argument("--seed", type=int, default=0)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--headline-only", action="store_true", help="skip the other configurations / the exchange variants")
  args = ap.parse_args()
  args.warmup = max(args.warmup, 3)
  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  if args.impl == "reference":
    run_reference(args, rank, world)
  else:
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
  main()
