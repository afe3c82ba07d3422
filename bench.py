"""Benchmark of the weight-quantized linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c2|c3|c1|c4]

Workload (default, N=1): the decode configuration the headline metric is quoted on - W4A16 blockwise
int4, w [14336, 4096] packed two per byte along K, block 128, scaler fp32 [32, 14336], x bf16 [M, 4096]
for M in {1, 8, 32}, bf16 output.  One STEP = `--reps` launches of the op for each M, every launch on
a different copy of the weights (a pool larger than L2), so no launch finds its weights in L2.

  value      tokens/s with inputs resident in HBM, timed with CUDA events around the K steps
             (steps are CUDA-graph replays, so launch latency of the Python layer is not in it).
  roofline   the dominant kernel's algorithmic bytes per launch / its average launch duration (CUDA
             events around each M's group of launches inside the timed region) vs the measured HBM peak.
  e2e        same metric through the public host-buffer API (xla_b200.HostPipeline: one library call per
             linear does copy-in, kernel and copy-out): pinned-host activations in, result in pinned host
             memory out, inside the timed region, every call; wall clock and CUDA events, the larger counts.
  cpu_baseline  the reference's CPU path (oracle/torch_port.py, same ATen operators) on the host
             cores, on a bounded sample.

With --gpus N > 1 every rank runs the same step on its own token batch (data-parallel replicas of the
weights, no collective on the data path): "scaling": "weak".  The tensor-parallel MLP (column- and
row-sharded, NCCL all-reduce on the row-parallel output) is reported under "tp" on the same line.
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
# workloads
# ------------------------------------------------------------------------------------------------


class C2Decode:
  """W4A16 blockwise decode GEMV: w int4 [14336,4096] packed, block 128, M in {1,8,32}."""
  name = "W4A16 blockwise int4 decode: w[14336,4096] packed, block 128, scaler f32 [32,14336], x bf16 [M,4096], M in {1,8,32}, bf16 out"
  N, K, BS = 14336, 4096, 128
  MS = (1, 8, 32)
  dtype = "bf16 activations x int4 weights, fp32 accumulate"

  def __init__(self, device, seed):
    import xla_b200
    self.dev = device
    g = torch.Generator(device=device).manual_seed(seed)
    S = self.K // self.BS
    per_copy = self.N * self.K // 2 + S * self.N * 4
    self.copies = max(2, -(-2 * L2_BYTES // per_copy))  # pool >= 2 x L2
    self.wp = [torch.randint(0, 256, (self.N, self.K // 2), generator=g, device=device, dtype=torch.uint8)
               for _ in range(self.copies)]
    self.scale = [(torch.rand(S, self.N, generator=g, device=device) * 0.045 + 0.005) for _ in range(self.copies)]
    self.x = {m: torch.randn(m, self.K, generator=g, device=device).bfloat16() for m in self.MS}
    self.op = torch.ops.xla_b200.quantized_matmul_packed
    self._i = 0

  def bytes_per_launch(self, m):
    S = self.K // self.BS
    return self.N * self.K // 2 + 4 * S * self.N + 2 * m * self.K + 2 * m * self.N

  def flops_per_launch(self, m):
    return 2 * m * self.N * self.K

  def launch(self, m, x=None):
    i = self._i = (self._i + 1) % self.copies
    return self.op(self.x[m] if x is None else x, self.wp[i], self.scale[i], block_size=self.BS, int4_weight=True,
                   weight_is_packed=True, out_dtype=torch.bfloat16)

  forced = "auto"  # kernel family forced with --variant

  def tokens_per_step(self, reps):
    return reps * sum(self.MS)


def variant_name(m, N, K, bs):
  from xla_b200 import _capi
  if C2Decode.forced != "auto":
    return C2Decode.forced
  return _capi.lib().qmm_variant_for(_capi.OP_W4A16_BLOCKWISE_PACKED, m, N, K, bs, 0).decode()


# ------------------------------------------------------------------------------------------------
# CPU baseline (reference CPU path restated with the same ATen operators)
# ------------------------------------------------------------------------------------------------


def cpu_baseline_c2(seed, budget_s=12.0):
  from oracle import torch_port as tp
  cores = os.cpu_count() or 1
  torch.set_num_threads(cores)
  g = torch.Generator().manual_seed(seed)
  N, K, BS = C2Decode.N, C2Decode.K, C2Decode.BS
  S = K // BS
  # the reference keeps int4 unpacked, [S, bs, N] int8; it needs fp32 activations with an fp32 scaler
  w = torch.randint(-8, 8, (S, BS, N), generator=g, dtype=torch.int8)
  sc = torch.rand(S, N, generator=g) * 0.045 + 0.005
  xs = {m: torch.randn(m, K, generator=g) for m in C2Decode.MS}
  for m in C2Decode.MS:  # warm-up
    tp.quantized_matmul_cpu(xs[m], w, sc, block_size=BS)
  t0 = time.perf_counter()
  passes = 0
  while True:
    for m in C2Decode.MS:
      tp.quantized_matmul_cpu(xs[m], w, sc, block_size=BS)
    passes += 1
    if time.perf_counter() - t0 > budget_s or passes >= 50:
      break
  dt = time.perf_counter() - t0
  return {"value": passes * sum(C2Decode.MS) / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
          "sample": f"{passes} passes of M in (1,8,32) on the full [14336,4096] weight in the reference's unpacked "
                    f"[32,128,14336] int8 layout, fp32 activations, {dt:.1f} s wall",
          "threads": torch.get_num_threads()}


# ------------------------------------------------------------------------------------------------
# the other benchmark configurations (reported beside the headline, N=1 only) and the TP MLP
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


def other_configs(dev, stream, peaks, seed):
  """Per-configuration kernel timings: W8A16 decode (config 1), W8A8 prefill (config 3), the
  Llama-3-8B-shaped layer (config 4) and the 70B-shaped MLP on one GPU (config 5)."""
  import xla_b200
  from xla_b200 import _capi
  g = torch.Generator(device=dev).manual_seed(seed + 100)
  qmm = torch.ops.xla.quantized_matmul
  packed = torch.ops.xla_b200.quantized_matmul_packed
  out = {}
  hbm = peaks["hbm_gbs"]

  # ---- config 1: W8A16 per-channel, x [16,4096], w [4096,4096] int8, module path ----
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
                                   "kernel": _capi.lib().qmm_variant_for(_capi.OP_W8A16_PERCHANNEL, 16, N, K, 0, 0).decode(),
                                   "out": "f32 (type promotion of bf16 x and f32 scaler)"}
  del mods

  # ---- config 3: W8A8, x [2048,4096] with 1% outliers x20, w [4096,4096] ----
  M = 2048
  xs = torch.randn(M, K, generator=g, device=dev)
  xs = torch.where(torch.rand(M, K, generator=g, device=dev) < 0.01, xs * 20.0, xs).bfloat16()
  ws = [_rand_i8(g, dev, N, K) for _ in range(8)]
  sc = torch.rand(N, generator=g, device=dev) * 0.019 + 0.001
  us_op = time_graph(lambda i: torch.ops.xla.quantized_matmul_int8(xs, ws[i % 8], sc, quantize_activation=True), stream,
                     reps=8)
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

  # int8 calibration with the vendor library (cuBLASLt through torch._int_mm): an 8192^3 burst as the int8
  # "measured peak" (MEASURED_PEAKS.json has none), and the same C3 shape for a like-for-like comparison
  def best_us(fn, n=10):
    best = float("inf")
    with torch.cuda.stream(stream):
      for _ in range(3):
        fn()
      for _ in range(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn()
        e1.record(stream)
        stream.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3)
    return best

  calib = {}
  try:
    big = 8192
    a8 = torch.randint(-127, 128, (big, big), generator=g, device=dev, dtype=torch.int8)
    b8 = torch.randint(-127, 128, (big, big), generator=g, device=dev, dtype=torch.int8)
    us_big = best_us(lambda: torch._int_mm(a8, b8.t()))
    try:  # same harness as our GEMM: graph replays over the rotating weight copies
      us_same = time_graph(lambda i: torch._int_mm(xq, ws[i % 8].t()), stream, reps=8)
      same_how = "graph replays over the same 8 rotating weight copies"
    except Exception:
      torch.cuda.synchronize(dev)
      us_same = best_us(lambda: torch._int_mm(xq, ws[0].t()), n=20)
      same_how = "best of 20 eager calls on one weight copy (L2-warm)"
    calib = {"int8_peak_tops": 2.0 * big ** 3 / us_big / 1e6, "vendor_gemm_us_same_shape": us_same,
             "vendor_gemm_tops_same_shape": ops / us_same / 1e6,
             "how": "cuBLASLt int8 GEMM (int32 out, no dequant epilogue) via torch._int_mm: best of 10 at 8192^3 "
                    "(peak); at the C3 shape " + same_how}
    del a8, b8
  except Exception as e:  # an int8 GEMM the library refuses is only a missing denominator
    calib = {"int8_peak_tops": None, "how": f"torch._int_mm unavailable ({type(e).__name__})"}
  out["c3_w8a8_M2048_4096x4096"] = {
      "us_op": us_op, "us_quantize": us_q, "us_gemm": us_g, "gemm_tops": ops / us_g / 1e6,
      "gemm_frac_of_int8_peak": (ops / us_g / 1e6 / calib["int8_peak_tops"]) if calib.get("int8_peak_tops") else None,
      "gemm_frac_of_2x_bf16_burst_peak": ops / us_g / 1e6 / (2 * peaks["bf16_tflops"]),
      "int8_calibration": calib,
      "quantize_gb_per_s": 3.0 * M * K / us_q / 1e3, "op_tokens_per_s": M / (us_op * 1e-6),
      "note": "int8 dense peak is not in MEASURED_PEAKS.json; it is calibrated here with the vendor GEMM"}
  del ws, xq, y

  # ---- config 4: one Llama-3-8B-shaped layer, int8 per-channel, bf16 out, M in {1,16,64,512} ----
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
                     "kernel": _capi.lib().qmm_variant_for(_capi.OP_W8A16_PERCHANNEL, M, 4096, 4096, 0, 0).decode()}
  out["c4_llama8b_layer_w8a16"] = res4
  del layers

  # ---- config 5 on one GPU: 70B-shaped MLP, W4A16 blockwise 128, M in {1,64,512} ----
  out["c5_llama70b_mlp_w4a16_G1"] = tp_mlp_times(dev, stream, g, world=1, rank=0, peaks=peaks)
  return out


def tp_mlp_times(dev, stream, g, world, rank, peaks, Ms=(1, 64, 512)):
  """gate/up [28672/G, 8192] column-sharded, down [8192, 28672/G] row-sharded + all-reduce (bf16)."""
  import torch.distributed as dist
  from xla_b200 import tensor_parallel as tp
  H, F, BS = 8192, 28672, 128
  fl_, hl = F // world, H
  mk = lambda n, k: torch.randint(0, 256, (n, k // 2), generator=g, device=dev, dtype=torch.uint8)
  mks = lambda k, n: torch.rand(k // BS, n, generator=g, device=dev) * 0.045 + 0.005
  gate_w, up_w, down_w = mk(fl_, H), mk(fl_, H), mk(hl, fl_)
  gate_s, up_s, down_s = mks(H, fl_), mks(H, fl_), mks(fl_, hl)
  op = torch.ops.xla_b200.quantized_matmul_packed
  res = {}
  gu = None
  peers = fused = None
  if world > 1:
    try:
      from xla_b200 import peer_reduce
      peers = peer_reduce.PeerAllReduce(max_elems=32 * hl)
      fused = peer_reduce.FusedRowParallelDecode(N=hl, max_M=8)
    except Exception as e:
      print(f"[bench] peer-memory all-reduce unavailable ({type(e).__name__}: {e})", file=sys.stderr)
  for M in Ms:
    x = torch.randn(M, H, generator=g, device=dev).bfloat16()

    def mlp(i):
      a = op(x, gate_w, gate_s, block_size=BS, int4_weight=True, weight_is_packed=True, out_dtype=torch.bfloat16)
      b = op(x, up_w, up_s, block_size=BS, int4_weight=True, weight_is_packed=True, out_dtype=torch.bfloat16)
      del a  # gate*up is not part of the configuration: the three linears and the all-reduce are timed
      y = op(b, down_w, down_s, block_size=BS, int4_weight=True, weight_is_packed=True, out_dtype=torch.bfloat16)
      if world > 1:
        dist.all_reduce(y)
      return y

    try:
      us = time_graph(mlp, stream, reps=4, iters=3)
      how = "cuda graph"
    except Exception as e:  # graph capture of the collective refused: time eager launches instead
      torch.cuda.synchronize(dev)
      with torch.cuda.stream(stream):
        for i in range(3):
          mlp(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(10):
          mlp(i)
        e1.record(stream)
        stream.synchronize()
      us = e0.elapsed_time(e1) * 1e3 / 10
      how = f"eager launches ({type(e).__name__} during capture)"
    if world > 1:
      t = torch.tensor([us], dtype=torch.float64, device=dev)
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
      us = float(t.item())
    byt = 3 * (fl_ * H // 2) + 4 * (2 * (H // BS) * fl_ + (fl_ // BS) * hl) + 2 * M * (2 * H + 3 * fl_ + hl)
    res[f"M{M}"] = {"us_per_mlp": us, "tokens_per_s": M / (us * 1e-6), "gb_per_s_per_gpu": byt / us / 1e3,
                    "frac_of_hbm_peak": byt / us / 1e3 / peaks["hbm_gbs"],
                    "tflops_per_gpu": 3 * 2.0 * M * fl_ * H / us / 1e6, "timing": how}
    if M <= 32 and fl_ % 8 == 0:
      # the same MLP with gate, up and silu(gate) * up in one kernel (one weight stream of 2 * F/G rows)
      if gu is None:
        import xla_b200
        gu = xla_b200.interleave_gate_up(gate_w, up_w, gate_s, up_s, BS)

      def mlp_fused(i):
        h = torch.ops.xla_b200.quantized_gate_up(x, gu[0], gu[1], block_size=BS, int4_weight=True, weight_is_packed=True,
                                                 out_dtype=torch.bfloat16)
        y = op(h, down_w, down_s, block_size=BS, int4_weight=True, weight_is_packed=True, out_dtype=torch.bfloat16)
        if world > 1:
          dist.all_reduce(y)
        return y

      try:
        usf = time_graph(mlp_fused, stream, reps=4, iters=3)
        if world > 1:
          t = torch.tensor([usf], dtype=torch.float64, device=dev)
          dist.all_reduce(t, op=dist.ReduceOp.MAX)
          usf = float(t.item())
        res[f"M{M}"]["us_per_mlp_fused_gate_up"] = usf
      except Exception as e:
        res[f"M{M}"]["us_per_mlp_fused_gate_up"] = f"not measured ({type(e).__name__})"
      if world > 1 and peers is not None and peers.fits(M, hl):
        # and with the down projection's partial results summed by the one-shot peer-memory kernel
        from xla_b200 import packed as _packed

        def mlp_peer(i):
          h = torch.ops.xla_b200.quantized_gate_up(x, gu[0], gu[1], block_size=BS, int4_weight=True, weight_is_packed=True,
                                                   out_dtype=torch.bfloat16)
          _packed.quantized_matmul_packed(h, down_w, down_s, block_size=BS, int4_weight=True, weight_is_packed=True,
                                          out_dtype=torch.float32, out=peers.partial_view(M, hl))
          return peers.reduce(M, hl, torch.bfloat16)

        try:
          usp = time_graph(mlp_peer, stream, reps=4, iters=3)
          t = torch.tensor([usp], dtype=torch.float64, device=dev)
          dist.all_reduce(t, op=dist.ReduceOp.MAX)
          res[f"M{M}"]["us_per_mlp_fused_gate_up_peer_allreduce"] = float(t.item())
        except Exception as e:
          res[f"M{M}"]["us_per_mlp_fused_gate_up_peer_allreduce"] = f"not measured ({type(e).__name__}: {e})"
      if world > 1 and fused is not None and fused.fits(M, hl):
        # two kernels per MLP: gate+up+silu, then the down projection whose epilogue also sums over the ranks
        def mlp_two(i):
          h = torch.ops.xla_b200.quantized_gate_up(x, gu[0], gu[1], block_size=BS, int4_weight=True, weight_is_packed=True,
                                                   out_dtype=torch.bfloat16)
          return fused(h, down_w, down_s, block_size=BS, weight_is_packed=True, out_dtype=torch.bfloat16)

        try:
          us2 = time_graph(mlp_two, stream, reps=4, iters=3)
          t = torch.tensor([us2], dtype=torch.float64, device=dev)
          dist.all_reduce(t, op=dist.ReduceOp.MAX)
          res[f"M{M}"]["us_per_mlp_fused_gate_up_fused_allreduce"] = float(t.item())
        except Exception as e:
          res[f"M{M}"]["us_per_mlp_fused_gate_up_fused_allreduce"] = f"not measured ({type(e).__name__}: {e})"
  if peers is not None:
    peers.close()
  if fused is not None:
    fused.close()
  return res


# ------------------------------------------------------------------------------------------------
# arms
# ------------------------------------------------------------------------------------------------


def run_reference(args, rank, world):
  if rank != 0:
    return
  t0 = time.perf_counter()
  per_step = []
  base = None
  for i in range(args.warmup + args.steps):
    base = cpu_baseline_c2(args.seed, budget_s=1.0 if i < args.warmup else max(1.0, min(6.0, 60.0 / args.steps)))
    if i >= args.warmup:
      per_step.append(base["value"])
  value = sum(per_step) / len(per_step)
  base["value"] = value
  line = {"impl": "reference", "metric": "qlinear_decode_tokens_per_s", "value": value, "unit": "tokens/s",
          "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
          "ms_per_step": 1e3 * (time.perf_counter() - t0) / max(1, args.steps + args.warmup),
          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations x int8-held int4",
          "data": "synthetic", "config": {"workload": C2Decode.name, "flush": "n/a (CPU)"},
          "cpu_baseline": base, "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
  print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
  import torch.distributed as dist
  import xla_b200  # noqa: F401  (registers the ops; raises if the CUDA library is missing)
  if not torch.cuda.is_available():
    raise RuntimeError("bench.py needs a CUDA device: xla_b200 has no CPU path")
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)
  peaks = measured_peaks()
  wl = C2Decode(dev, args.seed + rank)
  if args.variant != "auto":
    import xla_b200.quantized_matmul as _qm_mod
    C2Decode.forced = args.variant
    _qm_mod._variant = args.variant  # what xla_b200.force_variant sets, for the whole run
  reps = args.reps
  stream = torch.cuda.Stream(device=dev)

  # one CUDA graph per M: `reps` launches on rotating weight copies
  graphs = {}
  with torch.cuda.stream(stream):
    for m in wl.MS:
      for _ in range(3):
        wl.launch(m)
    stream.synchronize()
    for m in wl.MS:
      gph = torch.cuda.CUDAGraph()
      with torch.cuda.graph(gph, stream=stream):
        for _ in range(reps):
          wl.launch(m)
      graphs[m] = gph
  launches_per_step = reps * len(wl.MS)

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize(dev)

  def step(events=None):
    for m in wl.MS:
      if events is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
      graphs[m].replay()
      if events is not None:
        e1.record(stream)
        events[m].append((e0, e1))

  with torch.cuda.stream(stream):
    for _ in range(args.warmup):
      step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
      sampler.start()
    per_m = {m: [] for m in wl.MS}
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for _ in range(args.steps):
      step(per_m)
    t_end.record(stream)
    barrier()
    total_ms = t_start.elapsed_time(t_end)

    # ---- end to end through the public host-buffer API: host activations in, host result out, every call ----
    # xla_b200.HostPipeline does the copy-in, the linear and the copy-out of a call with ONE call into the
    # library, on three streams of its own (the copies of neighbouring calls overlap the kernel).  The weights
    # rotate through the same pool as in the device-resident timing.
    import xla_b200
    hx = {m: torch.randn(m, wl.K).bfloat16().pin_memory() for m in wl.MS}
    e2e_reps = max(1, min(reps, 8))
    hy = {m: [torch.empty(m, wl.N, dtype=torch.bfloat16).pin_memory() for _ in range(e2e_reps)] for m in wl.MS}
    pipe = xla_b200.HostPipeline(max_M=max(wl.MS), K=wl.K, N=wl.N, depth=8, device=dev)
    host_lin = [pipe.linear(wl.wp[i], wl.scale[i], block_size=wl.BS, weight_is_packed=True, variant=wl.forced)
                for i in range(wl.copies)]
    e2e_i = [0]

    def e2e_step():
      i = e2e_i[0]
      for m in wl.MS:
        x_host, outs = hx[m], hy[m]
        for r in range(e2e_reps):
          i = i + 1 if i + 1 < wl.copies else 0
          host_lin[i](x_host, outs[r])
      e2e_i[0] = i
      pipe.synchronize()  # every result of the step is in its host buffer

    for _ in range(max(3, args.warmup)):
      e2e_step()
    barrier()
    w0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
      e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), 1e3 * (time.perf_counter() - w0))
    # the last host result of the last step against the device operator on the same inputs
    m_last, i_last = wl.MS[-1], e2e_i[0]
    ref = wl.op(hx[m_last].to(dev), wl.wp[i_last], wl.scale[i_last], block_size=wl.BS, int4_weight=True,
                weight_is_packed=True, out_dtype=torch.bfloat16)
    if not torch.equal(ref.cpu(), hy[m_last][e2e_reps - 1]):
      raise RuntimeError("end-to-end result differs from the device operator")
    pipe.close()
  clocks = sampler.stop() if rank == 0 else None
  extras = {}
  if not args.headline_only:
    g2 = torch.Generator(device=dev).manual_seed(args.seed + 7)
    if world == 1:
      extras["other_configs"] = other_configs(dev, stream, peaks, args.seed)
    else:
      extras["tp"] = {"config": "Llama-3-70B-shaped MLP, W4A16 block 128: gate/up [28672/G,8192] column-sharded, down "
                                "[8192,28672/G] row-sharded, NCCL all-reduce of the bf16 output; scaling: strong",
                      "G": world, "results": tp_mlp_times(dev, stream, g2, world, rank, peaks)}

  times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
  if world > 1:
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
  total_ms, e2e_ms = times.tolist()

  if rank == 0:
    tokens = world * args.steps * wl.tokens_per_step(reps)
    value = tokens / (total_ms * 1e-3)
    per_kernel = []
    for m in wl.MS:
      ms = sum(a.elapsed_time(b) for a, b in per_m[m]) / (len(per_m[m]) * reps)
      gbs = wl.bytes_per_launch(m) / (ms * 1e-3) / 1e9
      per_kernel.append({"M": m, "kernel": variant_name(m, wl.N, wl.K, wl.BS), "us_per_launch": ms * 1e3,
                         "algorithmic_bytes": wl.bytes_per_launch(m), "gb_per_s": gbs,
                         "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "tflops": wl.flops_per_launch(m) / (ms * 1e-3) / 1e12})
    dom = max(per_kernel, key=lambda r: r["us_per_launch"])
    # dram__bytes_read.sum + dram__bytes_write.sum per launch of the headline kernel, from the ncu captures
    # summarised in profiles/decode_mma_kernel__w4a16_decode_14336x4096.md (the writes are below 0.1 MB:
    # the bf16 output is still in L2 when the kernel ends)
    ncu_traffic = {1: 31.21e6, 8: 31.27e6, 32: 31.48e6}
    e2e_tokens = world * args.steps * e2e_reps * sum(wl.MS)
    line = {
        "metric": "qlinear_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.name, "launches_per_step": launches_per_step, "reps_per_M": reps,
                   "flush": f"weights rotate through a pool of {wl.copies} copies ({wl.copies * wl.bytes_per_launch(1) / 2**20:.0f} MiB > L2)",
                   "parallelism": f"dp{world} replicas (no data-path collective)" if world > 1 else "single GPU",
                   "timing": "CUDA events on the launch stream; steps are CUDA-graph replays"},
        "roofline": {"bound": "hbm", "achieved": dom["gb_per_s"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": dom["gb_per_s"] / peaks["hbm_gbs"],
                     "traffic": ncu_traffic.get(dom["M"]) if dom["kernel"] == "mma" else None,
                     "peak_source": peaks["source"],
                     "kernel": f"{dom['kernel']} M={dom['M']}"},
        "per_kernel": per_kernel,
        "e2e": {"value": e2e_tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": e2e_reps * sum(2 * m * wl.K for m in wl.MS),
                "d2h_bytes_per_step": e2e_reps * sum(2 * m * wl.N for m in wl.MS)},
        "gpu_launches": args.steps * launches_per_step,
        "clocks": clocks,
    }
    line.update(extras)
    if not args.no_cpu_baseline and world == 1:
      line["cpu_baseline"] = cpu_baseline_c2(args.seed)
    print(json.dumps(line), flush=True)
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
  ap.add_argument("--reps", type=int, default=20, help="launches per M per step")
  ap.add_argument("--seed", type=int, default=0)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--headline-only", action="store_true", help="skip the other configurations / the TP MLP")
  ap.add_argument("--variant", default="auto", choices=["auto", "generic", "gemv", "tcgen05", "mma", "tmem"],
                  help="force one kernel family for the headline workload (profiling a non-default kernel); "
                       "the default lets the library choose by shape")
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
