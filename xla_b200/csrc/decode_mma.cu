// Decode kernel for K-minor weights (int8 [N,K] or packed int4 [N,K/2]) and small token batches
// (M <= 32): weights go from HBM straight into registers, are dequantised there (exactly) and fed
// to warp-level tensor-core MMAs as the A operand; the activations are the B operand.  There is no
// shared-memory round trip for the weights and no single issuing thread, so the kernel is a pure
// weight stream whose only per-value cost is the integer -> bf16/f16 conversion.
//
//   out[m,n] = sum_b scale[b,n] * (sum_{k in block b} x[m,k] * w[n,k])       (per-channel: one block)
//
// Mapping.  A CTA of 4 warps owns 16 consecutive output rows n; warp w takes the K steps s = w, w+4, ...
// One step covers 64 bytes of each weight row (128 int4 or 64 int8 values): lane (g = lane/4,
// t = lane%4) loads 16 bytes of row g and of row g+8 at byte offset 16*t of the step, i.e. each lane
// owns a contiguous k span and the four lanes of a quad own the whole step.  Because the contraction
// index may be permuted freely as long as both operands agree, the lane's k span maps onto the MMA's
// k slots in whatever order the conversion produces; the lane loads the matching activations of
// token g (B operand, column g) from global memory through L1 (x is a few KB and shared by all CTAs).
// After each scale block the 16x8 partial tile is folded into fp32 accumulators with scale[b,n].
// The int4 conversion leaves a constant bias in the weights (see Bias below); it is taken out again at
// every fold with bias * sum_k x, which an extra MMA against an all-ones operand supplies.
//
// Semantics: torch_xla/experimental/xla_quantized_matmul.py:152-159 (per channel), :165-170 (blockwise).
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace qmm {

namespace {


template <typename XT>
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<XT, __half>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Bias carried by the converted weights.  The conversion drops an offset-binary nibble (v + 8) or byte
// (v + 128) under the exponent of a power of two and does NOT subtract it again; the kernel removes
// bias * sum_k x[m,k] instead, which the tensor core computes for free from the same activation
// registers (an MMA against an all-ones A operand).  Saves one packed subtract per two weights.
template <typename XT, int WBITS>
struct Bias;
template <>
struct Bias<__nv_bfloat16, 4> { static constexpr float value = 136.f; static constexpr uint32_t ones = 0x3F803F80u; };
template <>
struct Bias<__half, 4> { static constexpr float value = 1032.f; static constexpr uint32_t ones = 0x3C003C00u; };
template <>
struct Bias<__nv_bfloat16, 8> { static constexpr float value = 0.f; static constexpr uint32_t ones = 0x3F803F80u; };
template <>
struct Bias<__half, 8> { static constexpr float value = 1152.f; static constexpr uint32_t ones = 0x3C003C00u; };

// 8 nibbles (nibble i = k offset i, two's complement) -> packed pairs (k0,k1)(k2,k3)(k4,k5)(k6,k7) of
// (v + 8) + 128 in bf16 or (v + 8) + 1024 in fp16: 9 integer instructions per 8 weights.
template <typename XT>
__device__ __forceinline__ void cvt_s4x8_biased(uint32_t w, uint32_t* p) {
  constexpr bool kBf16 = !std::is_same<XT, __half>::value;
  const uint32_t lo = (w & 0x0F0F0F0Fu) ^ 0x08080808u;         // k0 k2 k4 k6, offset binary
  const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;  // k1 k3 k5 k7
  const uint32_t q0 = __byte_perm(lo, hi, 0x5140);             // k0 k1 k2 k3
  const uint32_t q1 = __byte_perm(lo, hi, 0x7362);             // k4 k5 k6 k7
  const uint32_t expo = kBf16 ? 0x43434343u : 0x64646464u;     // exponent byte of 128.0 (bf16) / 1024.0 (f16)
  p[0] = __byte_perm(q0, expo, 0x4140);
  p[1] = __byte_perm(q0, expo, 0x4342);
  p[2] = __byte_perm(q1, expo, 0x4140);
  p[3] = __byte_perm(q1, expo, 0x4342);
}

// 4 int8 -> packed pairs (k0,k1)(k2,k3).  fp16: (v + 128) + 1024, bias left in (3 instructions);
// bf16 cannot hold a byte under an exponent, so it goes through fp32 and is exact (bias 0).
template <typename XT>
__device__ __forceinline__ void cvt_s8x4_biased(uint32_t w, uint32_t* p) {
  const uint32_t u = w ^ 0x80808080u;
  if constexpr (std::is_same<XT, __half>::value) {
    p[0] = __byte_perm(u, 0x64646464u, 0x4140);
    p[1] = __byte_perm(u, 0x64646464u, 0x4342);
  } else {
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.f;
    __nv_bfloat162 a = __floats2bfloat162_rn(f0, f1), b = __floats2bfloat162_rn(f2, f3);
    p[0] = *reinterpret_cast<uint32_t*>(&a);
    p[1] = *reinterpret_cast<uint32_t*>(&b);
  }
}

// NT = number of 8-token tiles (M <= 8*NT); RG = 16-row groups per CTA (each warp converts RG groups per
// step and reuses its activation registers for all of them); WARPS = warps splitting K.
// One "fold" = the end of a scale block (blockwise) or of a single step (per-channel): the partial tile,
// minus bias * sum(x), is added into the totals.
template <int WBITS, typename XT, int NT, int RG, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
    decode_mma_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ w, const float* __restrict__ scale,
                      void* __restrict__ out, int out_dt, int M, int64_t N, int64_t K, int steps_per_block,
                      int spb_shift, int blockwise) {
  constexpr int VPS = 512 / WBITS;      // values of one weight row per step: 128 (int4) or 64 (int8)
  constexpr int VPL = VPS / 4;          // values per lane per row per step: 32 or 16
  constexpr int XREGS = VPL / 2;        // packed activation pairs per lane per token tile: 16 or 8
  constexpr int ROWS = 16 * RG;         // output rows per CTA
  constexpr float kBias = Bias<XT, WBITS>::value;
  constexpr bool kHasBias = kBias != 0.f;
  constexpr uint32_t kOnes = Bias<XT, WBITS>::ones;
  __shared__ float s_part[WARPS][ROWS][NT * 8];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int64_t n0 = (int64_t)blockIdx.x * ROWS;
  const int64_t pitch = K * WBITS / 8;
  const int steps = (int)(K / VPS);
  // lane rows: group r -> rows n0 + 16r + g and n0 + 16r + g + 8 (clamped: tail rows are computed, not stored)
  const uint8_t* wrow[2 * RG];
  const float* srow[2 * RG];
#pragma unroll
  for (int r = 0; r < 2 * RG; ++r) {
    int64_t n = n0 + 16 * (r >> 1) + g + 8 * (r & 1);
    if (n >= N) n = N - 1;
    wrow[r] = w + n * pitch + 16 * t;
    srow[r] = scale + n;
  }

  // activation row of token (8*i + g) at this lane's offset inside a step; columns beyond M stay zero
  const XT* xrow[NT];
  bool tok_ok[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int tok = 8 * i + g;
    tok_ok[i] = tok < M;
    xrow[i] = x + (int64_t)(tok_ok[i] ? tok : 0) * K + t * VPL;
  }

  float total[RG][NT][4], part[RG][NT][4], xsum[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      xsum[i][j] = 0.f;
#pragma unroll
      for (int r = 0; r < RG; ++r) total[r][i][j] = part[r][i][j] = 0.f;
    }
  const uint32_t ones[4] = {kOnes, kOnes, kOnes, kOnes};

  // Software pipeline, one step deep: the weights of this warp's next step are in flight while the
  // current step is converted and multiplied.  (Prefetching the activations as well costs 24 registers
  // and measured slower: they come from L1.)
  constexpr bool kPrefetchX = false;
  auto load_x = [&](int step, uint32_t (&dst)[NT][XREGS]) {
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const uint4* xp = reinterpret_cast<const uint4*>(xrow[i] + (int64_t)step * VPS);
#pragma unroll
      for (int q = 0; q < XREGS / 4; ++q) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok_ok[i]) v = __ldg(xp + q);
        dst[i][4 * q] = v.x;
        dst[i][4 * q + 1] = v.y;
        dst[i][4 * q + 2] = v.z;
        dst[i][4 * q + 3] = v.w;
      }
    }
  };
  int s = warp;
  uint4 wn[2 * RG];
#pragma unroll
  for (int r = 0; r < 2 * RG; ++r) {
    wn[r] = make_uint4(0, 0, 0, 0);
    if (s < steps) wn[r] = ld_stream_u4(wrow[r] + (int64_t)s * 64);
  }
  // Programmatic dependent launch: the weights are static, so their first loads may overlap the tail
  // of the previous kernel in the stream; everything that depends on that kernel (the activations)
  // and every store of this kernel come after the wait.  Both are no-ops in an ordinary launch.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  uint32_t xn[NT][XREGS];
  if (kPrefetchX && s < steps) load_x(s, xn);
  for (; s < steps; s += WARPS) {
    uint4 wc[2 * RG];
#pragma unroll
    for (int r = 0; r < 2 * RG; ++r) wc[r] = wn[r];
    uint32_t xr[NT][XREGS];
    if (kPrefetchX) {
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int q = 0; q < XREGS; ++q) xr[i][q] = xn[i][q];
    }
    const int sn = s + WARPS;
    if (sn < steps) {
#pragma unroll
      for (int r = 0; r < 2 * RG; ++r) wn[r] = ld_stream_u4(wrow[r] + (int64_t)sn * 64);
      if (kPrefetchX) load_x(sn, xn);
    }
    // fold after this step?  (blockwise: this warp's next step belongs to another block)
    bool fold = true;
    float sc[2 * RG];
#pragma unroll
    for (int r = 0; r < 2 * RG; ++r) sc[r] = 1.f;
    if (blockwise) {
      const int b = spb_shift >= 0 ? (s >> spb_shift) : (s / steps_per_block);
      const int bn = spb_shift >= 0 ? (sn >> spb_shift) : (sn / steps_per_block);
      fold = sn >= steps || bn != b;
      if (fold) {
#pragma unroll
        for (int r = 0; r < 2 * RG; ++r) sc[r] = __ldg(srow[r] + (int64_t)b * N);
      }
    }
    if (!kPrefetchX) load_x(s, xr);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      if constexpr (WBITS == 4) {
        // word wi holds k = 8*wi .. 8*wi+7 of the lane's span: two MMAs of 4 values per row
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          uint32_t pa[4], pb[4];
          cvt_s4x8_biased<XT>(reinterpret_cast<const uint32_t*>(&wc[2 * r])[wi], pa);
          cvt_s4x8_biased<XT>(reinterpret_cast<const uint32_t*>(&wc[2 * r + 1])[wi], pb);
          const uint32_t a_lo[4] = {pa[0], pb[0], pa[1], pb[1]};
          const uint32_t a_hi[4] = {pa[2], pb[2], pa[3], pb[3]};
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            mma_16816<XT>(part[r][i], a_lo, xr[i][4 * wi], xr[i][4 * wi + 1]);
            mma_16816<XT>(part[r][i], a_hi, xr[i][4 * wi + 2], xr[i][4 * wi + 3]);
          }
        }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          mma_16816<XT>(xsum[i], ones, xr[i][4 * wi], xr[i][4 * wi + 1]);
          mma_16816<XT>(xsum[i], ones, xr[i][4 * wi + 2], xr[i][4 * wi + 3]);
        }
      } else {
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          uint32_t pa[2], pb[2];
          cvt_s8x4_biased<XT>(reinterpret_cast<const uint32_t*>(&wc[2 * r])[wi], pa);
          cvt_s8x4_biased<XT>(reinterpret_cast<const uint32_t*>(&wc[2 * r + 1])[wi], pb);
          const uint32_t a[4] = {pa[0], pb[0], pa[1], pb[1]};
#pragma unroll
          for (int i = 0; i < NT; ++i) mma_16816<XT>(part[r][i], a, xr[i][2 * wi], xr[i][2 * wi + 1]);
        }
        if constexpr (kHasBias) {
#pragma unroll
          for (int i = 0; i < NT; ++i) mma_16816<XT>(xsum[i], ones, xr[i][2 * wi], xr[i][2 * wi + 1]);
        }
      }
    }
    if (fold) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          // xsum rows are all equal: c0,c1 (tokens 2t, 2t+1) serve both row g and row g+8
          const float p0 = kHasBias ? fmaf(-kBias, xsum[i][0], part[r][i][0]) : part[r][i][0];
          const float p1 = kHasBias ? fmaf(-kBias, xsum[i][1], part[r][i][1]) : part[r][i][1];
          const float p2 = kHasBias ? fmaf(-kBias, xsum[i][0], part[r][i][2]) : part[r][i][2];
          const float p3 = kHasBias ? fmaf(-kBias, xsum[i][1], part[r][i][3]) : part[r][i][3];
          total[r][i][0] = fmaf(sc[2 * r], p0, total[r][i][0]);
          total[r][i][1] = fmaf(sc[2 * r], p1, total[r][i][1]);
          total[r][i][2] = fmaf(sc[2 * r + 1], p2, total[r][i][2]);
          total[r][i][3] = fmaf(sc[2 * r + 1], p3, total[r][i][3]);
#pragma unroll
          for (int j = 0; j < 4; ++j) part[r][i][j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) xsum[i][j] = 0.f;
      }
    }
  }

  // accumulator layout of m16n8: c0,c1 -> row g, tokens 2t,2t+1; c2,c3 -> row g+8
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      s_part[warp][16 * r + g][8 * i + 2 * t] = total[r][i][0];
      s_part[warp][16 * r + g][8 * i + 2 * t + 1] = total[r][i][1];
      s_part[warp][16 * r + g + 8][8 * i + 2 * t] = total[r][i][2];
      s_part[warp][16 * r + g + 8][8 * i + 2 * t + 1] = total[r][i][3];
    }
  __syncthreads();
  for (int idx = threadIdx.x; idx < ROWS * NT * 8; idx += WARPS * 32) {
    const int row = idx % ROWS, tok = idx / ROWS;  // consecutive threads -> consecutive n
    const int64_t n = n0 + row;
    if (n < N && tok < M) {
      float v = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) v += s_part[wi][row][tok];
      if (!blockwise) v *= __ldg(scale + n);
      store_from_f32(out, (int64_t)tok * N + n, out_dt, v);
    }
  }
}

// Launch with programmatic stream serialization: this kernel may be scheduled while the previous
// kernel of the stream drains, and parks at its griddepcontrol.wait until that kernel has finished.
template <typename Kernel, typename... Args>
cudaError_t launch_pdl(Kernel kern, unsigned grid, unsigned block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int WBITS, typename XT>
int launch_nt(const void* x, const void* w, const float* scale, void* out, int out_dt, int64_t M, int64_t N,
              int64_t K, int64_t block_size, cudaStream_t st) {
  constexpr int VPS = 512 / WBITS;
  const int spb = block_size > 0 ? (int)(block_size / VPS) : 1;
  int shift = -1;
  if ((spb & (spb - 1)) == 0) {
    shift = 0;
    while ((1 << shift) < spb) ++shift;
  }
  const int bw = block_size > 0 ? 1 : 0;
  const XT* xp = reinterpret_cast<const XT*>(x);
  const uint8_t* wp = reinterpret_cast<const uint8_t*>(w);
#define QMM_DECODE_LAUNCH(NT, RG, WARPS)                                                                        \
  launch_pdl(decode_mma_kernel<WBITS, XT, NT, RG, WARPS>, (unsigned)ceil_div(N, 16 * RG), WARPS * 32, st, xp, wp, \
             scale, out, out_dt, (int)M, N, K, spb, shift, bw)
  // measured on B200 (w [14336,4096] int4): 16 rows per CTA is best for one token tile; with two or four
  // tiles the activation traffic through L1 dominates and 32 rows per CTA (activation registers reused
  // for two row groups) wins
  cudaError_t err;
  if (M <= 8)
    err = QMM_DECODE_LAUNCH(1, 1, 4);
  else if (M <= 16)
    err = QMM_DECODE_LAUNCH(2, 2, 4);
  else
    err = QMM_DECODE_LAUNCH(4, 2, 4);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_LAUNCH, "decode_mma_kernel launch: %s", cudaGetErrorString(err));
  }
#undef QMM_DECODE_LAUNCH
  return check_launch("decode_mma_kernel");
}

}  // namespace

bool decode_mma_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x, int x_dt,
                          const void* w, bool has_zp) {
  if (has_zp) return false;
  if (x_dt != QMM_BF16 && x_dt != QMM_F16) return false;
  if (M < 1 || M > 32 || N < 1 || K < 1) return false;
  const int vps = 512 / wbits;
  if (K % vps != 0) return false;                                 // whole 64-byte steps per weight row
  if (block_size > 0 && block_size % vps != 0) return false;      // a step stays inside one scale block
  if (!aligned(x, 16) || !aligned(w, 16)) return false;
  if (ceil_div(N, 16) > 2147483647LL) return false;
  return true;
}

int launch_decode_mma(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt,
                      int64_t M, int64_t N, int64_t K, int64_t block_size, cudaStream_t st) {
  if (!decode_mma_supported(wbits, M, N, K, block_size, x, x_dt, w, false))
    return fail(QMM_ERR_UNSUPPORTED,
                "decode kernel: needs bf16/f16 activations, 1<=M<=32, K a multiple of %d, block_size a multiple of %d, "
                "16-byte aligned x/w, no zero point (M=%lld N=%lld K=%lld bs=%lld)",
                512 / wbits, 512 / wbits, (long long)M, (long long)N, (long long)K, (long long)block_size);
  if (wbits == 4) {
    if (x_dt == QMM_BF16) return launch_nt<4, __nv_bfloat16>(x, w, scale, out, out_dt, M, N, K, block_size, st);
    return launch_nt<4, __half>(x, w, scale, out, out_dt, M, N, K, block_size, st);
  }
  if (x_dt == QMM_BF16) return launch_nt<8, __nv_bfloat16>(x, w, scale, out, out_dt, M, N, K, block_size, st);
  return launch_nt<8, __half>(x, w, scale, out, out_dt, M, N, K, block_size, st);
}

}  // namespace qmm
