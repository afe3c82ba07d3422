// Decode (small-M) kernels for weights stored K-minor: int8 [N,K] or packed int4 [N,K/2].
//
// The work is HBM-bound: every weight byte is read exactly once with 128-bit streaming loads,
// dequantised in registers and multiplied into fp32 accumulators; the scale is applied to the
// finished dot product (per channel) or to each finished 128-bit slice of a block (blockwise),
// never to the weights, so the integer -> float conversion is exact.
//
// Mapping.  A CTA of 4 warps owns kRows = 8 consecutive output rows n.  A weight row is cut into
// 16-byte lane slices (16 int8 or 32 int4 values); slice q belongs to warp (q / 32) % 4, lane
// q % 32.  Each lane therefore has 8 independent 16-byte loads in flight per step (one per row)
// and reuses its activation slice for all 8 rows.  Partial sums meet in a warp-shuffle
// reduction and one pass through shared memory.
//
// Semantics: torch_xla/experimental/xla_quantized_matmul.py:139-183 (per channel: :152-159,
// blockwise: :165-170, zero point: :172-180).
#include "common.cuh"
#include "kernels.h"

namespace qmm {

namespace {

constexpr int kRows = 8;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

// 4 int8 values of a 32-bit word -> fp32, exact.  XOR turns two's complement into offset
// binary; byte_perm drops each byte into the mantissa of 2^23, and one subtraction removes
// 2^23 + 128.
__device__ __forceinline__ void dequant_s8x4(uint32_t w, float* f) {
  const uint32_t u = w ^ 0x80808080u;
  f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.f;
  f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.f;
  f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.f;
  f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.f;
}

// 8 int4 values of a 32-bit word (nibble i = k offset i) -> fp32, exact.  Each masked pair of
// nibbles is OR-ed into the mantissa of fp16 1024.0; the low nibble of a byte then reads
// 1024 + u, the high nibble 1024 + 16u, and one half2 operation each removes the bias.
__device__ __forceinline__ void dequant_s4x8(uint32_t w, float* f) {
  const uint32_t u = w ^ 0x88888888u;
  const uint32_t u2 = u >> 8;
  const uint32_t t0 = (u & 0x000F000Fu) | 0x64006400u;
  const uint32_t t1 = (u & 0x00F000F0u) | 0x64006400u;
  const uint32_t t2 = (u2 & 0x000F000Fu) | 0x64006400u;
  const uint32_t t3 = (u2 & 0x00F000F0u) | 0x64006400u;
  const __half2 bias_lo = __floats2half2_rn(1032.f, 1032.f);
  const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 bias_hi = __floats2half2_rn(-72.f, -72.f);
  const __half2 h0 = __hsub2(*reinterpret_cast<const __half2*>(&t0), bias_lo);
  const __half2 h1 = __hfma2(*reinterpret_cast<const __half2*>(&t1), sixteenth, bias_hi);
  const __half2 h2 = __hsub2(*reinterpret_cast<const __half2*>(&t2), bias_lo);
  const __half2 h3 = __hfma2(*reinterpret_cast<const __half2*>(&t3), sixteenth, bias_hi);
  const float2 a0 = __half22float2(h0), a1 = __half22float2(h1);
  const float2 a2 = __half22float2(h2), a3 = __half22float2(h3);
  f[0] = a0.x; f[4] = a0.y;
  f[1] = a1.x; f[5] = a1.y;
  f[2] = a2.x; f[6] = a2.y;
  f[3] = a3.x; f[7] = a3.y;
}

// 8 consecutive activations -> fp32
template <typename XT>
__device__ __forceinline__ void load_x8(const XT* p, float* f);

template <>
__device__ __forceinline__ void load_x8<float>(const float* p, float* f) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <>
__device__ __forceinline__ void load_x8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(r[i] << 16);
    f[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
  }
}

template <>
__device__ __forceinline__ void load_x8<__half>(const __half* p, float* f) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&r[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// WBITS: 8 or 4.  BLOCKWISE: scale/zp are [S,N] and apply per K block; else [N].
// MT: compile-time bound on the number of activation rows (runtime M <= MT).
template <int WBITS, bool BLOCKWISE, typename XT, int MT>
__global__ void __launch_bounds__(kThreads)
    gemv_nk_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ w,
                   const float* __restrict__ scale, const float* __restrict__ zp,
                   void* __restrict__ out, int out_dt, int M, int64_t N, int64_t K,
                   int block_size) {
  constexpr int VALS = 128 / WBITS;  // weights per 16-byte lane slice
  constexpr int NSUB = VALS / 8;     // groups of 8 values
  __shared__ float s_acc[kWarps][kRows][MT];
  __shared__ float s_xs[kWarps][MT];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t n0 = (int64_t)blockIdx.x * kRows;
  const int64_t pitch = K * WBITS / 8;  // bytes per weight row
  const int64_t nslices = pitch >> 4;

  float acc[kRows][MT];
  float xs_tot[MT];  // per-channel zero point: sum of the activations this lane has seen
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
#pragma unroll
  for (int m = 0; m < MT; ++m) xs_tot[m] = 0.f;

  const uint8_t* wrow[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const int64_t n = (n0 + r < N) ? n0 + r : N - 1;  // clamp: tail rows are computed, not stored
    wrow[r] = w + n * pitch;
  }

  for (int64_t q = (int64_t)warp * 32 + lane; q < nslices; q += kThreads) {
    uint4 wv[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) wv[r] = ld_stream_u4(wrow[r] + (q << 4));
    const int64_t k0 = q * VALS;

    float sc[kRows], zz[kRows];
    if (BLOCKWISE) {
      const int64_t b = k0 / block_size;
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const int64_t n = (n0 + r < N) ? n0 + r : N - 1;
        sc[r] = __ldg(scale + b * N + n);
        zz[r] = zp ? __ldg(zp + b * N + n) : 0.f;
      }
    }

#pragma unroll
    for (int sub = 0; sub < NSUB; ++sub) {
      float xf[MT][8];
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const int mm = (m < M) ? m : M - 1;
        load_x8<XT>(x + (int64_t)mm * K + k0 + sub * 8, xf[m]);
      }
      if (zp) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float s8 = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) s8 += xf[m][j];
          if (BLOCKWISE) {
#pragma unroll
            for (int r = 0; r < kRows; ++r) acc[r][m] = fmaf(-s8, zz[r], acc[r][m]);
          } else {
            xs_tot[m] += s8;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        float wf[8];
        const uint32_t* words = reinterpret_cast<const uint32_t*>(&wv[r]);
        if (WBITS == 8) {
          dequant_s8x4(words[2 * sub], wf);
          dequant_s8x4(words[2 * sub + 1], wf + 4);
        } else {
          dequant_s4x8(words[sub], wf);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (BLOCKWISE) {
            float p = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) p = fmaf(wf[j], xf[m][j], p);
            acc[r][m] = fmaf(sc[r], p, acc[r][m]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[r][m] = fmaf(wf[j], xf[m][j], acc[r][m]);
          }
        }
      }
    }
  }

  // warp reduction, then one trip through shared memory across the 4 warps
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float v = warp_sum(acc[r][m]);
      if (lane == 0) s_acc[warp][r][m] = v;
    }
  if (!BLOCKWISE && zp) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float v = warp_sum(xs_tot[m]);
      if (lane == 0) s_xs[warp][m] = v;
    }
  }
  __syncthreads();
  const int t = threadIdx.x;
  if (t < kRows * MT) {
    const int r = t % kRows, m = t / kRows;  // consecutive threads -> consecutive n
    const int64_t n = n0 + r;
    if (n < N && m < M) {
      float v = 0.f;
#pragma unroll
      for (int wi = 0; wi < kWarps; ++wi) v += s_acc[wi][r][m];
      if (!BLOCKWISE) {
        v *= __ldg(scale + n);
        if (zp) {
          float xs = 0.f;
#pragma unroll
          for (int wi = 0; wi < kWarps; ++wi) xs += s_xs[wi][m];
          v = fmaf(-xs, __ldg(zp + n), v);
        }
      }
      store_from_f32(out, (int64_t)m * N + n, out_dt, v);
    }
  }
}

template <int WBITS, bool BLOCKWISE, typename XT>
int launch_mt(const void* x, const void* w, const float* scale, const float* zp, void* out,
              int out_dt, int64_t M, int64_t N, int64_t K, int64_t block_size, cudaStream_t st) {
  const unsigned grid = (unsigned)ceil_div(N, kRows);
  const XT* xp = reinterpret_cast<const XT*>(x);
  const uint8_t* wp = reinterpret_cast<const uint8_t*>(w);
#define QMM_GEMV_LAUNCH(MT)                                                                    \
  gemv_nk_kernel<WBITS, BLOCKWISE, XT, MT><<<grid, kThreads, 0, st>>>(xp, wp, scale, zp, out,  \
                                                                      out_dt, (int)M, N, K,    \
                                                                      (int)block_size)
  if (M == 1)
    QMM_GEMV_LAUNCH(1);
  else if (M == 2)
    QMM_GEMV_LAUNCH(2);
  else if (M <= 4)
    QMM_GEMV_LAUNCH(4);
  else
    QMM_GEMV_LAUNCH(8);
#undef QMM_GEMV_LAUNCH
  return check_launch("gemv_nk_kernel");
}

}  // namespace

bool gemv_nk_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x,
                       int x_dt, const void* w) {
  if (M < 1 || M > 8 || N < 1 || K < 1) return false;
  const int vals = 128 / wbits;
  if (K % vals != 0) return false;                     // whole 16-byte slices per weight row
  if (block_size > 0 && block_size % vals != 0) return false;  // a slice stays inside one block
  if (!aligned(w, 16)) return false;
  if (!aligned(x, 16) || (K * (int64_t)dtype_size(x_dt)) % 16 != 0) return false;
  if (ceil_div(N, kRows) > 2147483647LL) return false;
  return true;
}

int launch_gemv_nk(int wbits, const void* x, int x_dt, const void* w, const float* scale,
                   const float* zp, void* out, int out_dt, int64_t M, int64_t N, int64_t K,
                   int64_t block_size, cudaStream_t st) {
  if (!gemv_nk_supported(wbits, M, N, K, block_size, x, x_dt, w))
    return fail(QMM_ERR_UNSUPPORTED,
                "gemv: needs 1<=M<=8, K a multiple of %d, block_size a multiple of %d and 16-byte "
                "aligned x/w (M=%lld N=%lld K=%lld bs=%lld)",
                128 / wbits, 128 / wbits, (long long)M, (long long)N, (long long)K,
                (long long)block_size);
  QMM_DISPATCH_DTYPE(x_dt, XT, {
    if (wbits == 8) {
      if (block_size > 0)
        return launch_mt<8, true, XT>(x, w, scale, zp, out, out_dt, M, N, K, block_size, st);
      return launch_mt<8, false, XT>(x, w, scale, zp, out, out_dt, M, N, K, block_size, st);
    }
    if (block_size > 0)
      return launch_mt<4, true, XT>(x, w, scale, zp, out, out_dt, M, N, K, block_size, st);
    return launch_mt<4, false, XT>(x, w, scale, zp, out, out_dt, M, N, K, block_size, st);
  });
  return QMM_OK;
}

}  // namespace qmm
