// Per-token dynamic activation quantizer (the W8A8 prologue).
//
// Restates _quantize_tensor (torch_xla/experimental/xla_quantized_matmul.py:56-73) bit for bit:
//   amax  = max_k |x[m,k]|                      (in x's dtype: exact)
//   scale = amax / 127                          (IEEE division, result rounded to x's dtype)
//   q     = x / scale                           (IEEE division, result rounded to x's dtype)
//   xq    = rint(q) -> int8                     (ties to even; the reference has no clamp)
// For bf16 activations the two roundings to bf16 are not optional: dropping the second one
// changes 0.6 % of the entries on N(0,1) data with outliers.
//
// One CTA per activation row.  bf16 rows of up to 8192 elements stay in registers between the two
// phases (amax, then quantize); other shapes read the row twice, the second time from L1/L2.  Either
// way HBM sees each activation once: 2 or 4 bytes in, 1 byte out per element.
#include "common.cuh"
#include "kernels.h"

namespace qmm {

namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ float round_to(float v) {
  return to_f32(from_f32<T>(v));
}

__device__ __forceinline__ int8_t to_int8(float r, bool saturate) {
  if (r != r) return 0;
  if (saturate) {
    r = fminf(fmaxf(r, -128.f), 127.f);
    return (int8_t)(int)r;
  }
  // wrap like a float -> int32 -> int8 conversion chain does for values in int32 range
  if (r > 2147483520.f || r < -2147483648.f) return 0;
  return (int8_t)(uint8_t)(((int)r) & 0xff);
}

template <typename T>
__device__ __forceinline__ int8_t quantize_one(T xv, float scale, bool saturate) {
  const float q = round_to<T>(__fdiv_rn(to_f32(xv), scale));
  return to_int8(rintf(q), saturate);
}

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack {
  T v[VEC];
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
    quantize_rows_kernel(const T* __restrict__ x, int8_t* __restrict__ xq,
                         float* __restrict__ x_scale, int32_t* __restrict__ rowsum, int64_t K,
                         int saturate, int vec_ok) {
  constexpr int VEC = 16 / sizeof(T);  // elements per 128-bit load
  __shared__ float s_red[kThreads / 32];
  __shared__ int s_isum[kThreads / 32];
  __shared__ float s_scale;
  const int64_t m = blockIdx.x;
  const T* row = x + m * K;
  int8_t* qrow = xq + m * K;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // pass 1: amax (NaN propagates like torch.amax)
  float amax = 0.f;
  bool has_nan = false;
  if (vec_ok) {
    const int64_t nvec = K / VEC;
    const Pack<T, VEC>* rv = reinterpret_cast<const Pack<T, VEC>*>(row);
    for (int64_t i = tid; i < nvec; i += kThreads) {
      Pack<T, VEC> p = rv[i];
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float a = fabsf(to_f32(p.v[j]));
        has_nan |= (a != a);
        amax = fmaxf(amax, a);
      }
    }
  } else {
    for (int64_t k = tid; k < K; k += kThreads) {
      const float a = fabsf(to_f32(row[k]));
      has_nan |= (a != a);
      amax = fmaxf(amax, a);
    }
  }
  if (has_nan) amax = __int_as_float(0x7fc00000);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, amax, o);
    amax = (amax != amax || other != other) ? __int_as_float(0x7fc00000) : fmaxf(amax, other);
  }
  if (lane == 0) s_red[warp] = amax;
  __syncthreads();
  if (tid == 0) {
    float a = s_red[0];
    for (int i = 1; i < kThreads / 32; ++i) {
      const float o = s_red[i];
      a = (a != a || o != o) ? __int_as_float(0x7fc00000) : fmaxf(a, o);
    }
    const float sc = round_to<T>(__fdiv_rn(a, 127.0f));
    s_scale = sc;
    x_scale[m] = sc;
  }
  __syncthreads();
  const float scale = s_scale;

  // pass 2: quantize (the row is still in L1/L2)
  int isum = 0;
  if (vec_ok) {
    const int64_t nvec = K / VEC;
    const Pack<T, VEC>* rv = reinterpret_cast<const Pack<T, VEC>*>(row);
    Pack<int8_t, VEC>* qv = reinterpret_cast<Pack<int8_t, VEC>*>(qrow);
    for (int64_t i = tid; i < nvec; i += kThreads) {
      Pack<T, VEC> p = rv[i];
      Pack<int8_t, VEC> q;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        q.v[j] = quantize_one<T>(p.v[j], scale, saturate != 0);
        isum += q.v[j];
      }
      qv[i] = q;
    }
  } else {
    for (int64_t k = tid; k < K; k += kThreads) {
      const int8_t q = quantize_one<T>(row[k], scale, saturate != 0);
      qrow[k] = q;
      isum += q;
    }
  }
  if (rowsum) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
    if (lane == 0) s_isum[warp] = isum;
    __syncthreads();
    if (tid == 0) {
      int t = 0;
      for (int i = 0; i < kThreads / 32; ++i) t += s_isum[i];
      rowsum[m] = t;
    }
  }
}


// ---- bf16 fast path: the row lives in registers; one global read, one global write -------------------
//
// amax is taken on the bit patterns: for non-negative floats the integer order is the float order, and
// a NaN pattern is larger than every number, so NaN propagates like torch.amax without extra tests.
//
// The quotient x / scale must be the correctly rounded fp32 quotient (it is rounded to bf16 next and
// ties decide).  One Newton step on q0 = x * (1/scale) gives it: both operands have 8-bit significands,
// so the exact quotient is either a tie (exactly representable: the step lands on it) or at least
// 2^-17 away from any bf16 rounding boundary, far more than the error of q0.
template <int CHUNKS>
__global__ void __launch_bounds__(kThreads)
    quantize_rows_bf16_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ xq,
                              float* __restrict__ x_scale, int32_t* __restrict__ rowsum, int64_t K,
                              int saturate) {
  __shared__ uint32_t s_red[kThreads / 32];
  __shared__ int s_isum[kThreads / 32];
  // the GEMM that consumes this kernel's output may start its set-up now; it waits for this grid to finish
  // (griddepcontrol.wait) before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int64_t m = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvec = (int)(K >> 3);  // 16-byte chunks (8 bf16) in the row
  const uint4* rv = reinterpret_cast<const uint4*>(x + m * K);
  uint4 v[CHUNKS];
  uint32_t amax_bits = 0;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = tid + c * kThreads;
    v[c] = make_uint4(0, 0, 0, 0);
    if (i < nvec) v[c] = rv[i];
    const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      amax_bits = max(amax_bits, w[j] & 0x7fffu);
      amax_bits = max(amax_bits, (w[j] >> 16) & 0x7fffu);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, o));
  if (lane == 0) s_red[warp] = amax_bits;
  __syncthreads();
  uint32_t a = s_red[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; ++i) a = max(a, s_red[i]);
  const float amax = __uint_as_float(a << 16);
  const float scale = round_to<__nv_bfloat16>(__fdiv_rn(amax, 127.0f));
  if (tid == 0) x_scale[m] = scale;
  const float rcp = __frcp_rn(scale);
  // scale == 0 (all-zero row), inf or NaN: the Newton step is not valid there; fall back to IEEE division
  const bool regular = scale > 1e-30f && scale < 1e30f;

  int isum = 0;
  uint2* qv = reinterpret_cast<uint2*>(xq + m * K);
  if (regular) {
    // Everything after the quotient stays on the FMA and integer pipes (no conversion-unit instruction):
    //   bf16 rounding   Veltkamp split with 2^16 + 1: g = q * 65537, qb = g + (q - g) is q rounded to 8
    //                   significant bits, ties to even (each step is one correctly rounded operation; the
    //                   explicit _rn intrinsics keep the compiler from fusing them)
    //   rint -> int     qb + 1.5 * 2^23 leaves the integer, rounded ties-to-even, in the low mantissa bits
    //   int8            clamp (or wrap) in integers, bytes gathered with prmt, row sum with dp4a
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = tid + c * kThreads;
      const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
      int qi[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xv = __uint_as_float((j & 1) ? (w[j >> 1] & 0xffff0000u) : (w[j >> 1] << 16));
        const float q0 = xv * rcp;
        const float r = fmaf(-q0, scale, xv);
        const float q = fmaf(r, rcp, q0);
        const float g = __fmul_rn(q, 65537.f);
        const float qb = __fadd_rn(g, __fsub_rn(q, g));
        int t = __float_as_int(__fadd_rn(qb, 12582912.f)) - 0x4B400000;
        if (saturate) t = max(-128, min(127, t));
        qi[j] = t;
      }
      uint32_t packed[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = __byte_perm((uint32_t)qi[4 * h], (uint32_t)qi[4 * h + 1], 0x0040);
        const uint32_t hi = __byte_perm((uint32_t)qi[4 * h + 2], (uint32_t)qi[4 * h + 3], 0x0040);
        packed[h] = __byte_perm(lo, hi, 0x5410);
        isum = __dp4a((int)packed[h], 0x01010101, isum);
      }
      if (i < nvec) qv[i] = make_uint2(packed[0], packed[1]);
    }
  } else {
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = tid + c * kThreads;
      const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
      uint32_t packed[2] = {0, 0};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xv = __uint_as_float((j & 1) ? (w[j >> 1] & 0xffff0000u) : (w[j >> 1] << 16));
        const float q = __fdiv_rn(xv, scale);
        const int8_t qi = to_int8(rintf(round_to<__nv_bfloat16>(q)), saturate != 0);
        isum += qi;
        packed[j >> 2] |= ((uint32_t)(uint8_t)qi) << (8 * (j & 3));
      }
      if (i < nvec) qv[i] = make_uint2(packed[0], packed[1]);
    }
  }
  if (rowsum) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
    if (lane == 0) s_isum[warp] = isum;
    __syncthreads();
    if (tid == 0) {
      int t = 0;
      for (int i = 0; i < kThreads / 32; ++i) t += s_isum[i];
      rowsum[m] = t;
    }
  }
}

}  // namespace

int launch_quantize_activation(const void* x, int x_dt, int8_t* xq, float* x_scale,
                               int32_t* rowsum, int64_t M, int64_t K, int saturate,
                               cudaStream_t st) {
  if (M == 0) return QMM_OK;
  if (M > 2147483647LL) return fail(QMM_ERR_UNSUPPORTED, "quantize_activation: M too large");
  if (x_dt == QMM_BF16 && K % 8 == 0 && K <= 8 * 4 * kThreads && aligned(x, 16) && aligned(xq, 8)) {
    const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
    const int chunks = (int)ceil_div(K / 8, kThreads);
    if (chunks <= 1)
      quantize_rows_bf16_kernel<1><<<(unsigned)M, kThreads, 0, st>>>(xp, xq, x_scale, rowsum, K, saturate);
    else if (chunks == 2)
      quantize_rows_bf16_kernel<2><<<(unsigned)M, kThreads, 0, st>>>(xp, xq, x_scale, rowsum, K, saturate);
    else
      quantize_rows_bf16_kernel<4><<<(unsigned)M, kThreads, 0, st>>>(xp, xq, x_scale, rowsum, K, saturate);
    return check_launch("quantize_rows_bf16_kernel");
  }
  QMM_DISPATCH_DTYPE(x_dt, T, {
    constexpr int VEC = 16 / sizeof(T);
    const int vec_ok = (K % VEC == 0) && aligned(x, 16) && aligned(xq, VEC) ? 1 : 0;
    quantize_rows_kernel<T><<<(unsigned)M, kThreads, 0, st>>>(reinterpret_cast<const T*>(x), xq,
                                                              x_scale, rowsum, K, saturate, vec_ok);
  });
  return check_launch("quantize_rows_kernel");
}

}  // namespace qmm
