// Shared host/device helpers for the quantized-linear kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qmm_b200.h"

namespace qmm {

// ---- error reporting (host) ---------------------------------------------------------------
int fail(int status, const char* fmt, ...);  // records the message for qmm_last_error_string
int check_launch(const char* what);          // cudaPeekAtLastError -> status

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Word that kernels with bounded waits set when a wait gives up (0 = healthy).
uint32_t* device_error_word();  // device address of the flag for the current device, or nullptr

// How long a kernel waits for another GPU before it gives up, in SM clock cycles (qmm_set_peer_wait_limit).
long long peer_wait_cycles();

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline bool valid_float_dtype(int dt) { return dt == QMM_F32 || dt == QMM_BF16 || dt == QMM_F16; }

inline size_t dtype_size(int dt) { return dt == QMM_F32 ? 4 : 2; }

int sm_count();
bool device_is_sm100();

// ---- element access (device) --------------------------------------------------------------
template <int DT>
struct ElemOf;
template <>
struct ElemOf<QMM_F32> {
  using type = float;
};
template <>
struct ElemOf<QMM_BF16> {
  using type = __nv_bfloat16;
};
template <>
struct ElemOf<QMM_F16> {
  using type = __half;
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
  return __float2half_rn(v);
}

// Runtime-typed scalar load/store for the kernels that are not specialised per dtype.
__device__ __forceinline__ float load_as_f32(const void* p, int64_t i, int dt) {
  if (dt == QMM_F32) return reinterpret_cast<const float*>(p)[i];
  if (dt == QMM_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ void store_from_f32(void* p, int64_t i, int dt, float v) {
  if (dt == QMM_F32)
    reinterpret_cast<float*>(p)[i] = v;
  else if (dt == QMM_BF16)
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

// 128-bit streaming load that does not pollute L1 (weights are read exactly once).
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Dispatch a runtime dtype to a compile-time one.
#define QMM_DISPATCH_DTYPE(dt, NAME, ...)          \
  switch (dt) {                                    \
    case QMM_F32: {                                \
      using NAME = float;                          \
      __VA_ARGS__;                                 \
    } break;                                       \
    case QMM_BF16: {                               \
      using NAME = __nv_bfloat16;                  \
      __VA_ARGS__;                                 \
    } break;                                       \
    default: {                                     \
      using NAME = __half;                         \
      __VA_ARGS__;                                 \
    } break;                                       \
  }

}  // namespace qmm
