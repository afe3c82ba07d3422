// An entry point for callers that may not allocate device memory.
//
// qmm_w8a8_perchannel needs scratch between its two kernels (the quantized activations, their
// scales and row sums) and asks the caller for it.  Some callers have nowhere to get it from: a
// serving process whose framework reserved the whole GPU at start-up and hands out no raw
// allocations to plugins, a real-time loop in which cudaMalloc's implicit device synchronisation
// is not acceptable, or host code written against a rule that nothing allocates after
// initialisation.  For them the scratch lives in this library's own device image: a fixed
// file-scope array that every GPU which loads the library carries until the process exits.
//
// The price is a hard size limit (QMM_STATIC_SCRATCH_BYTES) and one shared buffer: calls whose
// kernels can overlap on the GPU (different streams, different host threads) race on it.
#include "common.cuh"
#include "kernels.h"

namespace {

// Scratch of the no-allocation entry point.  Device code could name it directly; host code may
// not: on the host this identifier is only a handle for cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[QMM_STATIC_SCRATCH_BYTES];

// Device address of the array, looked up once per device with that device current.
void* static_scratch_address() {
  static void* cached[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    qmm::fail(QMM_ERR_DEVICE, "static scratch: no current CUDA device");
    return nullptr;
  }
  if (!cached[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) {
      cudaGetLastError();
      qmm::fail(QMM_ERR_DEVICE, "static scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cached[dev] = ptr;
  }
  return cached[dev];
}

}  // namespace

extern "C" int qmm_w8a8_perchannel_static(const void* x, int x_dtype, const int8_t* w,
                                          const float* w_scale, const float* zp, void* out,
                                          int out_dtype, int64_t M, int64_t N, int64_t K,
                                          int saturate, int variant, void* stream) {
  if (M < 0 || N < 0 || K < 0) return qmm::fail(QMM_ERR_BAD_SHAPE, "negative dimension");
  const size_t need = qmm_workspace_size(QMM_OP_W8A8_PERCHANNEL, M, N, K);
  if (need > (size_t)QMM_STATIC_SCRATCH_BYTES)
    return qmm::fail(QMM_ERR_WORKSPACE,
                     "qmm_w8a8_perchannel_static: M=%lld K=%lld needs %zu bytes of scratch, the built-in "
                     "buffer holds %zu; use qmm_w8a8_perchannel with caller-provided workspace",
                     (long long)M, (long long)K, need, (size_t)QMM_STATIC_SCRATCH_BYTES);
  if (M * N == 0) return QMM_OK;
  void* scratch = static_scratch_address();
  if (!scratch) return QMM_ERR_DEVICE;
  // Nothing in the scratch has to start at zero: every byte the contraction reads (quantized rows,
  // their scales, their row sums when a zero point is given) is written by the quantizer first.
  return qmm_w8a8_perchannel(x, x_dtype, w, w_scale, zp, out, out_dtype, M, N, K, saturate, variant,
                             scratch, (size_t)QMM_STATIC_SCRATCH_BYTES, stream);
}
