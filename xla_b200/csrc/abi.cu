// extern "C" entry points of libqmm_b200 (declared in include/qmm_b200.h): argument checks,
// kernel-family selection, and the host-side helpers the kernels share.
#include <cuda.h>
#include <atomic>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace qmm {

// ---- error reporting ----------------------------------------------------------------------
static thread_local char g_last_error[512] = "";

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();  // clear the sticky-less launch error so later calls start clean
    return fail(QMM_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  }
  return QMM_OK;
}

// ---- device queries -----------------------------------------------------------------------
struct DeviceInfo {
  bool known = false;
  int sms = 0;
  int cc_major = 0;
};
static DeviceInfo g_dev[64];

static DeviceInfo* device_info() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  DeviceInfo* d = &g_dev[dev];
  if (!d->known) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return nullptr;
    d->sms = prop.multiProcessorCount;
    d->cc_major = prop.major;
    d->known = true;
  }
  return d;
}

int sm_count() {
  DeviceInfo* d = device_info();
  return d ? d->sms : 1;
}

bool device_is_sm100() {
  DeviceInfo* d = device_info();
  return d && d->cc_major == 10;
}

// One error word per device, living in the library's own device image.
__device__ uint32_t g_qmm_error_word;

uint32_t* device_error_word() {
  static uint32_t* cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_qmm_error_word) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cached[dev] = reinterpret_cast<uint32_t*>(p);
  }
  return cached[dev];
}

static std::atomic<long long> g_peer_wait_cycles{2000000000ll};  // about a second of SM clock
long long peer_wait_cycles() { return g_peer_wait_cycles.load(std::memory_order_relaxed); }


// ---- tensor maps --------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int encode_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, bool is_float16_family,
                   uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(QMM_ERR_DEVICE, "driver does not provide cuTensorMapEncodeTiled");
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  if (elem_bytes == 2) dt = is_float16_family ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
  if (elem_bytes == 4) dt = CU_TENSOR_MAP_DATA_TYPE_UINT32;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(QMM_ERR_LAUNCH,
                "cuTensorMapEncodeTiled failed (%d) for [%llu x %llu] elem %d box [%u x %u]", (int)r,
                (unsigned long long)rows, (unsigned long long)cols, elem_bytes, box_rows, box_cols);
  return QMM_OK;
}

// ---- argument checks ----------------------------------------------------------------------
static int check_common(const void* x, int x_dt, const void* w, const float* scale, void* out,
                        int out_dt, int64_t M, int64_t N, int64_t K) {
  if (M < 0 || N < 0 || K < 0) return fail(QMM_ERR_BAD_SHAPE, "negative dimension (M=%lld N=%lld K=%lld)",
                                           (long long)M, (long long)N, (long long)K);
  if (!valid_float_dtype(x_dt) || !valid_float_dtype(out_dt))
    return fail(QMM_ERR_UNSUPPORTED, "dtype must be QMM_F32, QMM_BF16 or QMM_F16 (x=%d out=%d)", x_dt, out_dt);
  if (M * N == 0) return QMM_OK;
  if (!out) return fail(QMM_ERR_NULL, "out is NULL");
  if (K > 0 && (!x || !w)) return fail(QMM_ERR_NULL, "x or w is NULL");
  if (!scale) return fail(QMM_ERR_NULL, "scale is NULL");
  return QMM_OK;
}

static bool env_flag(const char* name) {
  const char* v = getenv(name);
  return v && v[0] && v[0] != '0';
}

static void log_choice(const char* op, const char* variant, int64_t M, int64_t N, int64_t K) {
  static int on = -1;
  if (on < 0) on = env_flag("QMM_B200_LOG") ? 1 : 0;
  if (on) fprintf(stderr, "[qmm_b200] %s M=%lld N=%lld K=%lld -> %s\n", op, (long long)M, (long long)N,
                  (long long)K, variant);
}

}  // namespace qmm

using namespace qmm;

extern "C" {

int qmm_abi_version(void) { return QMM_ABI_VERSION; }

const char* qmm_status_string(int status) {
  switch (status) {
    case QMM_OK: return "ok";
    case QMM_ERR_BAD_SHAPE: return "bad shape";
    case QMM_ERR_UNSUPPORTED: return "unsupported";
    case QMM_ERR_MISALIGNED: return "misaligned";
    case QMM_ERR_LAUNCH: return "launch failure";
    case QMM_ERR_WORKSPACE: return "workspace too small";
    case QMM_ERR_NULL: return "null pointer";
    case QMM_ERR_DEVICE: return "device not supported";
    case QMM_ERR_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

const char* qmm_last_error_string(void) { return g_last_error; }

// AUTO choice for the weight-only ops on K-minor weights: the register-dequant MMA kernel for decode
// batches, the tcgen05 kernel above that, the CUDA-core GEMV where those cannot go (zero points, f32
// activations), the any-shape kernel for everything else.
static int pick_weight_only(int wbits, int64_t M, int64_t N, int64_t K, int64_t bs, const void* x, int x_dt,
                            const void* w, bool has_zp) {
  if (decode_mma_supported(wbits, M, N, K, bs, x, x_dt, w, has_zp)) return QMM_VARIANT_MMA;
  if (mixed_tc_supported(wbits, M, N, K, bs, x, x_dt, w, has_zp)) return QMM_VARIANT_TCGEN05;
  if (gemv_nk_supported(wbits, M, N, K, bs, x, x_dt, w)) return QMM_VARIANT_GEMV;
  return QMM_VARIANT_GENERIC;
}

int qmm_w8a16_perchannel(const void* x, int x_dtype, const int8_t* w, const float* scale,
                         const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                         int64_t K, int variant, void* stream) {
  int rc = check_common(x, x_dtype, w, scale, out, out_dtype, M, N, K);
  if (rc != QMM_OK || M * N == 0) return rc;
  cudaStream_t st = as_stream(stream);
  if (variant == QMM_VARIANT_AUTO) variant = pick_weight_only(8, M, N, K, 0, x, x_dtype, w, zp != nullptr);
  switch (variant) {
    case QMM_VARIANT_GENERIC:
      log_choice("w8a16_perchannel", "generic", M, N, K);
      return launch_generic_nk(false, x, x_dtype, w, scale, zp, out, out_dtype, M, N, K, 0, st);
    case QMM_VARIANT_GEMV:
      log_choice("w8a16_perchannel", "gemv", M, N, K);
      return launch_gemv_nk(8, x, x_dtype, w, scale, zp, out, out_dtype, M, N, K, 0, st);
    case QMM_VARIANT_MMA:
      log_choice("w8a16_perchannel", "mma", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "the register-dequant decode kernel does not take a zero point");
      return launch_decode_mma(8, x, x_dtype, w, scale, out, out_dtype, M, N, K, 0, st);
    case QMM_VARIANT_TCGEN05:
      log_choice("w8a16_perchannel", "tcgen05", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "tcgen05 weight-only kernel does not take a zero point");
      return launch_mixed_tc(8, x, x_dtype, w, scale, out, out_dtype, M, N, K, 0, st);
    default:
      return fail(QMM_ERR_UNSUPPORTED, "unknown variant %d", variant);
  }
}

int qmm_blockwise_sbn(const void* x, int x_dtype, const int8_t* w, const float* scale,
                      const float* zp, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                      int64_t block_size, int variant, void* stream) {
  int rc = check_common(x, x_dtype, w, scale, out, out_dtype, M, N, K);
  if (rc != QMM_OK) return rc;
  if (block_size <= 0 || K % block_size != 0)
    return fail(QMM_ERR_BAD_SHAPE, "input_dim should be divisible by block_size, got input_dim: %lld, block_size: %lld",
                (long long)K, (long long)block_size);
  if (M * N == 0) return QMM_OK;
  cudaStream_t st = as_stream(stream);
  // This layout (N minor) is served by the any-shape kernel only: the streaming kernels want K-minor rows, and the
  // callers above this entry convert a weight once (qmm_pack_int4_sbn, or a transposed copy) and keep it.
  if (variant != QMM_VARIANT_AUTO && variant != QMM_VARIANT_GENERIC)
    return fail(QMM_ERR_UNSUPPORTED, "blockwise_sbn: variant %d is not available for this layout", variant);
  log_choice("blockwise_sbn", "generic", M, N, K);
  return launch_generic_sbn(x, x_dtype, w, scale, zp, out, out_dtype, M, N, K, block_size, st);
}

int qmm_w4a16_blockwise_packed(const void* x, int x_dtype, const uint8_t* wp, const float* scale,
                               const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                               int64_t K, int64_t block_size, int variant, void* stream) {
  int rc = check_common(x, x_dtype, wp, scale, out, out_dtype, M, N, K);
  if (rc != QMM_OK) return rc;
  if (K % 2 != 0) return fail(QMM_ERR_BAD_SHAPE, "packed int4 needs an even K, got %lld", (long long)K);
  if (block_size <= 0 || K % block_size != 0)
    return fail(QMM_ERR_BAD_SHAPE, "input_dim should be divisible by block_size, got input_dim: %lld, block_size: %lld",
                (long long)K, (long long)block_size);
  if (M * N == 0) return QMM_OK;
  cudaStream_t st = as_stream(stream);
  if (variant == QMM_VARIANT_AUTO) variant = pick_weight_only(4, M, N, K, block_size, x, x_dtype, wp, zp != nullptr);
  switch (variant) {
    case QMM_VARIANT_GENERIC:
      log_choice("w4a16_blockwise_packed", "generic", M, N, K);
      return launch_generic_nk(true, x, x_dtype, wp, scale, zp, out, out_dtype, M, N, K, block_size, st);
    case QMM_VARIANT_GEMV:
      log_choice("w4a16_blockwise_packed", "gemv", M, N, K);
      return launch_gemv_nk(4, x, x_dtype, wp, scale, zp, out, out_dtype, M, N, K, block_size, st);
    case QMM_VARIANT_MMA:
      log_choice("w4a16_blockwise_packed", "mma", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "the register-dequant decode kernel does not take a zero point");
      return launch_decode_mma(4, x, x_dtype, wp, scale, out, out_dtype, M, N, K, block_size, st);
    case QMM_VARIANT_TCGEN05:
      log_choice("w4a16_blockwise_packed", "tcgen05", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "tcgen05 weight-only kernel does not take a zero point");
      return launch_mixed_tc(4, x, x_dtype, wp, scale, out, out_dtype, M, N, K, block_size, st);
    default:
      return fail(QMM_ERR_UNSUPPORTED, "unknown variant %d", variant);
  }
}

int qmm_w8a16_blockwise(const void* x, int x_dtype, const int8_t* w, const float* scale, const float* zp, void* out,
                        int out_dtype, int64_t M, int64_t N, int64_t K, int64_t block_size, int variant, void* stream) {
  int rc = check_common(x, x_dtype, w, scale, out, out_dtype, M, N, K);
  if (rc != QMM_OK) return rc;
  if (block_size <= 0 || K % block_size != 0)
    return fail(QMM_ERR_BAD_SHAPE, "input_dim should be divisible by block_size, got input_dim: %lld, block_size: %lld",
                (long long)K, (long long)block_size);
  if (M * N == 0) return QMM_OK;
  cudaStream_t st = as_stream(stream);
  if (variant == QMM_VARIANT_AUTO) variant = pick_weight_only(8, M, N, K, block_size, x, x_dtype, w, zp != nullptr);
  switch (variant) {
    case QMM_VARIANT_GENERIC:
      log_choice("w8a16_blockwise", "generic", M, N, K);
      return launch_generic_nk(false, x, x_dtype, w, scale, zp, out, out_dtype, M, N, K, block_size, st);
    case QMM_VARIANT_GEMV:
      log_choice("w8a16_blockwise", "gemv", M, N, K);
      return launch_gemv_nk(8, x, x_dtype, w, scale, zp, out, out_dtype, M, N, K, block_size, st);
    case QMM_VARIANT_MMA:
      log_choice("w8a16_blockwise", "mma", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "the register-dequant decode kernel does not take a zero point");
      return launch_decode_mma(8, x, x_dtype, w, scale, out, out_dtype, M, N, K, block_size, st);
    case QMM_VARIANT_TCGEN05:
      log_choice("w8a16_blockwise", "tcgen05", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "tcgen05 weight-only kernel does not take a zero point");
      return launch_mixed_tc(8, x, x_dtype, w, scale, out, out_dtype, M, N, K, block_size, st);
    default:
      return fail(QMM_ERR_UNSUPPORTED, "unknown variant %d", variant);
  }
}

// ---- tuned kernel choice ------------------------------------------------------------------------------------------
// The counterpart of the reference's TUNED_BLOCK_SIZES / get_tuned_block_sizes
// (torch_xla/experimental/pallas_kernels/quantized_matmul_kernel.py:326-555): measured on a B200 by xla_b200/tune.py.
namespace {
struct TunedRow {
  int wbits, block_size;
  int64_t N, K;
  unsigned char choice[7];  // QMM_VARIANT_* for M <= 1, 2, 4, 8, 16, 32, 64; 0 = not measured
};
const TunedRow kTuned[] = {
#include "tuned_table.inc"
    {0, 0, 0, 0, {0, 0, 0, 0, 0, 0, 0}},  // end
};

int tuned_variant(int wbits, int64_t block_size, int64_t M, int64_t N, int64_t K) {
  if (M < 1 || M > 64) return 0;
  int bucket = 0;
  while ((1 << bucket) < M) ++bucket;
  for (const TunedRow* r = kTuned; r->wbits; ++r)
    if (r->wbits == wbits && r->block_size == block_size && r->N == N && r->K == K) return r->choice[bucket];
  return 0;
}
}  // namespace

int qmm_tuned_variant(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size) {
  return tuned_variant(wbits, block_size < 0 ? 0 : block_size, M, N, K);
}

const char* qmm_weight_only_variant_for(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, int has_zp) {
  // Shape-only view of qmm_weight_only's AUTO choice, for a caller that passes a sufficient workspace and aligned pointers.
  if (block_size < 0) block_size = 0;
  const void* ok = reinterpret_cast<const void*>(uintptr_t(256));
  const bool can = limb_tc_shape_ok(wbits, M, N, K, block_size, QMM_BF16, has_zp != 0);
  const int tuned = tuned_variant(wbits, block_size, M, N, K);
  if (can && (tuned ? tuned == QMM_VARIANT_I8TC : limb_tc_preferred(wbits, M, N, K, block_size))) return "i8tc";
  if (!has_zp && tuned == QMM_VARIANT_MMA && decode_mma_supported(wbits, M, N, K, block_size, ok, QMM_BF16, ok, false)) return "mma";
  if (!has_zp && tuned == QMM_VARIANT_TCGEN05 && mixed_tc_shape_ok(wbits, M, N, K, block_size, QMM_BF16, false)) return "tcgen05";
  if (decode_mma_supported(wbits, M, N, K, block_size, ok, QMM_BF16, ok, has_zp != 0)) return "mma";
  if (mixed_tc_shape_ok(wbits, M, N, K, block_size, QMM_BF16, has_zp != 0)) return "tcgen05";
  if (gemv_nk_supported(wbits, M, N, K, block_size, ok, QMM_BF16, ok)) return "gemv";
  return "generic";
}

size_t qmm_weight_only_workspace_size(int64_t max_M, int64_t K) {
  return limb_tc_workspace_bytes(max_M, K);
}

size_t qmm_weight_only_workspace_size_for(int wbits, int64_t max_M, int64_t N, int64_t K) {
  const size_t base = limb_tc_workspace_bytes(max_M, K);
  if (base == 0 || N < 1) return base;
  return (base + 255) / 256 * 256 + limb_tc_wide_bytes(wbits, max_M, N, K);
}

int qmm_weight_only(int wbits, const void* x, int x_dtype, const void* w, const float* scale, const float* zp, void* out,
                    int out_dtype, int64_t M, int64_t N, int64_t K, int64_t block_size, int variant, void* workspace,
                    size_t workspace_bytes, void* stream) {
  if (wbits != 4 && wbits != 8) return fail(QMM_ERR_BAD_SHAPE, "weight_only: wbits must be 4 or 8, got %d", wbits);
  if (block_size < 0) block_size = 0;
  if (variant == QMM_VARIANT_AUTO || variant == QMM_VARIANT_I8TC) {
    int rc = check_common(x, x_dtype, w, scale, out, out_dtype, M, N, K);
    if (rc != QMM_OK || M * N == 0) return rc;
    if (block_size > 0 && K % block_size != 0)
      return fail(QMM_ERR_BAD_SHAPE, "input_dim should be divisible by block_size, got input_dim: %lld, block_size: %lld",
                  (long long)K, (long long)block_size);
    const bool can = limb_tc_supported(wbits, M, N, K, block_size, x, x_dtype, w, zp != nullptr) && workspace &&
                     workspace_bytes >= limb_tc_workspace_bytes(M, K) && aligned(workspace, 256);
    // AUTO: the measured table first, the shape rule where the table has no entry for this shape
    const int tuned = variant == QMM_VARIANT_AUTO ? tuned_variant(wbits, block_size, M, N, K) : 0;
    bool use = variant == QMM_VARIANT_I8TC;
    if (variant == QMM_VARIANT_AUTO && can) use = tuned ? tuned == QMM_VARIANT_I8TC : limb_tc_preferred(wbits, M, N, K, block_size);
    if (!use && tuned && tuned != QMM_VARIANT_I8TC && !zp) {
      // the table names one of the kernels behind the entry points below; they refuse what they cannot run, and AUTO
      // then decides there
      const bool ok = tuned == QMM_VARIANT_MMA ? decode_mma_supported(wbits, M, N, K, block_size, x, x_dtype, w, false)
                                               : (tuned == QMM_VARIANT_TCGEN05 && mixed_tc_supported(wbits, M, N, K, block_size, x, x_dtype, w, false));
      if (ok) variant = tuned;
    }
    if (use) {
      log_choice("weight_only", "i8tc", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "the split-activation tensor-core kernel does not take a zero point");
      return launch_limb_tc(wbits, x, x_dtype, w, scale, out, out_dtype, M, N, K, block_size, 0, workspace, workspace_bytes,
                            as_stream(stream));
    }
  }
  if (wbits == 8) {
    if (block_size > 0)
      return qmm_w8a16_blockwise(x, x_dtype, static_cast<const int8_t*>(w), scale, zp, out, out_dtype, M, N, K, block_size, variant,
                                 stream);
    return qmm_w8a16_perchannel(x, x_dtype, static_cast<const int8_t*>(w), scale, zp, out, out_dtype, M, N, K, variant, stream);
  }
  if (block_size > 0)
    return qmm_w4a16_blockwise_packed(x, x_dtype, static_cast<const uint8_t*>(w), scale, zp, out, out_dtype, M, N, K, block_size,
                                      variant, stream);
  return qmm_w4a16_perchannel_packed(x, x_dtype, static_cast<const uint8_t*>(w), scale, zp, out, out_dtype, M, N, K, variant, stream);
}

int qmm_gate_up_decode(int wbits, const void* x, int x_dtype, const void* w, const float* scale, void* out,
                       int out_dtype, int64_t M, int64_t N2, int64_t K, int64_t block_size, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (wbits != 4 && wbits != 8) return fail(QMM_ERR_BAD_SHAPE, "gate_up_decode: wbits must be 4 or 8, got %d", wbits);
  if (!x || !w || !scale || !out) return fail(QMM_ERR_NULL, "gate_up_decode: null pointer");
  if (M < 0 || N2 < 0 || K < 0) return fail(QMM_ERR_BAD_SHAPE, "gate_up_decode: negative size");
  if (N2 % 16 != 0) return fail(QMM_ERR_BAD_SHAPE, "gate_up_decode: N2 must be a multiple of 16, got %lld", (long long)N2);
  if (block_size < 0 || (block_size > 0 && K % block_size != 0))
    return fail(QMM_ERR_BAD_SHAPE, "gate_up_decode: K (%lld) must be a multiple of block_size (%lld)", (long long)K,
                (long long)block_size);
  if (M == 0 || N2 == 0) return QMM_OK;
  if (!decode_mma_supported(wbits, M, N2, K, block_size, x, x_dtype, w, false))
    return fail(QMM_ERR_UNSUPPORTED, "gate_up_decode: needs 1<=M<=32, bf16/f16 activations, K a multiple of %d, 16-byte "
                "aligned x/w (M=%lld N2=%lld K=%lld bs=%lld)", 512 / wbits, (long long)M, (long long)N2, (long long)K,
                (long long)block_size);
  log_choice("gate_up_decode", "mma", M, N2, K);
  return launch_decode_mma(wbits, x, x_dtype, w, scale, out, out_dtype, M, N2, K, block_size, st, 1);
}

int qmm_gate_up(int wbits, const void* x, int x_dtype, const void* w, const float* scale, void* out, int out_dtype, int64_t M,
                int64_t N2, int64_t K, int64_t block_size, void* workspace, size_t workspace_bytes, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (wbits != 4 && wbits != 8) return fail(QMM_ERR_BAD_SHAPE, "gate_up: wbits must be 4 or 8, got %d", wbits);
  if (!x || !w || !scale || !out) return fail(QMM_ERR_NULL, "gate_up: null pointer");
  if (M < 0 || N2 < 0 || K < 0) return fail(QMM_ERR_BAD_SHAPE, "gate_up: negative size");
  if (N2 % 16 != 0) return fail(QMM_ERR_BAD_SHAPE, "gate_up: N2 must be a multiple of 16, got %lld", (long long)N2);
  if (block_size < 0 || (block_size > 0 && K % block_size != 0))
    return fail(QMM_ERR_BAD_SHAPE, "gate_up: K (%lld) must be a multiple of block_size (%lld)", (long long)K, (long long)block_size);
  if (M == 0 || N2 == 0) return QMM_OK;
  log_choice("gate_up", "i8tc", M, N2, K);
  return launch_limb_tc(wbits, x, x_dtype, w, scale, out, out_dtype, M, N2, K, block_size, 1, workspace, workspace_bytes, st);
}

int qmm_w4a16_perchannel_packed(const void* x, int x_dtype, const uint8_t* wp, const float* scale,
                                const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                                int64_t K, int variant, void* stream) {
  int rc = check_common(x, x_dtype, wp, scale, out, out_dtype, M, N, K);
  if (rc != QMM_OK) return rc;
  if (K % 2 != 0) return fail(QMM_ERR_BAD_SHAPE, "packed int4 needs an even K, got %lld", (long long)K);
  if (M * N == 0) return QMM_OK;
  cudaStream_t st = as_stream(stream);
  if (variant == QMM_VARIANT_AUTO) variant = pick_weight_only(4, M, N, K, 0, x, x_dtype, wp, zp != nullptr);
  switch (variant) {
    case QMM_VARIANT_GENERIC:
      log_choice("w4a16_perchannel_packed", "generic", M, N, K);
      return launch_generic_nk(true, x, x_dtype, wp, scale, zp, out, out_dtype, M, N, K, 0, st);
    case QMM_VARIANT_GEMV:
      log_choice("w4a16_perchannel_packed", "gemv", M, N, K);
      return launch_gemv_nk(4, x, x_dtype, wp, scale, zp, out, out_dtype, M, N, K, 0, st);
    case QMM_VARIANT_MMA:
      log_choice("w4a16_perchannel_packed", "mma", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "the register-dequant decode kernel does not take a zero point");
      return launch_decode_mma(4, x, x_dtype, wp, scale, out, out_dtype, M, N, K, 0, st);
    case QMM_VARIANT_TCGEN05:
      log_choice("w4a16_perchannel_packed", "tcgen05", M, N, K);
      if (zp) return fail(QMM_ERR_UNSUPPORTED, "tcgen05 weight-only kernel does not take a zero point");
      return launch_mixed_tc(4, x, x_dtype, wp, scale, out, out_dtype, M, N, K, 0, st);
    default:
      return fail(QMM_ERR_UNSUPPORTED, "unknown variant %d", variant);
  }
}

int qmm_quantize_activation(const void* x, int x_dtype, int8_t* xq, float* x_scale,
                            int32_t* xq_rowsum, int64_t M, int64_t K, int saturate, void* stream) {
  if (M < 0 || K < 0) return fail(QMM_ERR_BAD_SHAPE, "negative dimension");
  if (!valid_float_dtype(x_dtype)) return fail(QMM_ERR_UNSUPPORTED, "bad x dtype %d", x_dtype);
  if (M == 0) return QMM_OK;
  if (!x_scale || (K > 0 && (!x || !xq))) return fail(QMM_ERR_NULL, "x, xq or x_scale is NULL");
  return launch_quantize_activation(x, x_dtype, xq, x_scale, xq_rowsum, M, K, saturate, as_stream(stream));
}

int qmm_w8a8_gemm(const int8_t* xq, const int8_t* w, const float* w_scale, const float* zp,
                  const float* x_scale, const int32_t* xq_rowsum, int32_t* acc_out, void* out,
                  int out_dtype, int64_t M, int64_t N, int64_t K, int variant, void* stream) {
  if (M < 0 || N < 0 || K < 0) return fail(QMM_ERR_BAD_SHAPE, "negative dimension");
  if (M * N == 0) return QMM_OK;
  if (!acc_out && !out) return fail(QMM_ERR_NULL, "acc_out and out are both NULL");
  if (out && !valid_float_dtype(out_dtype)) return fail(QMM_ERR_UNSUPPORTED, "bad out dtype %d", out_dtype);
  if (out && (!w_scale || !x_scale)) return fail(QMM_ERR_NULL, "w_scale or x_scale is NULL");
  if (zp && !xq_rowsum) return fail(QMM_ERR_NULL, "a zero point needs xq_rowsum");
  if (K > 0 && (!xq || !w)) return fail(QMM_ERR_NULL, "xq or w is NULL");
  cudaStream_t st = as_stream(stream);
  if (variant == QMM_VARIANT_AUTO)
    variant = (w8a8_tc_supported(M, N, K, xq, w) && M >= 16) ? QMM_VARIANT_TCGEN05 : QMM_VARIANT_GENERIC;
  switch (variant) {
    case QMM_VARIANT_GENERIC:
      log_choice("w8a8_gemm", "generic", M, N, K);
      return launch_generic_w8a8(xq, w, w_scale, zp, x_scale, xq_rowsum, acc_out, out, out_dtype, M, N, K, st);
    case QMM_VARIANT_TCGEN05:
      log_choice("w8a8_gemm", "tcgen05", M, N, K);
      return launch_w8a8_tc(xq, w, w_scale, zp, x_scale, xq_rowsum, acc_out, out, out_dtype, M, N, K, st);
    default:
      return fail(QMM_ERR_UNSUPPORTED, "w8a8_gemm: variant %d is not available", variant);
  }
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t qmm_workspace_size(int op, int64_t M, int64_t N, int64_t K) {
  (void)N;
  if (op == QMM_OP_W8A8_PERCHANNEL) {
    if (M <= 0 || K < 0) return 0;
    // xq [M,K] int8 | x_scale [M] f32 | rowsum [M] i32, each 256-byte aligned
    return align_up((size_t)M * (size_t)K, 256) + 2 * align_up((size_t)M * 4, 256);
  }
  return 0;
}

int qmm_w8a8_perchannel(const void* x, int x_dtype, const int8_t* w, const float* w_scale,
                        const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                        int64_t K, int saturate, int variant, void* workspace,
                        size_t workspace_bytes, void* stream) {
  int rc = check_common(x, x_dtype, w, w_scale, out, out_dtype, M, N, K);
  if (rc != QMM_OK || M * N == 0) return rc;
  const size_t need = qmm_workspace_size(QMM_OP_W8A8_PERCHANNEL, M, N, K);
  if (!workspace || workspace_bytes < need)
    return fail(QMM_ERR_WORKSPACE, "w8a8_perchannel needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  if (!aligned(workspace, 256)) return fail(QMM_ERR_MISALIGNED, "workspace must be 256-byte aligned");
  uint8_t* base = reinterpret_cast<uint8_t*>(workspace);
  int8_t* xq = reinterpret_cast<int8_t*>(base);
  float* xs = reinterpret_cast<float*>(base + align_up((size_t)M * (size_t)K, 256));
  int32_t* rowsum = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(xs) + align_up((size_t)M * 4, 256));
  rc = qmm_quantize_activation(x, x_dtype, xq, xs, zp ? rowsum : nullptr, M, K, saturate, stream);
  if (rc != QMM_OK) return rc;
  return qmm_w8a8_gemm(xq, w, w_scale, zp, xs, zp ? rowsum : nullptr, nullptr, out, out_dtype, M, N, K,
                       variant, stream);
}

int qmm_pack_int4_nk(const int8_t* w, uint8_t* wp, int64_t N, int64_t K, void* stream) {
  if (N < 0 || K < 0 || K % 2 != 0) return fail(QMM_ERR_BAD_SHAPE, "pack_int4_nk: K must be even and sizes non-negative");
  if (N * K == 0) return QMM_OK;
  if (!w || !wp) return fail(QMM_ERR_NULL, "w or wp is NULL");
  return launch_pack_int4_nk(w, wp, N, K, as_stream(stream));
}

int qmm_pack_int4_sbn(const int8_t* w, uint8_t* wp, int64_t S, int64_t block_size, int64_t N,
                      void* stream) {
  if (S < 0 || block_size < 0 || N < 0 || (S * block_size) % 2 != 0)
    return fail(QMM_ERR_BAD_SHAPE, "pack_int4_sbn: K = S*block_size must be even and sizes non-negative");
  if (S * block_size * N == 0) return QMM_OK;
  if (!w || !wp) return fail(QMM_ERR_NULL, "w or wp is NULL");
  return launch_pack_int4_sbn(w, wp, S, block_size, N, as_stream(stream));
}

int qmm_unpack_int4_nk(const uint8_t* wp, int8_t* w, int64_t N, int64_t K, void* stream) {
  if (N < 0 || K < 0 || K % 2 != 0) return fail(QMM_ERR_BAD_SHAPE, "unpack_int4_nk: K must be even and sizes non-negative");
  if (N * K == 0) return QMM_OK;
  if (!w || !wp) return fail(QMM_ERR_NULL, "w or wp is NULL");
  return launch_unpack_int4_nk(wp, w, N, K, as_stream(stream));
}

int qmm_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]) {
  if (!ptr || !handle) return fail(QMM_ERR_NULL, "peer_buffer_create: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes ? bytes : 16);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    cudaGetLastError();
    return fail(QMM_ERR_DEVICE, "peer_buffer_create: %s", cudaGetErrorString(e));
  }
  memcpy(handle, &h, 64);
  *ptr = p;
  return QMM_OK;
}

int qmm_peer_buffer_open(const unsigned char handle[64], void** ptr) {
  if (!ptr || !handle) return fail(QMM_ERR_NULL, "peer_buffer_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_DEVICE, "peer_buffer_open: %s", cudaGetErrorString(e));
  }
  *ptr = p;
  return QMM_OK;
}

int qmm_peer_buffer_close(void* ptr) {
  if (!ptr) return QMM_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_DEVICE, "peer_buffer_close: %s", cudaGetErrorString(e));
  }
  return QMM_OK;
}

int qmm_peer_buffer_destroy(void* ptr) {
  if (!ptr) return QMM_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_DEVICE, "peer_buffer_destroy: %s", cudaGetErrorString(e));
  }
  return QMM_OK;
}

int qmm_allreduce_oneshot(void* const* data_ptrs, void* const* flag_ptrs, int rank, int world, uint32_t epoch, void* out,
                          int out_dtype, int64_t count, void* stream) {
  if (!data_ptrs || !flag_ptrs || !out) return fail(QMM_ERR_NULL, "allreduce_oneshot: null pointer");
  if (out_dtype != QMM_F32 && out_dtype != QMM_BF16 && out_dtype != QMM_F16)
    return fail(QMM_ERR_BAD_SHAPE, "allreduce_oneshot: bad out_dtype %d", out_dtype);
  return launch_peer_allreduce(data_ptrs, flag_ptrs, rank, world, epoch, out, out_dtype, count, as_stream(stream));
}

size_t qmm_rowparallel_buffer_bytes(int64_t max_M, int64_t N, int world) {
  if (max_M < 1 || N < 1 || world < 1) return 0;
  const size_t data = 2 * (size_t)world * (size_t)max_M * (size_t)N * sizeof(float);
  const size_t flags = ((size_t)world * (size_t)((N + 15) / 16) + 2) * sizeof(uint32_t);
  return (data + flags + 255) / 256 * 256;
}

int qmm_rowparallel_decode(int wbits, const void* x, int x_dtype, const void* w, const float* scale, void* out,
                           int out_dtype, int64_t M, int64_t N, int64_t K, int64_t block_size,
                           void* const* peer_bufs, int rank, int world, int64_t slot_floats, void* stream) {
  if (wbits != 4 && wbits != 8) return fail(QMM_ERR_BAD_SHAPE, "rowparallel_decode: wbits must be 4 or 8, got %d", wbits);
  if (!x || !w || !scale || !out || !peer_bufs) return fail(QMM_ERR_NULL, "rowparallel_decode: null pointer");
  if (M < 0 || N < 0 || K < 0) return fail(QMM_ERR_BAD_SHAPE, "rowparallel_decode: negative size");
  if (block_size < 0 || (block_size > 0 && K % block_size != 0))
    return fail(QMM_ERR_BAD_SHAPE, "rowparallel_decode: K (%lld) must be a multiple of block_size (%lld)", (long long)K,
                (long long)block_size);
  if (out_dtype != QMM_F32 && out_dtype != QMM_BF16 && out_dtype != QMM_F16)
    return fail(QMM_ERR_BAD_SHAPE, "rowparallel_decode: bad out_dtype %d", out_dtype);
  if (M == 0 || N == 0) return QMM_OK;
  log_choice("rowparallel_decode", "mma", M, N, K);
  return launch_decode_mma_allreduce(wbits, x, x_dtype, w, scale, out, out_dtype, M, N, K, block_size, peer_bufs, rank, world,
                                     slot_floats, as_stream(stream));
}

int qmm_device_error_flag(uint32_t* flag, void* stream) {
  if (!flag) return fail(QMM_ERR_NULL, "flag is NULL");
  uint32_t* word = device_error_word();
  if (!word) return fail(QMM_ERR_DEVICE, "no CUDA device or error word unavailable");
  cudaStream_t st = as_stream(stream);
  cudaError_t e = cudaMemcpyAsync(flag, word, sizeof(uint32_t), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(QMM_ERR_LAUNCH, "reading the device error word: %s", cudaGetErrorString(e));
  if (*flag != 0) {
    cudaMemsetAsync(word, 0, sizeof(uint32_t), st);
    return fail(QMM_ERR_TIMEOUT, "a device-side wait gave up (code %u, CTA %u)", *flag & 0xff, *flag >> 8);
  }
  return QMM_OK;
}

int qmm_stream_read(const void* p, size_t bytes, void* sink, void* stream) {
  return launch_stream_read(p, bytes, sink, as_stream(stream));
}

int qmm_set_activation_limbs(int limbs) {
  if (limbs != 0 && limbs != 3) return fail(QMM_ERR_BAD_SHAPE, "qmm_set_activation_limbs: 0 (by output type) or 3, got %d", limbs);
  limb_tc_set_limbs(limbs);
  return QMM_OK;
}

int qmm_set_peer_wait_limit(double seconds) {
  if (!(seconds > 0.0) || seconds > 60.0) return fail(QMM_ERR_BAD_SHAPE, "peer wait limit must be in (0, 60] seconds, got %g", seconds);
  g_peer_wait_cycles.store((long long)(seconds * 2.0e9), std::memory_order_relaxed);  // ~2 GHz SM clock
  return QMM_OK;
}

const char* qmm_variant_for(int op, int64_t M, int64_t N, int64_t K, int64_t block_size, int has_zp) {
  // Shape-only view of the AUTO heuristic (pointer alignment is assumed to be fine).
  const void* ok = reinterpret_cast<const void*>(uintptr_t(256));
  switch (op) {
    case QMM_OP_W8A16_PERCHANNEL:
    case QMM_OP_W4A16_BLOCKWISE_PACKED:
    case QMM_OP_W4A16_PERCHANNEL_PACKED: {
      const int wbits = op == QMM_OP_W8A16_PERCHANNEL ? 8 : 4;
      const int64_t bs = op == QMM_OP_W4A16_BLOCKWISE_PACKED ? block_size : 0;
      if (decode_mma_supported(wbits, M, N, K, bs, ok, QMM_BF16, ok, has_zp != 0)) return "mma";
      if (mixed_tc_shape_ok(wbits, M, N, K, bs, QMM_BF16, has_zp != 0)) return "tcgen05";
      if (gemv_nk_supported(wbits, M, N, K, bs, ok, QMM_BF16, ok)) return "gemv";
      return "generic";
    }
    case QMM_OP_BLOCKWISE_SBN:
      return "generic";
    case QMM_OP_W8A8_PERCHANNEL:
      return (M >= 16 && K % 16 == 0 && K >= 16) ? "tcgen05" : "generic";
    default:
      return "generic";
  }
}

}  // extern "C"
