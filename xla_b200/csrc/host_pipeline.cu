// Host-buffer front end of the weight-only linears.
//
// The device entry points take device pointers and a stream; a caller whose activations live in host memory
// (a serving front end that receives them over the network, a data loader) pays one copy in and one copy out per
// call, and when every call is enqueued from Python the host time of the five or six runtime calls around the
// kernel exceeds the kernel itself.  A pipeline object does the whole round trip in ONE call of this library:
// copy-in on its own stream, the linear on a second, copy-out on a third, handed over by events, with a ring
// of `depth` device staging slots so that the copy-in of call i+1 and the copy-out of call i-1 overlap the
// kernel of call i.  A submit returns as soon as its work is enqueued; the result is in the caller's host
// buffer after qmm_host_pipeline_sync.  Host buffers should be page-locked: with pageable memory the copies
// still work but stop overlapping.
//
// All device memory is allocated when the pipeline is created; a submit never allocates.
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace {

struct HostPipeline {
  int device = -1;
  int depth = 0;
  size_t x_bytes = 0, out_bytes = 0;
  cudaStream_t s_in = nullptr, s_k = nullptr, s_out = nullptr;
  std::vector<void*> xd, yd;
  std::vector<cudaEvent_t> ev_in, ev_k, ev_out;
  cudaEvent_t ev_dep = nullptr;  // orders the kernel stream after work the caller enqueued elsewhere
  void* ws = nullptr;            // scratch of the split-activation tensor-core kernel (zero-filled once)
  size_t ws_bytes = 0;
  unsigned long long calls = 0;
};

void release(HostPipeline* p) {
  for (void* q : p->xd)
    if (q) cudaFree(q);
  for (void* q : p->yd)
    if (q) cudaFree(q);
  for (auto* v : {&p->ev_in, &p->ev_k, &p->ev_out})
    for (cudaEvent_t e : *v)
      if (e) cudaEventDestroy(e);
  if (p->ev_dep) cudaEventDestroy(p->ev_dep);
  if (p->ws) cudaFree(p->ws);
  for (cudaStream_t s : {p->s_in, p->s_k, p->s_out})
    if (s) cudaStreamDestroy(s);
  delete p;
}

size_t dtype_bytes(int dt) { return dt == QMM_F32 ? 4 : 2; }

}  // namespace

extern "C" int qmm_host_pipeline_create(size_t max_x_bytes, size_t max_out_bytes, int depth, void** pipeline) {
  if (!pipeline) return qmm::fail(QMM_ERR_NULL, "host_pipeline_create: null pointer");
  if (depth < 1 || depth > 64 || max_x_bytes == 0 || max_out_bytes == 0)
    return qmm::fail(QMM_ERR_BAD_SHAPE, "host_pipeline_create: depth %d (1..64), %zu / %zu staging bytes", depth, max_x_bytes,
                     max_out_bytes);
  auto* p = new HostPipeline();
  p->depth = depth;
  p->x_bytes = max_x_bytes;
  p->out_bytes = max_out_bytes;
  p->xd.assign(depth, nullptr);
  p->yd.assign(depth, nullptr);
  p->ev_in.assign(depth, nullptr);
  p->ev_k.assign(depth, nullptr);
  p->ev_out.assign(depth, nullptr);
  cudaError_t e = cudaGetDevice(&p->device);
  for (cudaStream_t* s : {&p->s_in, &p->s_k, &p->s_out})
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(s, cudaStreamNonBlocking);
  for (int i = 0; i < depth && e == cudaSuccess; ++i) {
    e = cudaMalloc(&p->xd[i], max_x_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&p->yd[i], max_out_bytes);
    for (auto* v : {&p->ev_in, &p->ev_k, &p->ev_out})
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&(*v)[i], cudaEventDisableTiming);
  }
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->ev_dep, cudaEventDisableTiming);
  if (e == cudaSuccess) {
    // scratch for the kernels that want it: limbs of at most max_x_bytes / 2 activations (three bytes each), the
    // per-CTA partial tiles and the flag words; one buffer serves every call because the kernel stream orders them
    p->ws_bytes = 3 * (max_x_bytes / 2) + (size_t)qmm::kLimbMaxCtas * 64 * 128 * 4 + 8192;
    e = cudaMalloc(&p->ws, p->ws_bytes);
    if (e == cudaSuccess) e = cudaMemset(p->ws, 0, p->ws_bytes);
  }
  if (e != cudaSuccess) {
    release(p);
    cudaGetLastError();
    return qmm::fail(QMM_ERR_DEVICE, "host_pipeline_create: %s", cudaGetErrorString(e));
  }
  *pipeline = p;
  return QMM_OK;
}

extern "C" int qmm_host_pipeline_sync(void* pipeline) {
  if (!pipeline) return qmm::fail(QMM_ERR_NULL, "host_pipeline_sync: null pipeline");
  auto* p = static_cast<HostPipeline*>(pipeline);
  cudaError_t e = cudaStreamSynchronize(p->s_out);
  if (e == cudaSuccess) e = cudaStreamSynchronize(p->s_k);
  if (e != cudaSuccess) return qmm::fail(QMM_ERR_DEVICE, "host_pipeline_sync: %s", cudaGetErrorString(e));
  return QMM_OK;
}

extern "C" int qmm_host_pipeline_wait_stream(void* pipeline, void* stream) {
  if (!pipeline) return qmm::fail(QMM_ERR_NULL, "host_pipeline_wait_stream: null pipeline");
  auto* p = static_cast<HostPipeline*>(pipeline);
  cudaError_t e = cudaEventRecord(p->ev_dep, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamWaitEvent(p->s_k, p->ev_dep, 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return qmm::fail(QMM_ERR_DEVICE, "host_pipeline_wait_stream: %s", cudaGetErrorString(e));
  }
  return QMM_OK;
}

extern "C" int qmm_host_pipeline_destroy(void* pipeline) {
  if (!pipeline) return QMM_OK;
  auto* p = static_cast<HostPipeline*>(pipeline);
  cudaStreamSynchronize(p->s_in);
  cudaStreamSynchronize(p->s_k);
  cudaStreamSynchronize(p->s_out);
  release(p);
  return QMM_OK;
}

extern "C" int qmm_host_weight_only(void* pipeline, int layout, const void* x_host, int x_dtype, const void* w,
                                    const float* scale, const float* zp, void* out_host, int out_dtype, int64_t M,
                                    int64_t N, int64_t K, int64_t block_size, int variant) {
  if (!pipeline) return qmm::fail(QMM_ERR_NULL, "host_weight_only: null pipeline");
  if (M < 0 || N < 0 || K < 0) return qmm::fail(QMM_ERR_BAD_SHAPE, "negative dimension");
  if (x_dtype != QMM_F32 && x_dtype != QMM_BF16 && x_dtype != QMM_F16) return qmm::fail(QMM_ERR_UNSUPPORTED, "host_weight_only: x dtype %d", x_dtype);
  if (out_dtype != QMM_F32 && out_dtype != QMM_BF16 && out_dtype != QMM_F16)
    return qmm::fail(QMM_ERR_UNSUPPORTED, "host_weight_only: out dtype %d", out_dtype);
  auto* p = static_cast<HostPipeline*>(pipeline);
  const size_t xb = (size_t)M * K * dtype_bytes(x_dtype), ob = (size_t)M * N * dtype_bytes(out_dtype);
  if (xb > p->x_bytes || ob > p->out_bytes)
    return qmm::fail(QMM_ERR_WORKSPACE, "host_weight_only: the call needs %zu + %zu staging bytes, the pipeline has %zu + %zu", xb, ob,
                     p->x_bytes, p->out_bytes);
  if (M * N == 0) return QMM_OK;  // an empty call is a no-op, as in the device entry points
  if (!x_host || !out_host) return qmm::fail(QMM_ERR_NULL, "host_weight_only: null host buffer");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != p->device)
    return qmm::fail(QMM_ERR_DEVICE, "host_weight_only: the pipeline belongs to device %d, current device is %d", p->device, dev);
  const int slot = (int)(p->calls % (unsigned long long)p->depth);
  cudaError_t e = cudaSuccess;
  // the slot's previous result must have left the device before its staging buffers are reused
  if (p->calls >= (unsigned long long)p->depth) e = cudaEventSynchronize(p->ev_out[slot]);
  if (e == cudaSuccess) e = cudaMemcpyAsync(p->xd[slot], x_host, xb, cudaMemcpyHostToDevice, p->s_in);
  if (e == cudaSuccess) e = cudaEventRecord(p->ev_in[slot], p->s_in);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(p->s_k, p->ev_in[slot], 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return qmm::fail(QMM_ERR_DEVICE, "host_weight_only: copy-in: %s", cudaGetErrorString(e));
  }
  int wbits, blockwise;
  switch (layout) {
    case QMM_HOST_W4_BLOCKWISE_PACKED: wbits = 4; blockwise = 1; break;
    case QMM_HOST_W4_PERCHANNEL_PACKED: wbits = 4; blockwise = 0; break;
    case QMM_HOST_W8_PERCHANNEL: wbits = 8; blockwise = 0; break;
    case QMM_HOST_W8_BLOCKWISE_KMINOR: wbits = 8; blockwise = 1; break;
    default: return qmm::fail(QMM_ERR_UNSUPPORTED, "host_weight_only: unknown weight layout %d", layout);
  }
  if (blockwise && block_size <= 0) return qmm::fail(QMM_ERR_BAD_SHAPE, "host_weight_only: blockwise layout needs block_size > 0");
  const size_t ws_need = qmm_weight_only_workspace_size(M, K);
  const bool ws_ok = ws_need > 0 && ws_need <= p->ws_bytes;
  const int rc = qmm_weight_only(wbits, p->xd[slot], x_dtype, w, scale, zp, p->yd[slot], out_dtype, M, N, K, blockwise ? block_size : 0,
                                 variant, ws_ok ? p->ws : nullptr, ws_ok ? p->ws_bytes : 0, p->s_k);
  if (rc != QMM_OK) return rc;
  e = cudaEventRecord(p->ev_k[slot], p->s_k);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(p->s_out, p->ev_k[slot], 0);
  if (e == cudaSuccess) e = cudaMemcpyAsync(out_host, p->yd[slot], ob, cudaMemcpyDeviceToHost, p->s_out);
  if (e == cudaSuccess) e = cudaEventRecord(p->ev_out[slot], p->s_out);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return qmm::fail(QMM_ERR_DEVICE, "host_weight_only: copy-out: %s", cudaGetErrorString(e));
  }
  ++p->calls;
  return QMM_OK;
}
