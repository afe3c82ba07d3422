// One-shot all-reduce (sum) of the row-parallel linear's fp32 partial results over peer memory.
//
// The reference attaches no collective to the quantized linear; under SPMD it would let XLA insert an
// all-reduce after the K-sharded matmul (torch_xla/csrc/cross_replica_reduces.cpp:154).  For decode batches
// the payload is a few KB and a library all-reduce is pure latency, so here every rank keeps its partial
// result in a buffer that its peers can read directly (CUDA IPC mapping over NVLink) and one kernel per GPU
// does the exchange:
//   1. signal: write this call's epoch into my flag slot on every peer (system-scope release),
//   2. wait (bounded) until every peer's epoch has arrived in my own flag array,
//   3. read the same slice of all G partial results with plain peer loads, add them in rank order in fp32
//      (so every rank computes bit-identical sums), convert and store locally.
// Two data slots alternate between calls: a rank may start writing call e+1's partial while a slow peer still
// reads call e's, and passing the barrier of call e+1 proves that every peer has finished call e.
// No multicast, no TMA, no unbounded spin: a wait that exceeds its budget (about a second by default,
// qmm_set_peer_wait_limit) records an error, fills the result with NaN and returns.
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "kernels.h"

namespace qmm {

namespace {

constexpr int kMaxRanks = 8;

struct PeerPtrs {
  const float* data[kMaxRanks];  // slot base of every rank's partial (index = rank)
  uint32_t* flags[kMaxRanks];    // every rank's flag array (kMaxRanks words)
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256)
    peer_allreduce_kernel(PeerPtrs pp, int rank, int world, uint32_t epoch_arg, void* __restrict__ out, int out_dt,
                          int64_t count, uint32_t* err_word, long long wait_cycles) {
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;
  // epoch_arg == 0: the call number lives in device memory (word 8 of my flag array), so that a captured
  // launch advances it on every replay.  Every block reads it before any block can bump it: the bump is done
  // by whichever block finishes last (ticket in word 9).
  uint32_t* my_ctr = pp.flags[rank] + kMaxRanks;
  if (threadIdx.x == 0) s_epoch = epoch_arg ? epoch_arg : *reinterpret_cast<volatile uint32_t*>(my_ctr) + 1u;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  // 1. tell every peer (and myself) that my partial of this call is complete: it was written by an earlier
  //    kernel of this stream, so it is already visible device-wide; the release makes that order system-wide
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(pp.flags[threadIdx.x] + rank, epoch);
  }
  // 2. one thread per block waits for all peers, bounded
  if (threadIdx.x == 0) {
    int ok = 1;
    const long long t0 = clock64();
    for (int r = 0; r < world && ok; ++r) {
      uint32_t spins = 0;
      while ((int32_t)(ld_acquire_sys(pp.flags[rank] + r) - epoch) < 0) {
        if ((++spins & 0x3ff) == 0 && clock64() - t0 > wait_cycles) {
          ok = 0;
          if (err_word) atomicCAS(err_word, 0u, 7u | ((uint32_t)r << 8));
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (threadIdx.x == 0 && !epoch_arg) {
    // every block has its epoch by now (it read the counter before arriving here)
    if (atomicAdd(my_ctr + 1, 1u) == gridDim.x - 1) {
      my_ctr[1] = 0;
      *reinterpret_cast<volatile uint32_t*>(my_ctr) = epoch;
    }
  }
  const int64_t nvec = count >> 2;
  if (!s_ok) {
    // a peer never arrived: the device error word says so; the result is filled with NaN so that a caller who does
    // not look at the word cannot mistake stale memory for a sum
    const float nan = __uint_as_float(0x7fc00000u);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
      store_from_f32(out, i, out_dt, nan);
    return;
  }
  // 3. reduce my copy of the whole result (every rank needs all of it: the next layer is replicated)
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = ld_peer_f4(pp.data[r] + 4 * i);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    store_from_f32(out, 4 * i, out_dt, acc.x);
    store_from_f32(out, 4 * i + 1, out_dt, acc.y);
    store_from_f32(out, 4 * i + 2, out_dt, acc.z);
    store_from_f32(out, 4 * i + 3, out_dt, acc.w);
  }
}

}  // namespace

int launch_peer_allreduce(void* const* data_ptrs, void* const* flag_ptrs, int rank, int world, uint32_t epoch, void* out,
                          int out_dt, int64_t count, cudaStream_t st) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(QMM_ERR_BAD_SHAPE, "peer all-reduce: rank %d of %d (at most %d ranks)", rank, world, kMaxRanks);
  if (count < 0 || count % 4 != 0) return fail(QMM_ERR_BAD_SHAPE, "peer all-reduce: count must be a multiple of 4, got %lld", (long long)count);
  if (count == 0) return QMM_OK;
  PeerPtrs pp;
  for (int r = 0; r < kMaxRanks; ++r) {
    pp.data[r] = r < world ? reinterpret_cast<const float*>(data_ptrs[r]) : nullptr;
    pp.flags[r] = r < world ? reinterpret_cast<uint32_t*>(flag_ptrs[r]) : nullptr;
    if (r < world && (!pp.data[r] || !pp.flags[r])) return fail(QMM_ERR_NULL, "peer all-reduce: null buffer of rank %d", r);
    if (r < world && !aligned(pp.data[r], 16)) return fail(QMM_ERR_MISALIGNED, "peer all-reduce: data of rank %d not 16-byte aligned", r);
  }
  const int64_t nvec = count / 4;
  int blocks = (int)std::min<int64_t>(ceil_div(nvec, 256), 2 * sm_count());
  if (blocks < 1) blocks = 1;
  peer_allreduce_kernel<<<blocks, 256, 0, st>>>(pp, rank, world, epoch, out, out_dt, count, device_error_word(), peer_wait_cycles());
  return check_launch("peer_allreduce_kernel");
}

}  // namespace qmm
