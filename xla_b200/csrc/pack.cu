// int4 packing kernels: the device-side stand-in for the reference's CastInt4 node
// (torch_xla/csrc/ops/cast_int4.cpp:14-39), which narrows an int8 container to 4-bit storage.
// Packed layout: uint8 [N, K/2]; byte j of row n holds k = 2j in the low nibble and k = 2j+1 in
// the high nibble, two's complement.
#include "common.cuh"
#include "kernels.h"

namespace qmm {

namespace {

__global__ void pack_nk_kernel(const int8_t* __restrict__ w, uint8_t* __restrict__ wp,
                               int64_t total_bytes) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_bytes) return;
  const uint8_t lo = (uint8_t)w[2 * i] & 0xf;
  const uint8_t hi = (uint8_t)w[2 * i + 1] & 0xf;
  wp[i] = (uint8_t)(lo | (hi << 4));
}

// [S,bs,N] (N minor) -> [N,K/2].  A 32x64 tile of (n, k) goes through shared memory so that both
// the reads (along n) and the writes (along k) coalesce.
__global__ void pack_sbn_kernel(const int8_t* __restrict__ w, uint8_t* __restrict__ wp, int64_t K,
                                int64_t N) {
  __shared__ int8_t tile[64][33];
  const int64_t n_base = (int64_t)blockIdx.x * 32;
  const int64_t k_base = (int64_t)blockIdx.y * 64;
  for (int kk = threadIdx.y; kk < 64; kk += blockDim.y) {
    const int64_t k = k_base + kk, n = n_base + threadIdx.x;
    tile[kk][threadIdx.x] = (k < K && n < N) ? w[k * N + n] : (int8_t)0;
  }
  __syncthreads();
  // 32 rows of n, 32 packed bytes each
  for (int nn = threadIdx.y; nn < 32; nn += blockDim.y) {
    const int64_t n = n_base + nn;
    const int j = threadIdx.x;  // packed byte within the tile
    const int64_t k = k_base + 2 * j;
    if (n < N && k < K) {
      const uint8_t lo = (uint8_t)tile[2 * j][nn] & 0xf;
      const uint8_t hi = (uint8_t)tile[2 * j + 1][nn] & 0xf;
      wp[n * (K >> 1) + (k >> 1)] = (uint8_t)(lo | (hi << 4));
    }
  }
}

__global__ void unpack_nk_kernel(const uint8_t* __restrict__ wp, int8_t* __restrict__ w,
                                 int64_t total_bytes) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_bytes) return;
  const uint8_t b = wp[i];
  w[2 * i] = (int8_t)(((b & 0xf) ^ 8) - 8);
  w[2 * i + 1] = (int8_t)(((b >> 4) ^ 8) - 8);
}

}  // namespace

int launch_pack_int4_nk(const int8_t* w, uint8_t* wp, int64_t N, int64_t K, cudaStream_t st) {
  const int64_t total = N * (K / 2);
  if (total == 0) return QMM_OK;
  pack_nk_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(w, wp, total);
  return check_launch("pack_nk_kernel");
}

int launch_pack_int4_sbn(const int8_t* w, uint8_t* wp, int64_t S, int64_t bs, int64_t N,
                         cudaStream_t st) {
  const int64_t K = S * bs;
  if (K == 0 || N == 0) return QMM_OK;
  dim3 grid((unsigned)ceil_div(N, 32), (unsigned)ceil_div(K, 64));
  if (grid.y > 65535) return fail(QMM_ERR_UNSUPPORTED, "pack_int4_sbn: K too large");
  pack_sbn_kernel<<<grid, dim3(32, 8), 0, st>>>(w, wp, K, N);
  return check_launch("pack_sbn_kernel");
}

int launch_unpack_int4_nk(const uint8_t* wp, int8_t* w, int64_t N, int64_t K, cudaStream_t st) {
  const int64_t total = N * (K / 2);
  if (total == 0) return QMM_OK;
  unpack_nk_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(wp, w, total);
  return check_launch("unpack_nk_kernel");
}

}  // namespace qmm
