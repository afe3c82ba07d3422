// Weight-only (W8A16 / W4A16) linear on the tensor cores, for every batch size from decode to
// prefill:  out[m,n] = sum_b scale[b,n] * (sum_{k in block b} x[m,k] * w[n,k])
// (per-channel scales are the one-block case).  Weights are K-minor: int8 [N,K] or packed int4
// [N,K/2] (low nibble = even k).
//
// Replaces the reference's mixed-dtype dot and its blockwise einsum pair
// (torch_xla/experimental/xla_quantized_matmul.py:113-114, :120-124; XLA lowering
// torch_xla/csrc/xla_lower_util.cpp:477-481).
//
// "Swap-AB" orientation: the 128 weight rows of a CTA are the MMA M side, the token batch is the
// MMA N side (16..256), so a decode batch of 1..16 tokens still fills a legal tcgen05 shape and the
// kernel stays a pure weight stream.  Per CTA (12 warps):
//   warp 0       TMA: raw weight bytes, 128 rows x 128 B per stage (128B swizzle)
//   warp 1       MMA issuer (tcgen05.mma.kind::f16, M128 x N=MP x K16), owns the TMEM allocation
//   warp 2       TMA: activation tiles [MP x 64] (zero-filled beyond M / K)
//   warps 4..7   dequant: thread r converts row r of the raw stage to the activation dtype, exactly
//                (integers up to 256 are exact in bf16 and fp16), and writes the 128B-swizzled
//                K-major operand tile the MMA reads; no scale is applied here
//   warps 8..11  drain: after each scale block, tcgen05.ld the block's partial sums and fold them into
//                fp32 register accumulators with scale[b,n] - the reference's "dot per block, then
//                scale, then sum", in fp32; two TMEM buffers overlap drain and MMA
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace qmm {

namespace {

constexpr int BMW = 128;          // weight rows per CTA (UMMA M)
constexpr int BK = 64;            // k per operand tile (64 x 2 B = one 128-byte swizzle row)
constexpr int UMMA_K = 16;
constexpr int kAStages = 4;       // 16 KB each
constexpr int kRawBytes = BMW * 128;
constexpr int kABytes = BMW * BK * 2;
constexpr int kThreads = 384;

struct Params {
  const float* scale;
  void* out;
  int out_dt;
  int64_t M, N, K;
  int k_tiles;          // ceil(K / 64)
  int tiles_per_block;  // block_size / 64, or k_tiles for per-channel
  int blockwise;
  uint32_t* err_word;
  long long* trace;  // optional pipeline timestamps of CTA (0,0), see qmm_debug_set_trace
};

// Per-role event log: role r writes clock64() stamps to trace[r * kTraceStride + i].
constexpr int kTraceStride = 1024;
__device__ __forceinline__ void stamp(const Params& p, int role, int& idx) {
  if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && idx < kTraceStride) p.trace[role * kTraceStride + idx++] = clock64();
}

// Ring depths per token-tile width: decode tiles are HBM-bound and want a deep raw-weight ring; wide
// prefill tiles are tensor-bound and spend the shared memory on activation tiles instead.
template <int MP>
struct Rings {
  static constexpr int kRawStages = MP <= 64 ? 4 : (MP == 128 ? 3 : 2);  // 16 KB each
  static constexpr int kBStages = MP <= 64 ? 8 : (MP == 128 ? 4 : 3);    // MP x 128 B each
};

template <int MP>
constexpr size_t smem_bytes() {
  return 1024 + (size_t)Rings<MP>::kRawStages * kRawBytes + (size_t)kAStages * kABytes +
         (size_t)Rings<MP>::kBStages * MP * 128 + 512;
}

// ---- exact integer -> 16-bit float conversions, natural k order --------------------------------

// 4 bytes (offset binary u = v + 128 after the XOR) -> two packed pairs of XT.
template <typename XT>
__device__ __forceinline__ void cvt_s8x4(uint32_t w, uint32_t& p01, uint32_t& p23);

template <>
__device__ __forceinline__ void cvt_s8x4<__half>(uint32_t w, uint32_t& p01, uint32_t& p23) {
  const uint32_t u = w ^ 0x80808080u;
  // byte b under exponent byte 0x64 reads 1024 + b in fp16
  uint32_t a = __byte_perm(u, 0x64646464u, 0x4140);
  uint32_t b = __byte_perm(u, 0x64646464u, 0x4342);
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
  __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), bias);
  __half2 hb = __hsub2(*reinterpret_cast<__half2*>(&b), bias);
  p01 = *reinterpret_cast<uint32_t*>(&ha);
  p23 = *reinterpret_cast<uint32_t*>(&hb);
}

template <>
__device__ __forceinline__ void cvt_s8x4<__nv_bfloat16>(uint32_t w, uint32_t& p01, uint32_t& p23) {
  // bf16 has no 8-bit mantissa to drop a byte into: go through fp32 (byte under 2^23) and round-pack;
  // every int8 is exact in bf16, so the pack does not round.
  const uint32_t u = w ^ 0x80808080u;
  const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.f;
  const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.f;
  const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.f;
  const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.f;
  __nv_bfloat162 a = __floats2bfloat162_rn(f0, f1);
  __nv_bfloat162 b = __floats2bfloat162_rn(f2, f3);
  p01 = *reinterpret_cast<uint32_t*>(&a);
  p23 = *reinterpret_cast<uint32_t*>(&b);
}

// 8 nibbles of a word (nibble i = k offset i, two's complement) -> four packed pairs of XT,
// (k0,k1) (k2,k3) (k4,k5) (k6,k7).  XOR makes offset binary u = v + 8; the nibbles are spread to
// bytes, interleaved back into k order, dropped under the exponent byte of 128.0 (bf16) or 1024.0
// (fp16), and the bias is removed with one packed subtraction.
template <typename XT>
__device__ __forceinline__ void cvt_s4x8(uint32_t w, uint32_t* p) {
  constexpr bool kBf16 = !std::is_same<XT, __half>::value;
  const uint32_t u = w ^ 0x88888888u;
  const uint32_t lo = u & 0x0F0F0F0Fu;         // k0 k2 k4 k6
  const uint32_t hi = (u >> 4) & 0x0F0F0F0Fu;  // k1 k3 k5 k7
  const uint32_t q0 = __byte_perm(lo, hi, 0x5140);  // k0 k1 k2 k3
  const uint32_t q1 = __byte_perm(lo, hi, 0x7362);  // k4 k5 k6 k7
  const uint32_t expo = kBf16 ? 0x43434343u : 0x64646464u;
  uint32_t r0 = __byte_perm(q0, expo, 0x4140);
  uint32_t r1 = __byte_perm(q0, expo, 0x4342);
  uint32_t r2 = __byte_perm(q1, expo, 0x4140);
  uint32_t r3 = __byte_perm(q1, expo, 0x4342);
  if (kBf16) {
    const __nv_bfloat162 bias = __floats2bfloat162_rn(136.f, 136.f);
    __nv_bfloat162 h0 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&r0), bias);
    __nv_bfloat162 h1 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&r1), bias);
    __nv_bfloat162 h2 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&r2), bias);
    __nv_bfloat162 h3 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&r3), bias);
    p[0] = *reinterpret_cast<uint32_t*>(&h0);
    p[1] = *reinterpret_cast<uint32_t*>(&h1);
    p[2] = *reinterpret_cast<uint32_t*>(&h2);
    p[3] = *reinterpret_cast<uint32_t*>(&h3);
  } else {
    const __half2 bias = __floats2half2_rn(1032.f, 1032.f);
    __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&r0), bias);
    __half2 h1 = __hsub2(*reinterpret_cast<__half2*>(&r1), bias);
    __half2 h2 = __hsub2(*reinterpret_cast<__half2*>(&r2), bias);
    __half2 h3 = __hsub2(*reinterpret_cast<__half2*>(&r3), bias);
    p[0] = *reinterpret_cast<uint32_t*>(&h0);
    p[1] = *reinterpret_cast<uint32_t*>(&h1);
    p[2] = *reinterpret_cast<uint32_t*>(&h2);
    p[3] = *reinterpret_cast<uint32_t*>(&h3);
  }
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// WBITS 4|8; XT activation dtype (bf16|f16) = operand format of both MMA sides; MP = MMA N (tokens).
template <int WBITS, typename XT, int MP>
__global__ void __launch_bounds__(kThreads, 1)
    mixed_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const Params p) {
  constexpr int TPR = (WBITS == 4) ? 4 : 2;  // operand tiles produced per raw stage
  constexpr uint32_t kBBytes = MP * 128;
  constexpr uint32_t kTmemCols = (2 * MP < 32) ? 32 : 2 * MP;
  constexpr bool kIsBf16 = !std::is_same<XT, __half>::value;
  constexpr int kRawStages = Rings<MP>::kRawStages;
  constexpr int kBStages = Rings<MP>::kBStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* raw_base = smem;
  uint8_t* a_base = raw_base + (size_t)kRawStages * kRawBytes;
  uint8_t* b_base = a_base + (size_t)kAStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_base + (size_t)kBStages * kBBytes);
  uint64_t* raw_full = bars;                    // [kRawStages] TMA bytes
  uint64_t* raw_empty = raw_full + kRawStages;  // [kRawStages] 4 dequant warps
  uint64_t* a_full = raw_empty + kRawStages;    // [kAStages]   4 dequant warps
  uint64_t* a_empty = a_full + kAStages;        // [kAStages]   tcgen05.commit
  uint64_t* b_full = a_empty + kAStages;        // [kBStages]   TMA bytes
  uint64_t* b_empty = b_full + kBStages;        // [kBStages]   tcgen05.commit
  uint64_t* acc_full = b_empty + kBStages;      // [2]          tcgen05.commit
  uint64_t* acc_empty = acc_full + 2;           // [2]          4 drain warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n0 = (int64_t)blockIdx.x * BMW;
  const int64_t m0 = (int64_t)blockIdx.y * MP;
  const int k_tiles = p.k_tiles;
  const int n_raw = (k_tiles + TPR - 1) / TPR;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      ptx::mbar_init(&raw_full[s], 1);
      ptx::mbar_init(&raw_empty[s], 4);
    }
    for (int s = 0; s < kAStages; ++s) {
      ptx::mbar_init(&a_full[s], 4);
      ptx::mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < kBStages; ++s) {
      ptx::mbar_init(&b_full[s], 1);
      ptx::mbar_init(&b_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&acc_full[s], 1);
      ptx::mbar_init(&acc_empty[s], 4);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_w);
    ptx::prefetch_tensormap(&map_x);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- raw weight producer ----------------
    if (lane == 0) {
      int ti = 0;
      for (int r = 0; r < n_raw; ++r) {
        const int s = r % kRawStages;
        ptx::mbar_wait(&raw_empty[s], ((r / kRawStages) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
        stamp(p, 3, ti);
        ptx::mbar_expect_tx(&raw_full[s], kRawBytes);
        ptx::tma_load_2d(raw_base + (size_t)s * kRawBytes, &map_w, &raw_full[s], r * 128, (int32_t)n0);
      }
    }
  } else if (warp == 2) {
    // ---------------- activation tile producer ----------------
    if (lane == 0) {
      for (int t = 0; t < k_tiles; ++t) {
        const int s = t % kBStages;
        ptx::mbar_wait(&b_empty[s], ((t / kBStages) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
        ptx::mbar_expect_tx(&b_full[s], kBBytes);
        ptx::tma_load_2d(b_base + (size_t)s * kBBytes, &map_x, &b_full[s], t * BK, (int32_t)m0);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t fmt = kIsBf16 ? 1u : 0u;
      constexpr uint32_t idesc = ptx::make_idesc(/*f32*/ 1, fmt, fmt, BMW, MP);
      int blk = 0, in_blk = 0, ti = 0;
      for (int t = 0; t < k_tiles; ++t) {
        const int buf = blk & 1;
        if (in_blk == 0) {
          ptx::mbar_wait(&acc_empty[buf], ((blk >> 1) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitTmemEmpty);
          ptx::tcgen05_fence_after();
        }
        const int sa = t % kAStages, sb = t % kBStages;
        stamp(p, 1, ti);
        ptx::mbar_wait(&a_full[sa], (t / kAStages) & 1, abort_flag, p.err_word, ptx::kErrWaitConv);
        stamp(p, 1, ti);
        ptx::mbar_wait(&b_full[sb], (t / kBStages) & 1, abort_flag, p.err_word, ptx::kErrWaitFull);
        stamp(p, 1, ti);
        ptx::tcgen05_fence_after();
        stamp(p, 1, ti);
        const uint32_t a_addr = ptx::smem_u32(a_base + (size_t)sa * kABytes);
        const uint32_t b_addr = ptx::smem_u32(b_base + (size_t)sb * kBBytes);
        const uint32_t d_tmem = tmem_base + buf * MP;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          ptx::mma_f16_ss(d_tmem, ptx::make_sw128_kmajor_desc(a_addr + k * UMMA_K * 2),
                          ptx::make_sw128_kmajor_desc(b_addr + k * UMMA_K * 2), idesc, (in_blk | k) != 0 ? 1u : 0u);
          stamp(p, 1, ti);
        }
        ptx::mma_commit(&a_empty[sa]);
        stamp(p, 1, ti);
        ptx::mma_commit(&b_empty[sb]);
        stamp(p, 1, ti);
        ++in_blk;
        if (in_blk == p.tiles_per_block || t == k_tiles - 1) {
          ptx::mma_commit(&acc_full[buf]);
          in_blk = 0;
          ++blk;
        }
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ---------------- dequant: thread r owns weight row r of the stage ----------------
    const int r = threadIdx.x - 128;
    const uint32_t sw = (uint32_t)(r & 7);
    int t = 0;  // operand tile counter
    int ti = 0;
    const bool tracer = (threadIdx.x == 128);
    for (int rs = 0; rs < n_raw; ++rs) {
      const int s = rs % kRawStages;
      ptx::mbar_wait_warp(&raw_full[s], (rs / kRawStages) & 1, abort_flag, p.err_word, ptx::kErrWaitRaw);
      const uint32_t raw_row = ptx::smem_u32(raw_base + (size_t)s * kRawBytes) + r * 128;
#pragma unroll
      for (int a = 0; a < TPR; ++a, ++t) {
        if (t >= k_tiles) break;
        const int sa = t % kAStages;
        if (tracer) stamp(p, 0, ti);
        ptx::mbar_wait_warp(&a_empty[sa], ((t / kAStages) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
        if (tracer) stamp(p, 0, ti);
        const uint32_t a_row = ptx::smem_u32(a_base + (size_t)sa * kABytes) + r * 128;
        if (WBITS == 4) {
          // two raw chunks (32 nibbles each) -> eight operand chunks (8 values each)
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const uint4 v = lds128(raw_row + (((uint32_t)(2 * a + jj) ^ sw) << 4));
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              uint32_t pk[4];
              cvt_s4x8<XT>(words[wi], pk);
              sts128(a_row + (((uint32_t)(jj * 4 + wi) ^ sw) << 4), pk[0], pk[1], pk[2], pk[3]);
            }
          }
        } else {
          // four raw chunks (16 bytes each) -> eight operand chunks
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const uint4 v = lds128(raw_row + (((uint32_t)(4 * a + jj) ^ sw) << 4));
            uint32_t q0, q1, q2, q3;
            cvt_s8x4<XT>(v.x, q0, q1);
            cvt_s8x4<XT>(v.y, q2, q3);
            sts128(a_row + (((uint32_t)(jj * 2) ^ sw) << 4), q0, q1, q2, q3);
            cvt_s8x4<XT>(v.z, q0, q1);
            cvt_s8x4<XT>(v.w, q2, q3);
            sts128(a_row + (((uint32_t)(jj * 2 + 1) ^ sw) << 4), q0, q1, q2, q3);
          }
        }
        if (tracer) stamp(p, 0, ti);
        ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the MMA's async proxy
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&a_full[sa]);
        if (tracer) stamp(p, 0, ti);
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&raw_empty[s]);
    }
  } else if (warp >= 8) {
    // ---------------- drain / epilogue: thread owns output column n = n0 + its TMEM lane ----------------
    const int quad = warp & 3;
    const int64_t n = n0 + quad * 32 + lane;
    const bool n_ok = n < p.N;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int n_blocks = (k_tiles + p.tiles_per_block - 1) / p.tiles_per_block;
    if constexpr (MP <= 64) {
      float acc[MP];
#pragma unroll
      for (int j = 0; j < MP; ++j) acc[j] = 0.f;
      int ti = 0;
      const bool tracer = (threadIdx.x == 256);
      for (int b = 0; b < n_blocks; ++b) {
        const int buf = b & 1;
        const float s = n_ok ? __ldg(p.scale + (p.blockwise ? (int64_t)b * p.N + n : n)) : 0.f;
        if (tracer) stamp(p, 2, ti);
        ptx::mbar_wait_warp(&acc_full[buf], (b >> 1) & 1, abort_flag, p.err_word, ptx::kErrWaitTmemFull);
        ptx::tcgen05_fence_after();
        if (tracer) stamp(p, 2, ti);
#pragma unroll
        for (int c = 0; c < MP / 16; ++c) {
          uint32_t rr[16];
          ptx::tmem_ld_32x32b_x16(lane_addr + buf * MP + c * 16, rr);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(s, __uint_as_float(rr[j]), acc[c * 16 + j]);
        }
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
        if (tracer) stamp(p, 2, ti);
      }
      if (n_ok) {
#pragma unroll
        for (int j = 0; j < MP; ++j)
          if (m0 + j < p.M) store_from_f32(p.out, (m0 + j) * p.N + n, p.out_dt, acc[j]);
      }
    } else {
      // large token tiles: one scale block only (per-channel); scale and store straight from TMEM
      const float s = n_ok ? __ldg(p.scale + n) : 0.f;
      ptx::mbar_wait_warp(&acc_full[0], 0, abort_flag, p.err_word, ptx::kErrWaitTmemFull);
      ptx::tcgen05_fence_after();
#pragma unroll 1
      for (int c = 0; c < MP / 32; ++c) {
        uint32_t rr[32];
        __syncwarp();
        ptx::tmem_ld_32x32b_x32(lane_addr + c * 32, rr);
        ptx::tmem_ld_wait();
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int64_t m = m0 + c * 32 + j;
            if (m < p.M) store_from_f32(p.out, m * p.N + n, p.out_dt, s * __uint_as_float(rr[j]));
          }
        }
      }
      ptx::tcgen05_fence_before();
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int WBITS, typename XT, int MP>
int launch_one(const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, dim3 grid, cudaStream_t st) {
  auto kern = mixed_tc_kernel<WBITS, XT, MP>;
  constexpr size_t smem = smem_bytes<MP>();
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(QMM_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  kern<<<grid, kThreads, smem, st>>>(map_w, map_x, p);
  return check_launch("mixed_tc_kernel");
}

template <int WBITS, typename XT>
int launch_mp(int mp, const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, dim3 grid,
              cudaStream_t st) {
  switch (mp) {
    case 16: return launch_one<WBITS, XT, 16>(map_w, map_x, p, grid, st);
    case 32: return launch_one<WBITS, XT, 32>(map_w, map_x, p, grid, st);
    case 64: return launch_one<WBITS, XT, 64>(map_w, map_x, p, grid, st);
    case 128: return launch_one<WBITS, XT, 128>(map_w, map_x, p, grid, st);
    default: return launch_one<WBITS, XT, 256>(map_w, map_x, p, grid, st);
  }
}

}  // namespace

bool mixed_tc_shape_ok(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, int x_dt, bool has_zp) {
  if (has_zp) return false;
  if (x_dt != QMM_BF16 && x_dt != QMM_F16) return false;
  if (M < 1 || N < 1 || K < 64) return false;
  if ((K * wbits / 8) % 16 != 0 || (K * 2) % 16 != 0) return false;  // TMA row pitches
  if (block_size > 0 && (block_size % BK != 0 || K % block_size != 0)) return false;
  if (M > (1 << 20) || N > (1 << 28) || K > (1 << 28)) return false;
  return true;
}

bool mixed_tc_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x,
                        int x_dt, const void* w, bool has_zp) {
  if (!mixed_tc_shape_ok(wbits, M, N, K, block_size, x_dt, has_zp)) return false;
  if (!aligned(x, 16) || !aligned(w, 16)) return false;
  return device_is_sm100();
}

int launch_mixed_tc(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out,
                    int out_dt, int64_t M, int64_t N, int64_t K, int64_t block_size, cudaStream_t st) {
  if (!mixed_tc_supported(wbits, M, N, K, block_size, x, x_dt, w, false))
    return fail(QMM_ERR_UNSUPPORTED,
                "weight-only tcgen05 kernel: needs an sm_100 device, bf16/f16 activations, K >= 64 with 16-byte "
                "row pitches, block_size a multiple of 64 (M=%lld N=%lld K=%lld bs=%lld)",
                (long long)M, (long long)N, (long long)K, (long long)block_size);
  const bool blockwise = block_size > 0;
  // token tile: blockwise partial sums live in registers (<= 64 columns per pass)
  int mp;
  if (M <= 16) mp = 16;
  else if (M <= 32) mp = 32;
  else if (M <= 64 || blockwise) mp = 64;
  else if (M <= 128) mp = 128;
  else mp = 256;
  CUtensorMap map_w, map_x;
  int rc = encode_tmap_2d(&map_w, w, 1, false, (uint64_t)N, (uint64_t)(K * wbits / 8), BMW, 128);
  if (rc != QMM_OK) return rc;
  rc = encode_tmap_2d(&map_x, x, 2, true, (uint64_t)M, (uint64_t)K, (uint32_t)mp, BK);
  if (rc != QMM_OK) return rc;
  Params p;
  p.scale = scale;
  p.out = out;
  p.out_dt = out_dt;
  p.M = M;
  p.N = N;
  p.K = K;
  p.k_tiles = (int)ceil_div(K, BK);
  p.tiles_per_block = blockwise ? (int)(block_size / BK) : p.k_tiles;
  p.blockwise = blockwise ? 1 : 0;
  p.err_word = device_error_word();
  p.trace = debug_trace_buffer();
  dim3 grid((unsigned)ceil_div(N, BMW), (unsigned)ceil_div(M, mp));
  if (grid.y > 65535) return fail(QMM_ERR_UNSUPPORTED, "weight-only tcgen05 kernel: M too large");
  if (wbits == 4) {
    if (x_dt == QMM_BF16) return launch_mp<4, __nv_bfloat16>(mp, map_w, map_x, p, grid, st);
    return launch_mp<4, __half>(mp, map_w, map_x, p, grid, st);
  }
  if (x_dt == QMM_BF16) return launch_mp<8, __nv_bfloat16>(mp, map_w, map_x, p, grid, st);
  return launch_mp<8, __half>(mp, map_w, map_x, p, grid, st);
}

}  // namespace qmm
