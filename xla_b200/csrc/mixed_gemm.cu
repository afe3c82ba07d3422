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
// MMA N side (16..256), so a small batch still fills a legal tcgen05 shape and the kernel stays a
// weight stream.  Per CTA (16 warps):
//   warp 0        TMA: raw weight bytes, 128 rows x 128 B per stage (128B swizzle)
//   warp 1        MMA issuer (tcgen05.mma.kind::f16, M128 x N=MP x K16), owns the TMEM allocation
//   warp 2        TMA: activation tiles [MP x 64] (zero-filled beyond M / K), several tiles per barrier
//   warps 4,6,7,8,10,11  dequant: each converts whole operand tiles on its own (all 128 rows of a
//                 64-wide k tile), exactly (integers up to 256 are exact in bf16 and fp16), into the
//                 128B-swizzled K-major tile the MMA reads; six tiles are in flight at once.  They avoid
//                 the scheduler partition of the MMA issuer (warps 5 and 9 stay idle)
//   warps 12..15  drain: after each scale block, tcgen05.ld the block's partial sums and fold them into
//                 fp32 register accumulators with scale[b,n] - the reference's "dot per block, then
//                 scale, then sum", in fp32; two TMEM buffers overlap drain and MMA
// Shapes with few weight rows (N/128 CTAs cannot fill 148 SMs) split K over a thread-block cluster:
// the CTAs of a cluster take consecutive K ranges of the same 128 rows and the non-leaders add their
// fp32 partials into the leader's shared memory (DSMEM) before the leader stores - deterministic,
// no global scratch.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace qmm {

namespace {

constexpr int BMW = 128;          // weight rows per CTA (UMMA M)
constexpr int BK = 64;            // k per operand tile (64 x 2 B = one 128-byte swizzle row)
constexpr int UMMA_K = 16;
constexpr int kDequantWarps = 6;
constexpr int kRawBytes = BMW * 128;
constexpr int kABytes = BMW * BK * 2;
constexpr int kThreads = 512;

struct Params {
  const float* scale;
  void* out;
  int out_dt;
  int64_t M, N, K;
  int k_tiles;          // ceil(K / 64)
  int tiles_per_block;  // block_size / 64, or k_tiles for per-channel
  int tiles_per_cta;    // k tiles each CTA of a cluster takes (== k_tiles without split-K)
  int blockwise;
  uint32_t* err_word;
};

// Ring depths per weight width and token-tile width.  Decode-sized tiles are HBM-bound: deep raw-weight
// and operand rings, activation tiles grouped per barrier.  Prefill-sized tiles are tensor-bound and spend
// the shared memory on activation tiles instead.
//
// mbarrier waits only tell "the phase with this parity is over", so a waiter must never be two phases
// ahead of a barrier.  The rings make that structural: every converting warp owns one operand slot
// (kAStages == converting warps), and a warp waits for its operand slot before its raw stage.
template <int WBITS, int MP>
struct Rings {
  static constexpr int kTilesPerRaw = (WBITS == 4) ? 4 : 2;
  static constexpr int kAStages = kDequantWarps;                          // 16 KB each, one per converting warp
  static constexpr int kRawStages = 4;                                    // 16 KB each
  static constexpr int kBGroup = MP <= 32 ? 4 : (MP <= 128 ? 2 : 1);      // activation tiles per barrier
  static constexpr int kBStages = MP == 64 ? 4 : 2;                       // groups in flight
  // the converting warp waits for its operand slot first (tile t-kAStages consumed, hence every raw
  // stage up to that tile has landed); that covers the previous generation of its raw slot if
  static_assert(kRawStages * kTilesPerRaw - kTilesPerRaw + 1 >= kAStages, "raw ring generation vs operand ring");
  static constexpr size_t kBytes = (size_t)kRawStages * kRawBytes + (size_t)kAStages * kABytes +
                                   (size_t)kBStages * kBGroup * MP * 128;
  static_assert(kBytes + 2048 <= 227 * 1024, "shared memory budget");
};

template <int WBITS, int MP>
constexpr size_t smem_bytes() {
  return 1024 + Rings<WBITS, MP>::kBytes + 1024;
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

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// WBITS 4|8; XT activation dtype (bf16|f16) = operand format of both MMA sides; MP = MMA N (tokens);
// KSPLIT: the kernel is launched as clusters of gridDim.z CTAs along K (MP <= 64 only).
template <int WBITS, typename XT, int MP, bool KSPLIT>
__global__ void __launch_bounds__(kThreads, 1)
    mixed_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const Params p) {
  constexpr int TPR = (WBITS == 4) ? 4 : 2;  // operand tiles produced per raw stage
  constexpr uint32_t kBBytes = MP * 128;
  constexpr uint32_t kTmemCols = (2 * MP < 32) ? 32 : 2 * MP;
  constexpr bool kIsBf16 = !std::is_same<XT, __half>::value;
  using R = Rings<WBITS, MP>;
  constexpr int kRawStages = R::kRawStages;
  constexpr int kAStages = R::kAStages;
  constexpr int kBGroup = R::kBGroup;
  constexpr int kBStages = R::kBStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* raw_base = smem;
  uint8_t* a_base = raw_base + (size_t)kRawStages * kRawBytes;
  uint8_t* b_base = a_base + (size_t)kAStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_base + (size_t)kBStages * kBGroup * kBBytes);
  uint64_t* raw_full = bars;                    // [kRawStages] TMA bytes
  uint64_t* raw_empty = raw_full + kRawStages;  // [kRawStages] one arrival per tile of the stage
  uint64_t* a_full = raw_empty + kRawStages;    // [kAStages]   the converting warp
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
  const uint32_t krank = KSPLIT ? cluster_ctarank() : 0u;
  const int tile0 = (int)krank * p.tiles_per_cta;  // first k tile of this CTA
  int my_tiles = p.k_tiles - tile0;
  if (my_tiles > p.tiles_per_cta) my_tiles = p.tiles_per_cta;
  if (my_tiles < 0) my_tiles = 0;
  const int n_raw = (my_tiles + TPR - 1) / TPR;
  const int n_groups = (my_tiles + kBGroup - 1) / kBGroup;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      ptx::mbar_init(&raw_full[s], 1);
      ptx::mbar_init(&raw_empty[s], TPR);
    }
    for (int s = 0; s < kAStages; ++s) {
      ptx::mbar_init(&a_full[s], 1);
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
      const int byte0 = tile0 * (BK * WBITS / 8);
      for (int r = 0; r < n_raw; ++r) {
        const int s = r % kRawStages;
        ptx::mbar_wait<64>(&raw_empty[s], ((r / kRawStages) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
        ptx::mbar_expect_tx(&raw_full[s], kRawBytes);
        ptx::tma_load_2d(raw_base + (size_t)s * kRawBytes, &map_w, &raw_full[s], byte0 + r * 128, (int32_t)n0);
      }
    }
  } else if (warp == 2) {
    // ---------------- activation tile producer: kBGroup tiles per barrier ----------------
    if (lane == 0) {
      for (int gidx = 0; gidx < n_groups; ++gidx) {
        const int s = gidx % kBStages;
        ptx::mbar_wait<64>(&b_empty[s], ((gidx / kBStages) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
        int cnt = my_tiles - gidx * kBGroup;
        if (cnt > kBGroup) cnt = kBGroup;
        ptx::mbar_expect_tx(&b_full[s], (uint32_t)cnt * kBBytes);
        for (int j = 0; j < cnt; ++j)
          ptx::tma_load_2d(b_base + ((size_t)s * kBGroup + j) * kBBytes, &map_x, &b_full[s],
                           (tile0 + gidx * kBGroup + j) * BK, (int32_t)m0);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop and waits together; one lane issues.  (A warp left diverged for
    // the length of the kernel - one lane looping, 31 parked at the final barrier - runs that lane at a
    // fraction of the normal issue rate.)
    {
      // Both operands carry the activation type: kind::f16 with A = f16 and B = bf16 is rejected by the
      // hardware (illegal instruction on B200), so int8 weights cannot take the cheaper fp16 conversion
      // when the activations are bf16.
      constexpr uint32_t fmt = kIsBf16 ? 1u : 0u;
      constexpr uint32_t idesc = ptx::make_idesc(/*f32*/ 1, fmt, fmt, BMW, MP);
      // descriptor halves: the high word is constant, the low word is the tile address >> 4
      const uint32_t desc_hi = (uint32_t)(ptx::make_sw128_kmajor_desc(0) >> 32);
      const uint32_t a_lo0 = (uint32_t)ptx::make_sw128_kmajor_desc(ptx::smem_u32(a_base));
      const uint32_t b_lo0 = (uint32_t)ptx::make_sw128_kmajor_desc(ptx::smem_u32(b_base));
      int blk = 0, in_blk = 0;
      const uint32_t leader = lane == 0 ? 1u : 0u;
      // ring positions advance with adds and compares only: this warp's instruction count per tile is what
      // bounds the kernel at small token tiles, and a division by a ring depth costs as much as an MMA issue
      int sa = 0, a_par = 0;           // operand slot of tile t and the parity of its current use
      int sb = 0, jb = 0, b_par = 0;   // activation group slot, tile inside the group, parity
      uint32_t a_lo = a_lo0, b_lo = b_lo0;
      for (int t = 0; t < my_tiles; ++t) {
        const int buf = blk & 1;
        if (in_blk == 0) {
          ptx::mbar_wait(&acc_empty[buf], ((blk >> 1) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitTmemEmpty);
          ptx::tcgen05_fence_after();  // the drain warps' tcgen05.ld of this buffer precede the overwrite
        }
        if (jb == 0) ptx::mbar_wait(&b_full[sb], b_par, abort_flag, p.err_word, ptx::kErrWaitFull);
        ptx::mbar_wait(&a_full[sa], a_par, abort_flag, p.err_word, ptx::kErrWaitConv);
        const bool last_in_block = (in_blk + 1 == p.tiles_per_block) || (t == my_tiles - 1);
        const uint32_t d_tmem = tmem_base + buf * MP;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t ad = ((uint64_t)desc_hi << 32) | (uint64_t)(a_lo + k * (UMMA_K * 2 >> 4));
          const uint64_t bd = ((uint64_t)desc_hi << 32) | (uint64_t)(b_lo + k * (UMMA_K * 2 >> 4));
          ptx::mma_f16_ss_pred(d_tmem, ad, bd, idesc, (in_blk | k) != 0 ? 1u : 0u, leader);
        }
        ptx::mma_commit_pred(&a_empty[sa], leader);
        const bool group_done = (jb == kBGroup - 1) || (t == my_tiles - 1);
        if (group_done) ptx::mma_commit_pred(&b_empty[sb], leader);
        if (last_in_block) ptx::mma_commit_pred(&acc_full[buf], leader);
        ++in_blk;
        if (last_in_block) {
          in_blk = 0;
          ++blk;
        }
        // next operand slot
        a_lo += kABytes >> 4;
        if (++sa == kAStages) {
          sa = 0;
          a_par ^= 1;
          a_lo = a_lo0;
        }
        // next activation tile
        b_lo += kBBytes >> 4;
        if (++jb == kBGroup) {
          jb = 0;
          if (++sb == kBStages) {
            sb = 0;
            b_par ^= 1;
            b_lo = b_lo0;
          }
        }
      }
    }
  } else if (warp >= 4 && warp < 12 && (warp & 3) != 1) {
    // ---------------- dequant: warp d owns operand tiles d, d+8, ...; lane owns rows lane+32i ----------------
    // Each active warp owns ONE ring slot (slot == warp index), see Rings.
    // The converting warps sit on the three scheduler partitions the MMA issuer (warp 1) is NOT on:
    // they are ALU-saturated and would starve its few, latency-critical instructions of issue slots.
    constexpr int kActive = kDequantWarps;
    constexpr int kChunks = (WBITS == 4) ? 2 : 4;  // 16-byte raw chunks per row per operand tile
    const int dw = (warp - 4) - ((warp - 4) + 3) / 4;  // warps 4,6,7,8,10,11 -> 0..5
    for (int t = dw; t < my_tiles; t += kActive) {
      const int rs = t / TPR, a = t % TPR;
      const int s = rs % kRawStages, sa = t % kAStages;
      ptx::mbar_wait_warp<64>(&a_empty[sa], ((t / kAStages) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
      ptx::mbar_wait_warp<64>(&raw_full[s], (rs / kRawStages) & 1, abort_flag, p.err_word, ptx::kErrWaitRaw);
      const uint8_t* raw_tile = raw_base + (size_t)s * kRawBytes;
      uint8_t* a_tile = a_base + (size_t)sa * kABytes;
      // all loads of the tile first (plain loads: the compiler may keep them in flight together), then
      // convert and store; the barrier waits above and the proxy fence below order them
      uint4 rawv[4][kChunks];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = lane + 32 * i;
#pragma unroll
        for (int jj = 0; jj < kChunks; ++jj)
          rawv[i][jj] = *reinterpret_cast<const uint4*>(raw_tile + r * 128 + (((kChunks * a + jj) ^ (r & 7)) << 4));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = lane + 32 * i;
        const int sw = r & 7;
        uint8_t* a_row = a_tile + r * 128;
        if (WBITS == 4) {
          // two raw chunks (32 nibbles each) -> eight operand chunks (8 values each)
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const uint32_t words[4] = {rawv[i][jj].x, rawv[i][jj].y, rawv[i][jj].z, rawv[i][jj].w};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              uint32_t pk[4];
              cvt_s4x8<XT>(words[wi], pk);
              *reinterpret_cast<uint4*>(a_row + (((jj * 4 + wi) ^ sw) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          }
        } else {
          // four raw chunks (16 bytes each) -> eight operand chunks
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const uint4 v = rawv[i][jj];
            uint32_t q0, q1, q2, q3;
            cvt_s8x4<XT>(v.x, q0, q1);
            cvt_s8x4<XT>(v.y, q2, q3);
            *reinterpret_cast<uint4*>(a_row + (((jj * 2) ^ sw) << 4)) = make_uint4(q0, q1, q2, q3);
            cvt_s8x4<XT>(v.z, q0, q1);
            cvt_s8x4<XT>(v.w, q2, q3);
            *reinterpret_cast<uint4*>(a_row + (((jj * 2 + 1) ^ sw) << 4)) = make_uint4(q0, q1, q2, q3);
          }
        }
      }
      ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the MMA's async proxy
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(&a_full[sa]);
        ptx::mbar_arrive(&raw_empty[s]);
      }
    }
  } else if (warp >= 12) {
    // ---------------- drain / epilogue: thread owns output column n = n0 + its TMEM lane ----------------
    const int quad = warp & 3;
    const int nl = quad * 32 + lane;
    const int64_t n = n0 + nl;
    const bool n_ok = n < p.N;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int n_blocks = (my_tiles + p.tiles_per_block - 1) / p.tiles_per_block;
    const int block0 = tile0 / p.tiles_per_block;
    if constexpr (MP <= 64) {
      float acc[MP];
#pragma unroll
      for (int j = 0; j < MP; ++j) acc[j] = 0.f;
      for (int b = 0; b < n_blocks; ++b) {
        const int buf = b & 1;
        const float s = n_ok ? (p.blockwise ? __ldg(p.scale + (int64_t)(block0 + b) * p.N + n) : 1.f) : 0.f;
        ptx::mbar_wait_warp<32>(&acc_full[buf], (b >> 1) & 1, abort_flag, p.err_word, ptx::kErrWaitTmemFull);
        ptx::tcgen05_fence_after();
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
      }
      if constexpr (KSPLIT) {
        // (1) every CTA of the cluster is past its main loop: the leader's rings may be overwritten
        __syncwarp();
        cluster_sync_all();
        if (krank != 0) {
          const uint32_t base = map_to_cta(ptx::smem_u32(smem), 0) + ((krank - 1) * MP * BMW + nl) * 4;
#pragma unroll
          for (int j = 0; j < MP; ++j) st_cluster_f32(base + j * BMW * 4, acc[j]);
        }
        // (2) partials have landed in the leader
        __syncwarp();
        cluster_sync_all();
        if (krank == 0) {
          const float* part = reinterpret_cast<const float*>(smem);
          const int ks = (int)gridDim.z;
          for (int z = 0; z < ks - 1; ++z)
#pragma unroll
            for (int j = 0; j < MP; ++j) acc[j] += part[(z * MP + j) * BMW + nl];
        }
      }
      if (n_ok && krank == 0) {
        const float ps = p.blockwise ? 1.f : __ldg(p.scale + n);
#pragma unroll
        for (int j = 0; j < MP; ++j)
          if (m0 + j < p.M) store_from_f32(p.out, (m0 + j) * p.N + n, p.out_dt, acc[j] * ps);
      }
    } else {
      // large token tiles: one scale block only (per-channel); scale and store straight from TMEM
      const float s = n_ok ? __ldg(p.scale + n) : 0.f;
      if (my_tiles > 0) {
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
  }
  if constexpr (KSPLIT) {
    // the warps that are not drain warps take part in the two cluster barriers as well
    if (warp < 12) {
      __syncwarp();
      cluster_sync_all();
      __syncwarp();
      cluster_sync_all();
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int WBITS, typename XT, int MP, bool KSPLIT>
int launch_one(const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, dim3 grid, cudaStream_t st) {
  auto kern = mixed_tc_kernel<WBITS, XT, MP, KSPLIT>;
  constexpr size_t smem = smem_bytes<WBITS, MP>();
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(QMM_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  if (KSPLIT) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = grid.z;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_w, map_x, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_LAUNCH, "mixed_tc_kernel launch: %s", cudaGetErrorString(e));
  }
  return check_launch("mixed_tc_kernel");
}

template <int WBITS, typename XT>
int launch_mp(int mp, bool ksplit, const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, dim3 grid,
              cudaStream_t st) {
  switch (mp) {
    case 16:
      return ksplit ? launch_one<WBITS, XT, 16, true>(map_w, map_x, p, grid, st)
                    : launch_one<WBITS, XT, 16, false>(map_w, map_x, p, grid, st);
    case 32:
      return ksplit ? launch_one<WBITS, XT, 32, true>(map_w, map_x, p, grid, st)
                    : launch_one<WBITS, XT, 32, false>(map_w, map_x, p, grid, st);
    case 64:
      return ksplit ? launch_one<WBITS, XT, 64, true>(map_w, map_x, p, grid, st)
                    : launch_one<WBITS, XT, 64, false>(map_w, map_x, p, grid, st);
    case 128: return launch_one<WBITS, XT, 128, false>(map_w, map_x, p, grid, st);
    default: return launch_one<WBITS, XT, 256, false>(map_w, map_x, p, grid, st);
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
  const int64_t n_tiles = ceil_div(N, BMW), m_tiles = ceil_div(M, mp);
  if (m_tiles > 65535) return fail(QMM_ERR_UNSUPPORTED, "weight-only tcgen05 kernel: M too large");
  // split K over a cluster when the (n, m) tiles alone leave most SMs idle; the leader needs room for
  // (ks-1) fp32 partial tiles of 128 x mp in the shared memory its rings used
  int ks = 1;
  if (mp <= 64) {
    const int64_t ctas = n_tiles * m_tiles;
    const int room = 1 + (int)((160 * 1024) / (mp * BMW * 4));
    while (ks < 8 && ks * 2 <= room && ctas * ks * 2 <= (int64_t)sm_count() &&
           p.k_tiles / (ks * 2) >= 4 * (blockwise ? p.tiles_per_block : 1))
      ks *= 2;
  }
  const int unit = blockwise ? p.tiles_per_block : 1;  // a CTA's K range holds whole scale blocks
  p.tiles_per_cta = (int)(ceil_div(ceil_div(p.k_tiles, ks), unit) * unit);
  if (!blockwise && ks > 1) p.tiles_per_block = p.tiles_per_cta;  // per-channel: one block per CTA
  if (!blockwise && ks == 1) p.tiles_per_cta = p.k_tiles;
  dim3 grid((unsigned)n_tiles, (unsigned)m_tiles, (unsigned)ks);
  if (wbits == 4) {
    if (x_dt == QMM_BF16) return launch_mp<4, __nv_bfloat16>(mp, ks > 1, map_w, map_x, p, grid, st);
    return launch_mp<4, __half>(mp, ks > 1, map_w, map_x, p, grid, st);
  }
  if (x_dt == QMM_BF16) return launch_mp<8, __nv_bfloat16>(mp, ks > 1, map_w, map_x, p, grid, st);
  return launch_mp<8, __half>(mp, ks > 1, map_w, map_x, p, grid, st);
}

}  // namespace qmm
