// Weight-only (W8A16 / W4A16) linear for token batches up to 32 on the tcgen05 tensor cores, built
// around one measured fact: a warp running this kind of code (integer conversion chains, barrier waits,
// predicated issue) retires about one instruction every 6-7 cycles, so throughput comes from many warps
// that each execute few instructions per weight, not from a faster pipe.
//
//   out[m,n] = sum_b scale[b,n] * (sum_{k in block b} x[m,k] * w[n,k])       (per-channel: one block)
//
// Replaces the reference's mixed-dtype dot and blockwise einsum pair
// (torch_xla/experimental/xla_quantized_matmul.py:113-114, :120-124, :152-170).
//
// Orientation: 128 weight rows are the MMA M side, the tokens the MMA N side (16 or 32).  The A operand
// (weights) never touches shared memory: each converting warp loads 32 rows x one 64-wide k tile straight
// from HBM into registers, converts exactly to bf16/f16 and writes its 32 lanes of the operand tile into
// TENSOR MEMORY with tcgen05.st; the MMA reads A from tensor memory and B (activations) from shared memory.
//
// Work split.  A cluster of S CTAs owns a set of 128-row blocks; CTA rank r of the cluster takes the K slice
// [r*K/S, (r+1)*K/S) of every block, so its slice of the activations is loaded once (TMA) and stays
// resident.  At the end the S partial results meet through distributed shared memory.
//
// Per CTA, 24 warps:
//   warps 0..3    MMA issuers: issuer w takes the scale blocks w, w+4, ... and alternates between two TMEM
//                 accumulators of its own (warp 0 also allocates TMEM and starts the activation TMA)
//   warps 4..19   four converting groups of four warps (one warp per TMEM lane quadrant): group w converts
//                 the k tiles of issuer w into its two operand slots in turn, so each slot's barriers are
//                 used by one converter group and one issuer, strictly in order
//   warps 20..23  drain: per scale block tcgen05.ld the partial sums, fold scale[b,n] * partial into fp32
//                 registers; per row block park the totals in shared memory for the cluster reduction
// Per-channel scales run through the same pipeline with blocks of two k tiles and unit block scales.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace qmm {

namespace {

constexpr int BMW = 128;   // weight rows per block (UMMA M)
constexpr int BK = 64;     // k per operand tile
constexpr int UMMA_K = 16;
constexpr int kGroups = 4;         // converting groups == operand slots in tensor memory (two per MMA issuer)
constexpr int kFirstConvWarp = 4;
constexpr int kFirstDrainWarp = kFirstConvWarp + 4 * kGroups;
constexpr int kWarps = kFirstDrainWarp + 4;
constexpr int kThreads = kWarps * 32;
constexpr int kIssuers = 4;
constexpr uint32_t kAccCols = 256;                // eight accumulators (two per MMA issuer) of up to 32 columns
constexpr uint32_t kSlotCols = BK / 2;            // 32 columns per operand slot (two 16-bit values per column)
constexpr int kSlots = 2 * kGroups;               // two operand slots per converting group
constexpr uint32_t kTmemCols = 512;               // 256 + 8 * 32
constexpr int kSmemCap = 200 * 1024;

struct Params {
  const uint8_t* w;
  const float* scale;
  void* out;
  int out_dt;
  int M, N, K;
  int64_t pitch;        // bytes per weight row
  int S;                // CTAs per cluster == K slices (1, 2, 4 or 8)
  int s_shift;          // log2(S)
  int kt_slice;         // k tiles per CTA and row block
  int tb;               // k tiles per scale block (a power of two)
  int tb_shift;
  int blockwise;
  int row_blocks;       // ceil(N / 128)
  int nclusters;
  int rounds;           // row blocks per cluster (ceil)
  int rounds_per_pass;  // row blocks whose partial sums fit in shared memory at once
  uint32_t x_bytes;     // activation slice in shared memory
  uint32_t* err_word;
  long long* trace;  // optional pipeline timestamps of CTA 0, see qmm_debug_set_trace
};

constexpr int kTraceStride = 1024;
__device__ __forceinline__ void stamp(const Params& p, int role, int& idx) {
  if (p.trace && blockIdx.x == 0 && idx < kTraceStride) p.trace[role * kTraceStride + idx++] = clock64();
}

template <typename XT>
__device__ __forceinline__ uint32_t sub_pair(uint32_t p, float bias) {
  if constexpr (std::is_same<XT, __half>::value) {
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&p), __float2half2_rn(bias));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&p), __float2bfloat162_rn(bias));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}

// 8 nibbles (nibble i = k offset i, two's complement) -> packed pairs (k0,k1)(k2,k3)(k4,k5)(k6,k7), exact:
// the offset-binary nibble is dropped under the exponent byte of 128.0 (bf16) or 1024.0 (f16) and the
// bias is taken out with one packed subtract.
// SUB = false leaves the bias in: the values read v + 136 (bf16) and the drain takes 136 * sum_k x back out.
template <typename XT, bool SUB>
__device__ __forceinline__ void cvt_s4x8(uint32_t w, uint32_t* p) {
  constexpr bool kBf16 = !std::is_same<XT, __half>::value;
  const uint32_t lo = (w & 0x0F0F0F0Fu) ^ 0x08080808u;
  const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
  const uint32_t q0 = __byte_perm(lo, hi, 0x5140);
  const uint32_t q1 = __byte_perm(lo, hi, 0x7362);
  const uint32_t expo = kBf16 ? 0x43434343u : 0x64646464u;
  constexpr float bias = kBf16 ? 136.f : 1032.f;
  p[0] = __byte_perm(q0, expo, 0x4140);
  p[1] = __byte_perm(q0, expo, 0x4342);
  p[2] = __byte_perm(q1, expo, 0x4140);
  p[3] = __byte_perm(q1, expo, 0x4342);
  if constexpr (SUB) {
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = sub_pair<XT>(p[i], bias);
  }
}

// 4 int8 -> packed pairs (k0,k1)(k2,k3), exact.
template <typename XT>
__device__ __forceinline__ void cvt_s8x4(uint32_t w, uint32_t* p) {
  const uint32_t u = w ^ 0x80808080u;
  if constexpr (std::is_same<XT, __half>::value) {
    p[0] = sub_pair<XT>(__byte_perm(u, 0x64646464u, 0x4140), 1152.f);
    p[1] = sub_pair<XT>(__byte_perm(u, 0x64646464u, 0x4342), 1152.f);
  } else {
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.f;
    __nv_bfloat162 a = __floats2bfloat162_rn(f0, f1), b = __floats2bfloat162_rn(f2, f3);
    p[0] = *reinterpret_cast<uint32_t*>(&a);
    p[1] = *reinterpret_cast<uint32_t*>(&b);
  }
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ uint32_t cluster_index() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

template <int WBITS, typename XT, int MP>
__global__ void __launch_bounds__(kThreads, 1)
    decode_tc_kernel(const __grid_constant__ CUtensorMap map_x, const Params p) {
  constexpr int WORDS = BK * WBITS / 32;      // 32-bit weight words per row per k tile: 8 (int4) or 16 (int8)
  constexpr int TILE_BYTES = BK * WBITS / 8;  // weight bytes per row per k tile: 32 or 64
  constexpr int DEPTH = (WBITS == 4) ? 2 : 1; // k tiles of weights in flight per converting warp beyond the current
  constexpr uint32_t kXTile = MP * 128;       // activation tile [MP x 64] in shared memory
  constexpr bool kIsBf16 = !std::is_same<XT, __half>::value;
  // int4 -> bf16 leaves the conversion bias (136) in the operand; 136 is small enough for the fp32
  // accumulation to absorb.  The f16 bias (1032) is not, so that path subtracts in the conversion.
  constexpr bool kBiasLeftIn = WBITS == 4 && kIsBf16;
  constexpr float kBias = 136.f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* x_base = smem;
  float* part = reinterpret_cast<float*>(smem + p.x_bytes);  // [rounds_per_pass][MP][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.x_bytes + (size_t)p.rounds_per_pass * MP * BMW * 4);
  uint64_t* x_full = bars;               // TMA bytes
  uint64_t* a_full = x_full + 1;         // [kSlots] 4 converting warps
  uint64_t* a_empty = a_full + kSlots;   // [kSlots] tcgen05.commit
  uint64_t* acc_full = a_empty + kSlots;   // [2 * kIssuers] tcgen05.commit
  uint64_t* acc_empty = acc_full + 2 * kIssuers;  // [2 * kIssuers] 4 drain warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2 * kIssuers);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* xsum = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 512);  // [blocks per slice][MP]: sum_k x per block and token

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int cluster = (int)cluster_index();
  const int k0_tile = (int)rank * p.kt_slice;   // first k tile of this CTA's slice
  // row blocks of this cluster: cluster, cluster + nclusters, ...
  int my_rounds = 0;
  if (cluster < p.row_blocks) my_rounds = (p.row_blocks - cluster + p.nclusters - 1) / p.nclusters;
  const int passes = (p.rounds + p.rounds_per_pass - 1) / p.rounds_per_pass;  // same for every cluster

  if (threadIdx.x == 0) {
    ptx::mbar_init(x_full, 1);
    for (int s = 0; s < kSlots; ++s) {
      ptx::mbar_init(&a_full[s], 4);
      ptx::mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < 2 * kIssuers; ++s) {
      ptx::mbar_init(&acc_full[s], 1);
      ptx::mbar_init(&acc_empty[s], 4);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_x);
  }
  if (warp == 0) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int bpr = p.kt_slice / p.tb;  // scale blocks per row block in this CTA's slice

  for (int pass = 0; pass < passes; ++pass) {
    const int r_begin = min(pass * p.rounds_per_pass, my_rounds);
    const int r_end = min(r_begin + p.rounds_per_pass, my_rounds);

    if (warp < kIssuers) {
      // ---------------- MMA issuers ----------------
      if (warp == 0 && pass == 0 && lane == 0) {
        // the activation slice is loaded once
        ptx::mbar_expect_tx(x_full, (uint32_t)p.kt_slice * kXTile);
        for (int j = 0; j < p.kt_slice; ++j)
          ptx::tma_load_2d(x_base + (size_t)j * kXTile, &map_x, x_full, (k0_tile + j) * BK, 0);
      }
      __syncwarp();
      const int iw = warp;
      constexpr uint32_t fmt = kIsBf16 ? 1u : 0u;
      constexpr uint32_t idesc = ptx::make_idesc(/*f32*/ 1, fmt, fmt, BMW, MP);
      const uint32_t desc_hi = (uint32_t)(ptx::make_sw128_kmajor_desc(0) >> 32);
      const uint32_t b_lo0 = (uint32_t)ptx::make_sw128_kmajor_desc(ptx::smem_u32(x_base));
      if (pass == 0) ptx::mbar_wait(x_full, 0, abort_flag, p.err_word, ptx::kErrWaitFull);
      const int blk_begin = r_begin * bpr, blk_end = r_end * bpr;
      // blocks of this issuer: iw, iw + 4, ...; nb = how many of them lie before this pass
      const int nb = (blk_begin + kIssuers - 1 - iw) / kIssuers;
      int blk = nb * kIssuers + iw;
      int i = nb << p.tb_shift;  // this issuer's running tile count
      int ti = 0;
      for (; blk < blk_end; blk += kIssuers) {
        // the issuer alternates between its two accumulators, so the drain of one block overlaps the next
        const int use = blk / kIssuers, buf = 2 * iw + (use & 1);
        const uint32_t d_tmem = tmem_base + buf * 32;
        ptx::mbar_wait(&acc_empty[buf], ((use >> 1) & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitTmemEmpty);
        int t_in_round = (blk << p.tb_shift) % p.kt_slice;  // tiles of one block are consecutive
        for (int ib = 0; ib < p.tb; ++ib, ++i, ++t_in_round) {
          const int slot = 2 * iw + (i & 1), suse = i >> 1;
          if (iw == 1 && lane == 0) stamp(p, 1, ti);
          ptx::mbar_wait(&a_full[slot], suse & 1, abort_flag, p.err_word, ptx::kErrWaitConv);
          ptx::tcgen05_fence_after();
          if (iw == 1 && lane == 0) stamp(p, 1, ti);
          if (lane == 0) {
            const uint32_t a_tmem = tmem_base + kAccCols + (uint32_t)slot * kSlotCols;
            const uint32_t b_lo = b_lo0 + (uint32_t)t_in_round * (kXTile >> 4);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t bd = ((uint64_t)desc_hi << 32) | (uint64_t)(b_lo + k * (UMMA_K * 2 >> 4));
              ptx::mma_f16_ts(d_tmem, a_tmem + k * (UMMA_K / 2), bd, idesc, (ib | k) != 0 ? 1u : 0u);
            }
            ptx::mma_commit(&a_empty[slot]);
            if (ib == p.tb - 1) ptx::mma_commit(&acc_full[buf]);
          }
          __syncwarp();
          if (iw == 1 && lane == 0) stamp(p, 1, ti);
        }
      }
    } else if (warp >= kFirstConvWarp && warp < kFirstDrainWarp) {
      // ---------------- converting groups ----------------
      // group g converts the tiles of issuer g, alternating between operand slots 2g and 2g+1
      const int g = (warp - kFirstConvWarp) >> 2, quad = warp & 3;
      const int row = quad * 32 + lane;
      const uint32_t st_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + kAccCols + (uint32_t)(2 * g) * kSlotCols;
      const int blk_begin = r_begin * bpr;
      // The group walks issuer g's tile sequence: scale blocks g, g+4, ... (global block index), tb tiles
      // each.  Two cursors over that sequence, one for the tile being converted and one DEPTH+1 tiles
      // ahead for the loads; a cursor is (tile in block, block in slice, row block round) and advances with
      // adds only.
      struct Cursor {
        int ib, kblk, round;
      };
      auto advance = [&](Cursor& c) {
        if (++c.ib == p.tb) {
          c.ib = 0;
          c.kblk += kIssuers;
          while (c.kblk >= bpr) {
            c.kblk -= bpr;
            ++c.round;
          }
        }
      };
      int i = ((blk_begin + kIssuers - 1 - g) / kIssuers) << p.tb_shift;  // issuer g's running tile count
      Cursor cc;
      {
        const int blk0 = (i >> p.tb_shift) * kIssuers + g;
        cc.ib = 0;
        cc.round = blk0 / bpr;
        cc.kblk = blk0 - cc.round * bpr;
      }
      Cursor fc = cc;
      const uint8_t* frow = nullptr;  // start of this lane's weight row (at the slice) for round fc.round
      int frow_round = -1;
      uint4 q[DEPTH + 1][WORDS / 4];
      auto fetch = [&](uint4 (&dst)[WORDS / 4]) {
        if (fc.round < my_rounds) {
          if (fc.round != frow_round) {
            int n = (cluster + fc.round * p.nclusters) * BMW + row;
            if (n >= p.N) n = p.N - 1;
            frow = p.w + (int64_t)n * p.pitch + (int64_t)k0_tile * TILE_BYTES;
            frow_round = fc.round;
          }
          const uint8_t* src = frow + ((fc.kblk << p.tb_shift) + fc.ib) * TILE_BYTES;
#pragma unroll
          for (int j = 0; j < WORDS / 4; ++j) dst[j] = ld_stream_u4(src + 16 * j);
        }
        advance(fc);
      };
#pragma unroll
      for (int d = 0; d <= DEPTH; ++d) {
#pragma unroll
        for (int j = 0; j < WORDS / 4; ++j) q[d][j] = make_uint4(0, 0, 0, 0);
        fetch(q[d]);
      }
      int ti = 0;
      const bool tracer = warp == kFirstConvWarp && lane == 0;
      bool more = true;
      while (more) {
#pragma unroll
        for (int d = 0; d <= DEPTH; ++d) {
          if (!more || cc.round >= r_end) {
            more = false;
            continue;
          }
          const int slot = 2 * g + (i & 1), use = i >> 1;
          if (tracer) stamp(p, 0, ti);
          ptx::mbar_wait_warp<32>(&a_empty[slot], (use & 1) ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
          ptx::tcgen05_fence_after();
          if (tracer) stamp(p, 0, ti);
          // two halves of 16 columns (32 k values) each
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t o[16];
            if constexpr (WBITS == 4) {
              const uint32_t words[4] = {q[d][h].x, q[d][h].y, q[d][h].z, q[d][h].w};
#pragma unroll
              for (int wi = 0; wi < 4; ++wi) cvt_s4x8<XT, !kBiasLeftIn>(words[wi], o + 4 * wi);
            } else {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const uint4 v = q[d][2 * h + j];
                cvt_s8x4<XT>(v.x, o + 8 * j);
                cvt_s8x4<XT>(v.y, o + 8 * j + 2);
                cvt_s8x4<XT>(v.z, o + 8 * j + 4);
                cvt_s8x4<XT>(v.w, o + 8 * j + 6);
              }
            }
            if (tracer) stamp(p, 0, ti);
            ptx::tmem_st_32x32b_x16(st_addr + (uint32_t)(i & 1) * kSlotCols + 16 * h, o);
            if (tracer) stamp(p, 0, ti);
          }
          fetch(q[d]);
          advance(cc);
          if (tracer) stamp(p, 0, ti);
          ptx::tmem_st_wait();
          ptx::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&a_full[slot]);
          if (tracer) stamp(p, 0, ti);
          ++i;
        }
      }
    } else if (warp >= kFirstDrainWarp) {
      // ---------------- drain: thread owns output row n = row block base + its TMEM lane ----------------
      const int quad = warp & 3;
      const int nl = quad * 32 + lane;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
      if (kBiasLeftIn && pass == 0) {
        // per scale block and token: sum_k x[token, k] over the block, from the resident (swizzled) tiles;
        // the swizzle only permutes 16-byte units inside a token's 128-byte row, so a row sum ignores it
        ptx::mbar_wait_warp<32>(x_full, 0, abort_flag, p.err_word, ptx::kErrWaitFull);
        for (int e = nl; e < bpr * MP; e += 128) {
          const int b = e / MP, j = e - b * MP;
          float sx = 0.f;
          for (int t = 0; t < p.tb; ++t) {
            const uint4* rowp = reinterpret_cast<const uint4*>(x_base + (size_t)(b * p.tb + t) * kXTile + j * 128);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const uint4 v = rowp[u];
              const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int c = 0; c < 4; ++c) sx += __uint_as_float(wv[c] << 16) + __uint_as_float(wv[c] & 0xffff0000u);
            }
          }
          xsum[e] = sx;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four drain warps
      }
      float acc[MP];
#pragma unroll
      for (int j = 0; j < MP; ++j) acc[j] = 0.f;
      const int block0 = k0_tile / p.tb;  // first scale block of this CTA's slice
      int ti = 0;
      const bool tracer = warp == kFirstDrainWarp && lane == 0;
      // the owner of this thread's row in the cluster reduction, and where the row sits in the owner's buffer
      const int rpc = BMW / p.S;
      const uint32_t owner = (uint32_t)(nl / rpc);
      const uint32_t recv0 = map_to_cta(ptx::smem_u32(part), owner) + (uint32_t)(nl % rpc) * 4;
      for (int r = r_begin; r < r_end; ++r) {
        const int n = (cluster + r * p.nclusters) * BMW + nl;
        const bool n_ok = n < p.N;
        for (int b = 0; b < bpr; ++b) {
          const int blk = r * bpr + b;
          const int use = blk / kIssuers, buf = 2 * (blk % kIssuers) + (use & 1);
          const float s = p.blockwise ? (n_ok ? __ldg(p.scale + (int64_t)(block0 + b) * p.N + n) : 0.f) : 1.f;
          if (tracer) stamp(p, 2, ti);
          ptx::mbar_wait_warp<32>(&acc_full[buf], (use >> 1) & 1, abort_flag, p.err_word, ptx::kErrWaitTmemFull);
          ptx::tcgen05_fence_after();
          if (tracer) stamp(p, 2, ti);
#pragma unroll
          for (int c = 0; c < MP / 16; ++c) {
            uint32_t rr[16];
            ptx::tmem_ld_32x32b_x16(lane_addr + buf * 32 + c * 16, rr);
            ptx::tmem_ld_wait();
            if constexpr (kBiasLeftIn) {
              const float4* xs = reinterpret_cast<const float4*>(xsum + b * MP + c * 16);
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                const float4 xv = xs[j4];
                const float xe[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int j = 4 * j4 + e;
                  acc[c * 16 + j] = fmaf(s, fmaf(-kBias, xe[e], __uint_as_float(rr[j])), acc[c * 16 + j]);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(s, __uint_as_float(rr[j]), acc[c * 16 + j]);
            }
          }
          ptx::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
          if (tracer) stamp(p, 2, ti);
        }
        // push this row block's totals into the owner's buffer: [round in pass][source rank][token][row]
        const uint32_t dst = recv0 + (uint32_t)((((r - r_begin) * p.S + (int)rank) * MP) * rpc) * 4;
#pragma unroll
        for (int j = 0; j < MP; ++j) {
          st_cluster_f32(dst + (uint32_t)(j * rpc) * 4, acc[j]);
          acc[j] = 0.f;
        }
      }
    }

    // ---------------- pass end: the S partial results of every row block meet here ----------------
    int te = 0;
    if (threadIdx.x == 0) stamp(p, 3, te);
    __syncwarp();
    cluster_sync_all();  // every peer's pushes of this pass have landed in this CTA's buffer
    if (threadIdx.x == 0) stamp(p, 3, te);
    {
      // CTA `rank` finishes rows [rank*128/S, (rank+1)*128/S) of every row block from the S partial sums
      // its peers pushed into its buffer, four rows per thread step (all sizes are powers of two)
      constexpr int kMpShift = MP == 32 ? 5 : 4;
      const int q_shift = 5 - p.s_shift;  // log2(quads of rows per CTA): 128 / S / 4
      const int rpc = BMW >> p.s_shift;
      const int total = (r_end - r_begin) << (kMpShift + q_shift);
      for (int idx = threadIdx.x; idx < total; idx += kThreads) {
        const int ql = idx & ((1 << q_shift) - 1);
        const int j = (idx >> q_shift) & (MP - 1);
        const int rr = idx >> (kMpShift + q_shift);
        const float* src = part + ((size_t)((rr << p.s_shift) * MP + j) << (7 - p.s_shift)) + 4 * ql;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        for (int z = 0; z < p.S; ++z) {
          const float4 pv = *reinterpret_cast<const float4*>(src + (size_t)z * MP * rpc);
          v[0] += pv.x;
          v[1] += pv.y;
          v[2] += pv.z;
          v[3] += pv.w;
        }
        const int n0 = (cluster + (r_begin + rr) * p.nclusters) * BMW + (int)rank * rpc + 4 * ql;
        if (j < p.M) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = n0 + e;
            if (n < p.N) store_from_f32(p.out, (int64_t)j * p.N + n, p.out_dt, p.blockwise ? v[e] : v[e] * __ldg(p.scale + n));
          }
        }
      }
    }
    if (threadIdx.x == 0) stamp(p, 3, te);
    if (pass + 1 < passes) {
      __syncwarp();
      cluster_sync_all();  // the next pass pushes into the same buffers
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 0) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

struct Plan {
  int S, nclusters, rounds, rounds_per_pass, kt_slice, tb;
  uint32_t x_bytes;
  size_t smem;
};

template <int WBITS, typename XT, int MP>
int launch_cfg(const void* x, const void* w, const float* scale, void* out, int out_dt, int64_t M, int64_t N, int64_t K,
               int64_t block_size, cudaStream_t st) {
  auto kern = decode_tc_kernel<WBITS, XT, MP>;
  static bool attr_set[64] = {};
  static int max_clusters[64][4] = {};  // per device, per log2(S): co-resident clusters at the largest footprint
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return fail(QMM_ERR_DEVICE, "decode_tc: device index %d", dev);
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemCap + 2048);
    if (e != cudaSuccess) return fail(QMM_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    for (int ls = 0; ls < 4; ++ls) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(sm_count() / (1 << ls)) * (1 << ls));
      cfg.blockDim = dim3(kThreads);
      cfg.dynamicSmemBytes = kSmemCap + 2048;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1u << ls;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      max_clusters[dev][ls] = n;
    }
    attr_set[dev] = true;
  }
  const bool blockwise = block_size > 0;
  const int kt = (int)(K / BK);
  const int row_blocks = (int)ceil_div(N, BMW);
  Plan best = {};
  int64_t best_cost = -1;
  for (int ls = 3; ls >= 0; --ls) {
    const int S = 1 << ls;
    if (max_clusters[dev][ls] < 1) continue;
    if (kt % S != 0) continue;
    const int kts = kt / S;
    int tb;
    if (blockwise) {
      tb = (int)(block_size / BK);
      if (kts % tb != 0) continue;  // a slice holds whole scale blocks
    } else {
      tb = (kts % 2 == 0) ? 2 : 1;
    }
    const uint32_t x_bytes = (uint32_t)kts * MP * 128;
    const int part_bytes = MP * BMW * 4;
    if ((int64_t)x_bytes + part_bytes + 5120 > kSmemCap) continue;
    if (WBITS == 4 && !std::is_same<XT, __half>::value && kts / tb * MP * 4 > 4096) continue;  // per-block activation sums
    const int nclusters = std::min(max_clusters[dev][ls], row_blocks);
    const int rounds = (int)ceil_div(row_blocks, nclusters);
    const int rpp = std::min(rounds, (int)((kSmemCap - 5120 - (int64_t)x_bytes) / part_bytes));
    const int passes = (int)ceil_div(rounds, rpp);
    const int64_t cost = (int64_t)rounds * kts + 8 * passes;  // tile times on the busiest CTA (+ reduction)
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = Plan{S, nclusters, rounds, rpp, kts, tb, x_bytes, (size_t)x_bytes + (size_t)rpp * part_bytes + 1024 + 5120};
    }
  }
  if (best_cost < 0) return fail(QMM_ERR_UNSUPPORTED, "decode_tc: no K split fits (K=%lld bs=%lld)", (long long)K, (long long)block_size);

  CUtensorMap map_x;
  int rc = encode_tmap_2d(&map_x, x, 2, true, (uint64_t)M, (uint64_t)K, (uint32_t)MP, BK);
  if (rc != QMM_OK) return rc;
  Params p;
  p.w = reinterpret_cast<const uint8_t*>(w);
  p.scale = scale;
  p.out = out;
  p.out_dt = out_dt;
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.pitch = K * WBITS / 8;
  p.S = best.S;
  p.s_shift = best.S == 8 ? 3 : (best.S == 4 ? 2 : (best.S == 2 ? 1 : 0));
  p.kt_slice = best.kt_slice;
  p.tb = best.tb;
  p.tb_shift = 0;
  while ((1 << p.tb_shift) < best.tb) ++p.tb_shift;
  p.blockwise = blockwise ? 1 : 0;
  p.row_blocks = row_blocks;
  p.nclusters = best.nclusters;
  p.rounds = best.rounds;
  p.rounds_per_pass = best.rounds_per_pass;
  p.x_bytes = best.x_bytes;
  p.err_word = device_error_word();
  p.trace = debug_trace_buffer();
  if (getenv("QMM_B200_LOG"))
    fprintf(stderr, "[qmm] decode_tc max clusters by S=1,2,4,8: %d %d %d %d; plan: S=%d clusters=%d rounds=%d rounds/pass=%d k tiles/slice=%d tiles/block=%d smem=%zu\n",
            max_clusters[dev][0], max_clusters[dev][1], max_clusters[dev][2], max_clusters[dev][3], best.S, best.nclusters, best.rounds, best.rounds_per_pass, best.kt_slice, best.tb, best.smem);

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(best.nclusters * best.S));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = best.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)best.S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_x, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_LAUNCH, "decode_tc_kernel launch: %s", cudaGetErrorString(e));
  }
  return check_launch("decode_tc_kernel");
}

template <int WBITS, typename XT>
int launch_mp(const void* x, const void* w, const float* scale, void* out, int out_dt, int64_t M, int64_t N, int64_t K,
              int64_t block_size, cudaStream_t st) {
  if (M <= 16) return launch_cfg<WBITS, XT, 16>(x, w, scale, out, out_dt, M, N, K, block_size, st);
  return launch_cfg<WBITS, XT, 32>(x, w, scale, out, out_dt, M, N, K, block_size, st);
}

}  // namespace

bool decode_tc_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x, int x_dt,
                         const void* w, bool has_zp) {
  if (has_zp) return false;
  if (x_dt != QMM_BF16 && x_dt != QMM_F16) return false;
  if (M < 1 || M > 32 || N < 1 || K < BK || K % BK != 0) return false;
  if (block_size > 0) {
    const int64_t tb = block_size / BK;
    if (block_size % BK != 0 || K % block_size != 0 || (tb & (tb - 1)) != 0) return false;  // blocks of 2^i k tiles
  }
  if (N > (1 << 28) || K > (1 << 24)) return false;
  {
    // some split of K over 1..8 CTAs must leave a slice of whole blocks whose activations fit in shared memory
    const int mp = M <= 16 ? 16 : 32;
    const int64_t kt = K / BK, tb = block_size > 0 ? block_size / BK : 1;
    bool any = false;
    for (int S = 8; S >= 1; S >>= 1)
      any |= kt % S == 0 && (kt / S) % tb == 0 && (kt / S) * mp * 128 + (int64_t)mp * BMW * 4 + 5120 <= kSmemCap &&
             (wbits != 4 || x_dt != QMM_BF16 || (kt / S) / tb * mp * 4 <= 4096);
    if (!any) return false;
  }
  if (!aligned(x, 16) || !aligned(w, 16)) return false;
  return device_is_sm100();
}

int launch_decode_tc(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt,
                     int64_t M, int64_t N, int64_t K, int64_t block_size, cudaStream_t st) {
  if (!decode_tc_supported(wbits, M, N, K, block_size, x, x_dt, w, false))
    return fail(QMM_ERR_UNSUPPORTED,
                "tensor-memory decode kernel: needs an sm_100 device, bf16/f16 activations, 1<=M<=32, K a multiple of 64, "
                "block_size a multiple of 64, 16-byte aligned x/w, no zero point (M=%lld N=%lld K=%lld bs=%lld)",
                (long long)M, (long long)N, (long long)K, (long long)block_size);
  if (wbits == 4) {
    if (x_dt == QMM_BF16) return launch_mp<4, __nv_bfloat16>(x, w, scale, out, out_dt, M, N, K, block_size, st);
    return launch_mp<4, __half>(x, w, scale, out, out_dt, M, N, K, block_size, st);
  }
  if (x_dt == QMM_BF16) return launch_mp<8, __nv_bfloat16>(x, w, scale, out, out_dt, M, N, K, block_size, st);
  return launch_mp<8, __half>(x, w, scale, out, out_dt, M, N, K, block_size, st);
}

}  // namespace qmm
