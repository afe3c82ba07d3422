// Decode kernel for K-minor weights (int8 [N,K] or packed int4 [N,K/2]) and small token batches
// (M <= 32): weights go from HBM straight into registers, are dequantised there (exactly) and fed
// to warp-level tensor-core MMAs as the A operand; the activations are the B operand.  There is no
// shared-memory round trip for the weights and no single issuing thread, so the kernel is a pure
// weight stream whose only per-value cost is the integer -> bf16/f16 conversion.
//
//   out[m,n] = sum_b scale[b,n] * (sum_{k in block b} x[m,k] * w[n,k])       (per-channel: one block)
//
// Mapping.  A CTA of W warps (4, 8 or 16: see launch_nt) owns 16 consecutive output rows n; warp w takes the K steps s = w, w+W, ...
// One step covers 64 bytes of each weight row (128 int4 or 64 int8 values): lane (g = lane/4,
// t = lane%4) loads 16 bytes of row g and of row g+8 at byte offset 16*t of the step, i.e. each lane
// owns a contiguous k span and the four lanes of a quad own the whole step.  Because the contraction
// index may be permuted freely as long as both operands agree, the lane's k span maps onto the MMA's
// k slots in whatever order the conversion produces; the lane loads the matching activations of
// token g (B operand, column g) from global memory through L1 (x is a few KB and shared by all CTAs).
// After each scale block the 16x8 partial tile is folded into fp32 accumulators with scale[b,n].
// The int4 conversion leaves a constant bias in the weights (see Bias below); it is taken out again at
// every fold with bias * sum_k x, which an extra MMA against an all-ones operand supplies.
//
// Semantics: torch_xla/experimental/xla_quantized_matmul.py:152-159 (per channel), :165-170 (blockwise).
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace qmm {

namespace {


template <typename XT>
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<XT, __half>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// same MMA as mma_16816 but not volatile: the compiler may interleave independent accumulator chains
template <typename XT>
__device__ __forceinline__ void mma_16816_nv(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<XT, __half>::value) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Bias carried by the converted weights.  The conversion drops an offset-binary nibble (v + 8) or byte
// (v + 128) under the exponent of a power of two and does NOT subtract it again; the kernel removes
// bias * sum_k x[m,k] instead, which the tensor core computes for free from the same activation
// registers (an MMA against an all-ones A operand).  Saves one packed subtract per two weights.
template <typename XT, int WBITS>
struct Bias;
template <>
struct Bias<__nv_bfloat16, 4> { static constexpr float value = 136.f; static constexpr uint32_t ones = 0x3F803F80u; };
template <>
struct Bias<__half, 4> { static constexpr float value = 1032.f; static constexpr uint32_t ones = 0x3C003C00u; };
template <>
struct Bias<__nv_bfloat16, 8> { static constexpr float value = 0.f; static constexpr uint32_t ones = 0x3F803F80u; };
template <>
struct Bias<__half, 8> { static constexpr float value = 1152.f; static constexpr uint32_t ones = 0x3C003C00u; };

// 8 nibbles (nibble i = k offset i, two's complement) -> packed pairs (k0,k1)(k2,k3)(k4,k5)(k6,k7) of
// (v + 8) + 128 in bf16 or (v + 8) + 1024 in fp16: 9 integer instructions per 8 weights.
template <typename XT>
__device__ __forceinline__ void cvt_s4x8_biased(uint32_t w, uint32_t* p) {
  constexpr bool kBf16 = !std::is_same<XT, __half>::value;
  const uint32_t lo = (w & 0x0F0F0F0Fu) ^ 0x08080808u;         // k0 k2 k4 k6, offset binary
  const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;  // k1 k3 k5 k7
  const uint32_t q0 = __byte_perm(lo, hi, 0x5140);             // k0 k1 k2 k3
  const uint32_t q1 = __byte_perm(lo, hi, 0x7362);             // k4 k5 k6 k7
  const uint32_t expo = kBf16 ? 0x43434343u : 0x64646464u;     // exponent byte of 128.0 (bf16) / 1024.0 (f16)
  p[0] = __byte_perm(q0, expo, 0x4140);
  p[1] = __byte_perm(q0, expo, 0x4342);
  p[2] = __byte_perm(q1, expo, 0x4140);
  p[3] = __byte_perm(q1, expo, 0x4342);
}

// 4 int8 -> packed pairs (k0,k1)(k2,k3).  fp16: (v + 128) + 1024, bias left in (3 instructions);
// bf16 cannot hold a byte under an exponent, so it goes through fp32 and is exact (bias 0).
template <typename XT>
__device__ __forceinline__ void cvt_s8x4_biased(uint32_t w, uint32_t* p) {
  const uint32_t u = w ^ 0x80808080u;
  if constexpr (std::is_same<XT, __half>::value) {
    p[0] = __byte_perm(u, 0x64646464u, 0x4140);
    p[1] = __byte_perm(u, 0x64646464u, 0x4342);
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

// packed pair minus (bias, bias): exact, the operands are small integers
template <typename XT>
__device__ __forceinline__ uint32_t sub_bias(uint32_t p, float bias) {
  if constexpr (std::is_same<XT, __half>::value) {
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&p), __float2half2_rn(bias));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&p), __float2bfloat162_rn(bias));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}

// Fused MLP epilogue: the weight rows are stored in groups of 16, eight rows of the gate projection followed
// by the eight rows of the up projection for the same outputs; the kernel then writes silu(gate) * up, one
// column per pair, computed in fp32 from the fp32 accumulators.
__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.f + expf(-gate)) * up; }
__device__ __forceinline__ int64_t gate_up_column(int64_t n) { return ((n >> 4) << 3) + (n & 7); }

// Row-parallel exchange fused into the decode kernel (AR = true): the CTA's 16 x M partial sums go to the
// peer-visible buffers, the CTA tells every peer that ITS tile is there (one flag word per rank and tile, holding
// the call number), waits - bounded - for the same tile from every peer and writes the sum of the G partials, added
// in rank order.  Tiles are exchanged as they finish, so the waiting of one CTA overlaps the weight stream of the
// others.  The partial sums are PUSHED: a CTA stores its tile into every rank's buffer, so the final sum reads local
// memory only and the exchange costs one NVLink crossing, not a round trip.  Buffer layout (per rank): two slots
// (call e uses slot e & 1) of `world` regions of slot_floats fp32, region r written by rank r; then world x tiles
// flag words, then the call counter and a ticket.  The call number is kept in device memory, so a
// launch captured in a CUDA graph stays valid on replay; the previous call of the stream has completed before
// this one signals (it waits on griddepcontrol.wait first), which is what makes two slots enough.
constexpr int kArMaxRanks = 8;
struct ArParams {
  float* data[kArMaxRanks];      // base of every rank's buffer (index = rank); entry `rank` is this GPU's own
  int rank, world;
  uint32_t slot_floats;          // fp32 elements per data slot (>= M * N)
  uint32_t tiles;                // CTAs of the launch = flag words per rank
  long long wait_cycles;         // how long a CTA waits for its peers' tiles before it gives up
};
__device__ __forceinline__ uint32_t* ar_flags(const ArParams& a, int owner) {
  return reinterpret_cast<uint32_t*>(a.data[owner] + 2 * (size_t)a.world * a.slot_floats);
}
__device__ __forceinline__ void ar_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ar_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ar_ld_peer(const float* p) {
  float v;
  asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// NT = number of 8-token tiles (M <= 8*NT); RG = 16-row groups per CTA (each warp converts RG groups per
// step and reuses its activation registers for all of them); WARPS = warps splitting K.
// One "fold" = the end of a scale block (blockwise) or of a single step (per-channel): the partial tile,
// minus bias * sum(x), is added into the totals.
template <int WBITS, typename XT, int NT, int RG, int WARPS, bool AR = false>
__global__ void __launch_bounds__(WARPS * 32)
    decode_mma_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ w, const float* __restrict__ scale,
                      void* __restrict__ out, int out_dt, int M, int64_t N, int64_t K, int steps_per_block,
                      int spb_shift, int blockwise, int gate_up, const ArParams ar, uint32_t* err_word) {
  // ar.wait_cycles bounds the wait for the peers' tiles (AR only)
  constexpr int VPS = 512 / WBITS;      // values of one weight row per step: 128 (int4) or 64 (int8)
  constexpr int VPL = VPS / 4;          // values per lane per row per step: 32 or 16
  constexpr int XREGS = VPL / 2;        // packed activation pairs per lane per token tile: 16 or 8
  constexpr int ROWS = 16 * RG;         // output rows per CTA
  // With one token tile the bias stays in and a ones-MMA removes it (the integer pipe is the limiter
  // there); with more tiles the tensor pipe matters more, so the bias is subtracted in the conversion
  // (a packed subtract on the otherwise idle FMA pipe) and the extra MMAs disappear.
  constexpr float kBias = Bias<XT, WBITS>::value;
  constexpr bool kHasBias = kBias != 0.f && NT == 1;
  constexpr bool kSubBias = kBias != 0.f && NT != 1;
  constexpr uint32_t kOnes = Bias<XT, WBITS>::ones;
  __shared__ float s_part[WARPS][ROWS][NT * 8];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int64_t n0 = (int64_t)blockIdx.x * ROWS;
  const int64_t pitch = K * WBITS / 8;
  const int steps = (int)(K / VPS);
  // lane rows: group r -> rows n0 + 16r + g and n0 + 16r + g + 8 (clamped: tail rows are computed, not stored)
  const uint8_t* wrow[2 * RG];
  const float* srow[2 * RG];
#pragma unroll
  for (int r = 0; r < 2 * RG; ++r) {
    int64_t n = n0 + 16 * (r >> 1) + g + 8 * (r & 1);
    if (n >= N) n = N - 1;
    wrow[r] = w + n * pitch + 16 * t;
    srow[r] = scale + n;
  }

  // activation row of token (8*i + g) at this lane's offset inside a step; the columns of tokens beyond M
  // are computed from token 0 and never stored (an MMA column depends on its own B column only)
  const XT* xrow[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const int tok = 8 * i + g;
    xrow[i] = x + (int64_t)(tok < M ? tok : 0) * K + t * VPL;
  }

  float total[RG][NT][4], part[RG][NT][4], xsum[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      xsum[i][j] = 0.f;
#pragma unroll
      for (int r = 0; r < RG; ++r) total[r][i][j] = part[r][i][j] = 0.f;
    }
  const uint32_t ones[4] = {kOnes, kOnes, kOnes, kOnes};

  // Software pipeline, one step deep: the weights of this warp's next step are in flight while the
  // current step is converted and multiplied.  (Prefetching the activations as well costs 24 registers
  // and measured slower: they come from L1.)
  constexpr bool kPrefetchX = false;
  auto load_x = [&](int step, uint32_t (&dst)[NT][XREGS]) {
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const uint4* xp = reinterpret_cast<const uint4*>(xrow[i] + (int64_t)step * VPS);
#pragma unroll
      for (int q = 0; q < XREGS / 4; ++q) {
        const uint4 v = __ldg(xp + q);  // an absent token reads token 0: its column is computed, never stored
        dst[i][4 * q] = v.x;
        dst[i][4 * q + 1] = v.y;
        dst[i][4 * q + 2] = v.z;
        dst[i][4 * q + 3] = v.w;
      }
    }
  };
  int s = warp;
  uint4 wn[2 * RG];
#pragma unroll
  for (int r = 0; r < 2 * RG; ++r) {
    wn[r] = make_uint4(0, 0, 0, 0);
    if (s < steps) wn[r] = ld_stream_u4(wrow[r] + (int64_t)s * 64);
  }
  // Programmatic dependent launch: the weights are static, so their first loads may overlap the tail
  // of the previous kernel in the stream; everything that depends on that kernel (the activations)
  // and every store of this kernel come after the wait.  Both are no-ops in an ordinary launch.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  uint32_t xn[NT][XREGS];
  if (kPrefetchX && s < steps) load_x(s, xn);
  for (; s < steps; s += WARPS) {
    uint4 wc[2 * RG];
#pragma unroll
    for (int r = 0; r < 2 * RG; ++r) wc[r] = wn[r];
    uint32_t xr[NT][XREGS];
    if (kPrefetchX) {
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int q = 0; q < XREGS; ++q) xr[i][q] = xn[i][q];
    }
    const int sn = s + WARPS;
    if (sn < steps) {
#pragma unroll
      for (int r = 0; r < 2 * RG; ++r) wn[r] = ld_stream_u4(wrow[r] + (int64_t)sn * 64);
      if (kPrefetchX) load_x(sn, xn);
    }
    // fold after this step?  (blockwise: this warp's next step belongs to another block)
    bool fold = true;
    float sc[2 * RG];
#pragma unroll
    for (int r = 0; r < 2 * RG; ++r) sc[r] = 1.f;
    if (blockwise) {
      const int b = spb_shift >= 0 ? (s >> spb_shift) : (s / steps_per_block);
      const int bn = spb_shift >= 0 ? (sn >> spb_shift) : (sn / steps_per_block);
      fold = sn >= steps || bn != b;
      if (fold) {
#pragma unroll
        for (int r = 0; r < 2 * RG; ++r) sc[r] = __ldg(srow[r] + (int64_t)b * N);
      }
    }
    if (!kPrefetchX) load_x(s, xr);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      if constexpr (WBITS == 4) {
        // word wi holds k = 8*wi .. 8*wi+7 of the lane's span: two MMAs of 4 values per row
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          uint32_t pa[4], pb[4];
          cvt_s4x8_biased<XT>(reinterpret_cast<const uint32_t*>(&wc[2 * r])[wi], pa);
          cvt_s4x8_biased<XT>(reinterpret_cast<const uint32_t*>(&wc[2 * r + 1])[wi], pb);
          if constexpr (kSubBias) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              pa[q] = sub_bias<XT>(pa[q], kBias);
              pb[q] = sub_bias<XT>(pb[q], kBias);
            }
          }
          const uint32_t a_lo[4] = {pa[0], pb[0], pa[1], pb[1]};
          const uint32_t a_hi[4] = {pa[2], pb[2], pa[3], pb[3]};
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            mma_16816_nv<XT>(part[r][i], a_lo, xr[i][4 * wi], xr[i][4 * wi + 1]);
            mma_16816_nv<XT>(part[r][i], a_hi, xr[i][4 * wi + 2], xr[i][4 * wi + 3]);
          }
        }
        if constexpr (kHasBias) {
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            mma_16816_nv<XT>(xsum[i], ones, xr[i][4 * wi], xr[i][4 * wi + 1]);
            mma_16816_nv<XT>(xsum[i], ones, xr[i][4 * wi + 2], xr[i][4 * wi + 3]);
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          uint32_t pa[2], pb[2];
          cvt_s8x4_biased<XT>(reinterpret_cast<const uint32_t*>(&wc[2 * r])[wi], pa);
          cvt_s8x4_biased<XT>(reinterpret_cast<const uint32_t*>(&wc[2 * r + 1])[wi], pb);
          if constexpr (kSubBias) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              pa[q] = sub_bias<XT>(pa[q], kBias);
              pb[q] = sub_bias<XT>(pb[q], kBias);
            }
          }
          const uint32_t a[4] = {pa[0], pb[0], pa[1], pb[1]};
#pragma unroll
          for (int i = 0; i < NT; ++i) mma_16816_nv<XT>(part[r][i], a, xr[i][2 * wi], xr[i][2 * wi + 1]);
        }
        if constexpr (kHasBias) {
#pragma unroll
          for (int i = 0; i < NT; ++i) mma_16816_nv<XT>(xsum[i], ones, xr[i][2 * wi], xr[i][2 * wi + 1]);
        }
      }
    }
    if (fold) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          // xsum rows are all equal: c0,c1 (tokens 2t, 2t+1) serve both row g and row g+8
          const float p0 = kHasBias ? fmaf(-kBias, xsum[i][0], part[r][i][0]) : part[r][i][0];
          const float p1 = kHasBias ? fmaf(-kBias, xsum[i][1], part[r][i][1]) : part[r][i][1];
          const float p2 = kHasBias ? fmaf(-kBias, xsum[i][0], part[r][i][2]) : part[r][i][2];
          const float p3 = kHasBias ? fmaf(-kBias, xsum[i][1], part[r][i][3]) : part[r][i][3];
          total[r][i][0] = fmaf(sc[2 * r], p0, total[r][i][0]);
          total[r][i][1] = fmaf(sc[2 * r], p1, total[r][i][1]);
          total[r][i][2] = fmaf(sc[2 * r + 1], p2, total[r][i][2]);
          total[r][i][3] = fmaf(sc[2 * r + 1], p3, total[r][i][3]);
#pragma unroll
          for (int j = 0; j < 4; ++j) part[r][i][j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) xsum[i][j] = 0.f;
      }
    }
  }

  // accumulator layout of m16n8: c0,c1 -> row g, tokens 2t,2t+1; c2,c3 -> row g+8
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      s_part[warp][16 * r + g][8 * i + 2 * t] = total[r][i][0];
      s_part[warp][16 * r + g][8 * i + 2 * t + 1] = total[r][i][1];
      s_part[warp][16 * r + g + 8][8 * i + 2 * t] = total[r][i][2];
      s_part[warp][16 * r + g + 8][8 * i + 2 * t + 1] = total[r][i][3];
    }
  __syncthreads();
  if constexpr (AR) {
    // ---- fused row-parallel exchange ----
    __shared__ uint32_t s_epoch;
    __shared__ int s_ok;
    uint32_t* my_flags = ar_flags(ar, ar.rank);
    uint32_t* ctr = my_flags + (size_t)ar.world * ar.tiles;  // [0] call counter, [1] ticket
    if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(ctr) + 1u;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    // push: my partial goes into region [slot][my rank] of EVERY rank's buffer (plain stores, local or over
    // NVLink); the sum later reads local memory only
    const size_t region = ((size_t)(epoch & 1u) * ar.world + ar.rank) * ar.slot_floats;
    for (int idx = threadIdx.x; idx < ROWS * NT * 8; idx += WARPS * 32) {
      const int row = idx % ROWS, tok = idx / ROWS;
      const int64_t n = n0 + row;
      if (n < N && tok < M) {
        float v = 0.f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) v += s_part[wi][row][tok];
        if (!blockwise) v *= __ldg(scale + n);
        const size_t o = region + (size_t)tok * N + n;
#pragma unroll
        for (int r = 0; r < kArMaxRanks; ++r)
          if (r < ar.world) ar.data[r][o] = v;
      }
    }
    // the barrier orders the CTA's stores before the signalling threads; their release stores (system scope,
    // cumulative) then publish them - one fence per signal instead of one per thread
    __syncthreads();
    if (threadIdx.x < ar.world)
      ar_st_release(ar_flags(ar, threadIdx.x) + (size_t)ar.rank * ar.tiles + blockIdx.x, epoch);
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < ar.world) {
      const uint32_t* f = my_flags + (size_t)threadIdx.x * ar.tiles + blockIdx.x;
      const long long t0 = clock64();
      uint32_t spins = 0;
      while ((int32_t)(ar_ld_acquire(f) - epoch) < 0) {
        if ((++spins & 0x3ff) == 0 && clock64() - t0 > ar.wait_cycles) {  // give up, report
          s_ok = 0;
          if (err_word) atomicCAS(err_word, 0u, 8u | ((uint32_t)threadIdx.x << 8));
          break;
        }
      }
    }
    __syncthreads();
    if (s_ok) {
      const float* mine = ar.data[ar.rank] + (size_t)(epoch & 1u) * ar.world * ar.slot_floats;
      for (int idx = threadIdx.x; idx < ROWS * NT * 8; idx += WARPS * 32) {
        const int row = idx % ROWS, tok = idx / ROWS;
        const int64_t n = n0 + row;
        if (n < N && tok < M) {
          const int64_t o = (int64_t)tok * N + n;
          float v = 0.f;
          for (int r = 0; r < ar.world; ++r) v += ar_ld_peer(mine + (size_t)r * ar.slot_floats + o);
          store_from_f32(out, o, out_dt, v);
        }
      }
    } else {
      // a peer's tile never arrived (the device error word says which rank): NaN instead of stale memory
      for (int idx = threadIdx.x; idx < ROWS * NT * 8; idx += WARPS * 32) {
        const int row = idx % ROWS, tok = idx / ROWS;
        const int64_t n = n0 + row;
        if (n < N && tok < M) store_from_f32(out, (int64_t)tok * N + n, out_dt, __uint_as_float(0x7fc00000u));
      }
    }
    // the CTA that finishes last advances the call counter (every CTA has read it by then)
    if (threadIdx.x == 0 && atomicAdd(ctr + 1, 1u) == gridDim.x - 1) {
      ctr[1] = 0;
      *reinterpret_cast<volatile uint32_t*>(ctr) = epoch;
    }
    return;
  }
  for (int idx = threadIdx.x; idx < ROWS * NT * 8; idx += WARPS * 32) {
    const int row = idx % ROWS, tok = idx / ROWS;  // consecutive threads -> consecutive n
    const int64_t n = n0 + row;
    if (n < N && tok < M) {
      float v = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) v += s_part[wi][row][tok];
      if (!blockwise) v *= __ldg(scale + n);
      if (!gate_up) {
        store_from_f32(out, (int64_t)tok * N + n, out_dt, v);
      } else if ((row & 8) == 0) {
        // rows come in groups of 16: eight gate rows, then the eight up rows of the same outputs
        float u = 0.f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) u += s_part[wi][row + 8][tok];
        if (!blockwise) u *= __ldg(scale + n + 8);
        store_from_f32(out, (int64_t)tok * (N >> 1) + gate_up_column(n), out_dt, silu_mul(v, u));
      }
    }
  }
}

// ---- token batches of 9..32 ----------------------------------------------------------------------------
//
// With more than one token tile the activations (M*K*2 bytes: 256 KB for 32 tokens of 4096) no longer
// stay in L1, and the kernel above re-reads them from L2 once per CTA: 448 CTAs x 256 KB is four times
// the weight stream.  This kernel runs one 16-warp CTA per SM instead.  The CTA owns up to TR row tiles
// (16 output rows each) at a time, WK = 16/TR warps share the K steps of one tile, and all of them read
// the activations from a shared-memory ring that the whole CTA fills with cp.async, one chunk of 8 steps
// at a time: the activations cross L2 -> SM once per CTA and round.  Weights still go HBM -> registers,
// two steps ahead of their use.
//
// Shared-memory layout of a chunk: one row per token, 16-byte units of the row permuted by
// u ^ (((u >> 3) & 1) << 1) and rows pitched by one extra unit; with that the 16-byte fragment reads of
// a quarter warp (two tokens x four k spans) spread over all 32 banks.
constexpr int kStagedWarps = 16;
constexpr int kChunkSteps = 8;

__device__ __forceinline__ int swz_unit(int u) { return u ^ (((u >> 3) & 1) << 1); }

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// first MMA of an accumulator chain: C = 0 comes from the zero register, no accumulator set-up
template <typename XT>
__device__ __forceinline__ void mma_16816_nv_first(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<XT, __half>::value) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  }
}

struct StagedStep {  // one K step of a warp in flight: 16 bytes of two weight rows and their block scales
  uint4 w[2];
  float sc[2];
};

template <int WBITS, typename XT, int NT, bool FOLD_EVERY>
__global__ void __launch_bounds__(kStagedWarps * 32, 1)
    decode_mma_staged_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ w, const float* __restrict__ scale,
                             void* __restrict__ out, int out_dt, int M, int N, int K, int steps_per_block,
                             int spb_shift, int blockwise, int tiles, int TR, int WK, int rounds, int gate_up) {
  constexpr int VPS = 512 / WBITS;            // weight values per row per step
  constexpr int UPS = VPS * 2 / 16;           // 16-byte activation units per token per step: 16 or 8
  constexpr int UPL = UPS / 4;                // units per lane per step: 4 or 2
  constexpr int ROWS_X = NT * 8;              // token rows held in shared memory
  constexpr int CHUNK_UNITS = kChunkSteps * UPS;
  constexpr int PITCH = CHUNK_UNITS * 16 + 16;
  constexpr int STAGE_BYTES = ROWS_X * PITCH;
  constexpr int THREADS = kStagedWarps * 32;
  constexpr float kBias = Bias<XT, WBITS>::value;
  constexpr int kRedPitch = 17;
  constexpr bool kLateFetch = NT == 4;
  static_assert(kStagedWarps * kRedPitch * ROWS_X * 4 <= 2 * STAGE_BYTES, "the reduction buffer reuses the ring");
  extern __shared__ __align__(16) unsigned char smem[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ts = warp / WK, wk = warp - ts * WK;   // tile slot of this warp and its share of the K steps
  const int64_t pitch = (int64_t)K * WBITS / 8;
  const int steps = K / VPS;
  const int nchunks = (steps + kChunkSteps - 1) / kChunkSteps;
  // FOLD_EVERY: every step of this warp ends a scale block (blockwise, and the warp's stride of WK steps is
  // a multiple of the block length); the per-step accumulators then start from zero in every step.
  // Fragment reads: a lane reads UPL units of 16 bytes per token and step.  The swizzle bit of unit
  // 16*ls + 4*t + q (int4) is bit 1 of t, a per-lane constant, and it only exchanges the unit pairs {0,1} and
  // {2,3}; for int8 (unit 8*ls + 2*t + q) it is the parity of the step and moves the pair by +-2 units.
  const uint32_t lane_row = (uint32_t)g * PITCH;
  uint32_t off_a, off_b;  // int4: byte offsets of weight words {0,1} and {2,3}; int8: even / odd steps
  if constexpr (WBITS == 4) {
    const uint32_t sw = (uint32_t)(t >> 1) << 5;
    off_a = lane_row + 64u * t + sw;
    off_b = lane_row + 64u * t + (sw ^ 32u);
  } else {
    off_a = lane_row + 32u * t;
    off_b = lane_row + ((32u * t) ^ 32u);
  }
  const int last_step = steps - 1;

  // cp.async of chunk c into ring slot c & 1 (tokens beyond M are zero-filled)
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
  constexpr int ROW_STEP = THREADS / CHUNK_UNITS;  // token rows covered by one pass of the CTA
  static_assert(THREADS % CHUNK_UNITS == 0, "a thread keeps its unit over the passes");
  const int cp_u = tid % CHUNK_UNITS, cp_r = tid / CHUNK_UNITS;
  const uint32_t cp_dst = smem_base + cp_r * PITCH + swz_unit(cp_u) * 16;
  const XT* cp_src = x + (int64_t)cp_r * K + cp_u * 8;
  auto issue_chunk = [&](int c) {
    const int units_here = min(kChunkSteps, steps - c * kChunkSteps) * UPS;
    if (cp_u < units_here) {
      const uint32_t dst = cp_dst + (uint32_t)(c & 1) * STAGE_BYTES;
      const XT* src = cp_src + (int64_t)c * (kChunkSteps * VPS);
#pragma unroll
      for (int it = 0; it < ROWS_X / ROW_STEP; ++it) {
        const bool ok = cp_r + it * ROW_STEP < M;
        cp_async_16(dst + it * ROW_STEP * PITCH, ok ? (const void*)(src + (int64_t)it * ROW_STEP * K) : (const void*)x, ok ? 16 : 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  static_assert((ROWS_X * CHUNK_UNITS) % THREADS == 0, "whole copies per thread");

  bool first = true;
  for (int round = 0; round < rounds; ++round) {
    const int tile = blockIdx.x + (round * TR + ts) * gridDim.x;
    const bool active = ts < TR && tile < tiles;
    const uint8_t* wrow[2];
    const float* srow[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int n = (active ? tile : 0) * 16 + g + 8 * r;
      if (n >= N) n = N - 1;
      wrow[r] = w + n * pitch + 16 * t;
      srow[r] = scale + n;
    }
    // the step after which this warp adds its per-step sums, times the block scale, to the totals
    auto folds = [&](int s) {
      if constexpr (FOLD_EVERY) return true;
      const int sn = s + WK;
      if (sn >= steps) return true;
      if (!blockwise) return false;
      const int b = spb_shift >= 0 ? (s >> spb_shift) : (s / steps_per_block);
      const int bn = spb_shift >= 0 ? (sn >> spb_shift) : (sn / steps_per_block);
      return bn != b;
    };
    // Weight and scale loads of the warp's steps, in step order.  In the four-tile FOLD_EVERY kernel the pointers
    // just advance by the warp's stride; otherwise the address comes from the step index.  A step beyond the
    // warp's share re-reads the last one (in bounds, never used).
    const uint8_t* wp0 = wrow[0] + wk * 64;
    const uint8_t* wp1 = wrow[1] + wk * 64;
    const int64_t wstride = (int64_t)WK * 64;
    const float *sp0 = srow[0], *sp1 = srow[1];
    int64_t sstride = 0;
    if constexpr (FOLD_EVERY && kLateFetch) {
      sp0 += (int64_t)(wk >> spb_shift) * N;
      sp1 += (int64_t)(wk >> spb_shift) * N;
      sstride = (int64_t)(WK >> spb_shift) * N;
    }
    auto fetch = [&](int s, StagedStep& d) {
      if constexpr (FOLD_EVERY && kLateFetch) {
        d.w[0] = ld_stream_u4(wp0);
        d.w[1] = ld_stream_u4(wp1);
        d.sc[0] = __ldg(sp0);
        d.sc[1] = __ldg(sp1);
        if (s + WK < steps) {
          wp0 += wstride;
          wp1 += wstride;
          sp0 += sstride;
          sp1 += sstride;
        }
      } else {
        const int sf = min(s, last_step);
#pragma unroll
        for (int r = 0; r < 2; ++r) d.w[r] = ld_stream_u4(wrow[r] + sf * 64);
        if (blockwise) {
          const int b = spb_shift >= 0 ? (sf >> spb_shift) : (sf / steps_per_block);
#pragma unroll
          for (int r = 0; r < 2; ++r) d.sc[r] = __ldg(srow[r] + (int64_t)b * N);
        }
      }
    };
    StagedStep qa, qb;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      qa.w[r] = qb.w[r] = make_uint4(0, 0, 0, 0);
      qa.sc[r] = qb.sc[r] = 1.f;
    }
    if (active && wk < steps) {
      fetch(wk, qa);
      fetch(wk + WK, qb);
    }
    if (first) {
      // weights are static: their first loads may overlap the previous kernel of the stream; the
      // activations and every store of this kernel come after the wait
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      asm volatile("griddepcontrol.wait;" ::: "memory");
      first = false;
    }
    issue_chunk(0);
    if (nchunks > 1) issue_chunk(1);

    float total[NT][4], part[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) total[i][j] = part[i][j] = 0.f;

    // one K step: convert q's weights, multiply with the chunk's activations, fold, refill q two steps ahead
    auto do_step = [&](int s, int c, StagedStep& q) {
      const uint4 w0 = q.w[0], w1 = q.w[1];
      const float sc0 = q.sc[0], sc1 = q.sc[1];
      if constexpr (!kLateFetch) fetch(s + 2 * WK, q);
      const int ls = s - c * kChunkSteps;
      const unsigned char* xs = smem + ((uint32_t)(c & 1) * STAGE_BYTES + (uint32_t)ls * (UPS * 16));
      if constexpr (FOLD_EVERY && !kLateFetch) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
      }
      if constexpr (WBITS == 4) {
        const unsigned char* xa = xs + off_a;
        const unsigned char* xb = xs + off_b;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          uint32_t pa[4], pb[4];
          cvt_s4x8_biased<XT>(reinterpret_cast<const uint32_t*>(&w0)[wi], pa);
          cvt_s4x8_biased<XT>(reinterpret_cast<const uint32_t*>(&w1)[wi], pb);
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) {
            pa[qd] = sub_bias<XT>(pa[qd], kBias);
            pb[qd] = sub_bias<XT>(pb[qd], kBias);
          }
          const uint32_t a_lo[4] = {pa[0], pb[0], pa[1], pb[1]};
          const uint32_t a_hi[4] = {pa[2], pb[2], pa[3], pb[3]};
          const unsigned char* xp = (wi < 2 ? xa : xb) + (wi & 1) * 16;
          uint4 xv[NT];
#pragma unroll
          for (int i = 0; i < NT; ++i) xv[i] = *reinterpret_cast<const uint4*>(xp + i * 8 * PITCH);
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            if (FOLD_EVERY && kLateFetch && wi == 0)
              mma_16816_nv_first<XT>(part[i], a_lo, xv[i].x, xv[i].y);
            else
              mma_16816_nv<XT>(part[i], a_lo, xv[i].x, xv[i].y);
          }
#pragma unroll
          for (int i = 0; i < NT; ++i) mma_16816_nv<XT>(part[i], a_hi, xv[i].z, xv[i].w);
        }
      } else {
        const unsigned char* xq = xs + ((ls & 1) ? off_b : off_a);
#pragma unroll
        for (int wp = 0; wp < 2; ++wp) {  // two weight words share one 16-byte activation unit
          uint32_t a[2][4];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t pa[2], pb[2];
            cvt_s8x4_biased<XT>(reinterpret_cast<const uint32_t*>(&w0)[2 * wp + h], pa);
            cvt_s8x4_biased<XT>(reinterpret_cast<const uint32_t*>(&w1)[2 * wp + h], pb);
            if constexpr (kBias != 0.f) {
#pragma unroll
              for (int qd = 0; qd < 2; ++qd) {
                pa[qd] = sub_bias<XT>(pa[qd], kBias);
                pb[qd] = sub_bias<XT>(pb[qd], kBias);
              }
            }
            a[h][0] = pa[0];
            a[h][1] = pb[0];
            a[h][2] = pa[1];
            a[h][3] = pb[1];
          }
          const unsigned char* xp = xq + wp * 16;
          uint4 xv[NT];
#pragma unroll
          for (int i = 0; i < NT; ++i) xv[i] = *reinterpret_cast<const uint4*>(xp + i * 8 * PITCH);
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            if (FOLD_EVERY && kLateFetch && wp == 0)
              mma_16816_nv_first<XT>(part[i], a[0], xv[i].x, xv[i].y);
            else
              mma_16816_nv<XT>(part[i], a[0], xv[i].x, xv[i].y);
          }
#pragma unroll
          for (int i = 0; i < NT; ++i) mma_16816_nv<XT>(part[i], a[1], xv[i].z, xv[i].w);
        }
      }
      // refill q for the step after next.  With four token tiles a step is long enough for the loads to land
      // when they are issued at its end, which saves the register copies of q; with two tiles they go first.
      if constexpr (kLateFetch) fetch(s + 2 * WK, q);
      if (folds(s)) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          total[i][0] = fmaf(sc0, part[i][0], total[i][0]);
          total[i][1] = fmaf(sc0, part[i][1], total[i][1]);
          total[i][2] = fmaf(sc1, part[i][2], total[i][2]);
          total[i][3] = fmaf(sc1, part[i][3], total[i][3]);
          if constexpr (!FOLD_EVERY) {
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
          }
        }
      }
    };

    int s = wk;
    for (int c = 0; c < nchunks; ++c) {
      if (c + 1 < nchunks)
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      else
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
      const int s_end = min((c + 1) * kChunkSteps, steps);
      if (active) {
        // steps alternate between the two in-flight slots; pairs keep the slot names static
        for (; s + WK < s_end; s += 2 * WK) {
          do_step(s, c, qa);
          do_step(s + WK, c, qb);
        }
        if (s < s_end) {  // odd count in this chunk: run one step and swap the slots
          do_step(s, c, qa);
          s += WK;
          const StagedStep tmp = qa;
          qa = qb;
          qb = tmp;
        }
      }
      __syncthreads();  // every warp is done with ring slot c & 1
      if (c + 2 < nchunks) issue_chunk(c + 2);
    }

    // cross-warp reduction through the (now idle) ring, then the store
    float* red = reinterpret_cast<float*>(smem);
    if (active) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        // token-major with a pitch of 17 floats: rows g, g+8 of tokens 2t, 2t+1 land on distinct banks
        float* r0 = red + (warp * ROWS_X + 8 * i + 2 * t) * kRedPitch + g;
        r0[0] = total[i][0];
        r0[kRedPitch] = total[i][1];
        r0[8] = total[i][2];
        r0[kRedPitch + 8] = total[i][3];
      }
    }
    __syncthreads();
    for (int idx = tid; idx < TR * 16 * ROWS_X; idx += THREADS) {
      const int slot = idx / (16 * ROWS_X), rem = idx - slot * (16 * ROWS_X);
      const int row = rem & 15, tok = rem >> 4;  // consecutive threads -> consecutive n
      const int otile = blockIdx.x + (round * TR + slot) * gridDim.x;
      const int n = otile * 16 + row;
      if (otile < tiles && n < N && tok < M) {
        float v = 0.f;
        for (int j = 0; j < WK; ++j) v += red[((slot * WK + j) * ROWS_X + tok) * kRedPitch + row];
        if (!blockwise) v *= __ldg(scale + n);
        if (!gate_up) {
          store_from_f32(out, (int64_t)tok * N + n, out_dt, v);
        } else if ((row & 8) == 0) {
          float u = 0.f;
          for (int j = 0; j < WK; ++j) u += red[((slot * WK + j) * ROWS_X + tok) * kRedPitch + row + 8];
          if (!blockwise) u *= __ldg(scale + n + 8);
          store_from_f32(out, (int64_t)tok * (N >> 1) + gate_up_column(n), out_dt, silu_mul(v, u));
        }
      }
    }
    __syncthreads();  // the ring is refilled next round
  }
}

// Launch with programmatic stream serialization: this kernel may be scheduled while the previous
// kernel of the stream drains, and parks at its griddepcontrol.wait until that kernel has finished.
template <typename Kernel, typename... Args>
cudaError_t launch_pdl(Kernel kern, unsigned grid, unsigned block, size_t smem_bytes, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int WBITS, typename XT, int NT>
cudaError_t launch_staged(const XT* xp, const uint8_t* wp, const float* scale, void* out, int out_dt, int64_t M,
                          int64_t N, int64_t K, int spb, int shift, int bw, int gate_up, cudaStream_t st) {
  constexpr int VPS = 512 / WBITS;
  constexpr int PITCH = kChunkSteps * (VPS * 2 / 16) * 16 + 16;
  constexpr size_t kSmem = 2 * (size_t)(NT * 8) * PITCH;
  const int tiles = (int)ceil_div(N, 16);
  const int grid = (int)std::min<int64_t>(sm_count(), tiles);
  const int per_cta = (int)ceil_div(tiles, grid);
  int tr = 1;
  while (tr < per_cta && tr < 8) tr *= 2;          // row tiles a CTA works on at a time
  const int wk = std::min(kStagedWarps / tr, 8);   // warps sharing the K steps of one tile
  const int rounds = (int)ceil_div(per_cta, tr);
  const bool fold_every = bw && wk % spb == 0;
  auto kern = fold_every ? decode_mma_staged_kernel<WBITS, XT, NT, true> : decode_mma_staged_kernel<WBITS, XT, NT, false>;
  static bool configured[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !configured[dev][fold_every]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
    if (e != cudaSuccess) return e;
    if (dev < 64) configured[dev][fold_every] = true;
  }
  return launch_pdl(kern, (unsigned)grid, kStagedWarps * 32, kSmem, st, xp, wp, scale, out, out_dt, (int)M, (int)N, (int)K, spb,
                    shift, bw, tiles, tr, wk, rounds, gate_up);
}

template <int WBITS, typename XT>
int launch_nt(const void* x, const void* w, const float* scale, void* out, int out_dt, int64_t M, int64_t N,
              int64_t K, int64_t block_size, int gate_up, cudaStream_t st, const ArParams* ar = nullptr) {
  constexpr int VPS = 512 / WBITS;
  const int spb = block_size > 0 ? (int)(block_size / VPS) : 1;
  int shift = -1;
  if ((spb & (spb - 1)) == 0) {
    shift = 0;
    while ((1 << shift) < spb) ++shift;
  }
  const int bw = block_size > 0 ? 1 : 0;
  const XT* xp = reinterpret_cast<const XT*>(x);
  const uint8_t* wp = reinterpret_cast<const uint8_t*>(w);
#define QMM_DECODE_LAUNCH(NT, RG, WARPS)                                                                        \
  launch_pdl(decode_mma_kernel<WBITS, XT, NT, RG, WARPS>, (unsigned)ceil_div(N, 16 * RG), WARPS * 32, 0, st, xp, wp, \
             scale, out, out_dt, (int)M, N, K, spb, shift, bw, gate_up, ArParams{}, (uint32_t*)nullptr)
  // one token tile: many small CTAs, activations through L1 (64 KB for 8 tokens of 4096);
  // two or four tiles: one CTA per SM with the activations staged in shared memory
  //
  // Warps per 16-row tile of the one-token-tile kernel.  With few row tiles (a narrow projection, a tensor-parallel
  // shard) four warps per tile leave an SM with a dozen warps, too few to cover the load latency; more warps then
  // share the tile's K steps.  Thresholds measured on B200 (M = 1 and 8): int4 weights 16 warps up to 512 tiles
  // (8192 x 28672: 76.7 -> 46.4 us; 4096 x 4096: 9.2 -> 5.2 us) and 4 from 896 tiles on; int8 weights 16 warps up to
  // 256 tiles (4096 x 4096: 12.9 -> 5.7 us), 8 up to 896 tiles (14336 x 4096: 20.6 -> 16.6 us; 8192 x 8192:
  // 37.9 -> 16.9 us), 4 at 1792 tiles.
  const int64_t tiles = ceil_div(N, 16), sms = sm_count();
  int warps;
  if (WBITS == 4)
    warps = tiles < 5 * sms ? 16 : 4;
  else
    warps = tiles < 2 * sms ? 16 : tiles < 8 * sms ? 8 : 4;
  cudaError_t err;
  if (ar) {
    if (M > 8 || gate_up) return fail(QMM_ERR_UNSUPPORTED, "fused row-parallel exchange: M <= 8 only (got %lld)", (long long)M);
    ArParams a = *ar;
    a.tiles = (uint32_t)tiles;
    // always four warps per tile here: a CTA that waits for its peers' tiles holds its SM slot, and with 16-warp
    // CTAs only one is resident per SM, so nothing else would run under the wait (measured: 86 vs 81 us on the
    // two-GPU MLP)
    err = launch_pdl(decode_mma_kernel<WBITS, XT, 1, 1, 4, true>, (unsigned)tiles, 128, 0, st, xp, wp, scale, out, out_dt,
                     (int)M, N, K, spb, shift, bw, 0, a, device_error_word());
  } else if (M <= 8) {
    if (warps >= 16)
      err = QMM_DECODE_LAUNCH(1, 1, 16);
    else if (warps >= 8)
      err = QMM_DECODE_LAUNCH(1, 1, 8);
    else
      err = QMM_DECODE_LAUNCH(1, 1, 4);
  }
  else if (M <= 16)
    err = launch_staged<WBITS, XT, 2>(xp, wp, scale, out, out_dt, M, N, K, spb, shift, bw, gate_up, st);
  else
    err = launch_staged<WBITS, XT, 4>(xp, wp, scale, out, out_dt, M, N, K, spb, shift, bw, gate_up, st);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_LAUNCH, "decode_mma_kernel launch: %s", cudaGetErrorString(err));
  }
#undef QMM_DECODE_LAUNCH
  return check_launch("decode_mma_kernel");
}

}  // namespace

int launch_decode_mma_allreduce(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt,
                                int64_t M, int64_t N, int64_t K, int64_t block_size, void* const* peer_bufs, int rank,
                                int world, int64_t slot_floats, cudaStream_t st) {
  if (world < 1 || world > kArMaxRanks || rank < 0 || rank >= world)
    return fail(QMM_ERR_BAD_SHAPE, "fused row-parallel exchange: rank %d of %d (at most %d ranks)", rank, world, kArMaxRanks);
  if (M > 8 || !decode_mma_supported(wbits, M, N, K, block_size, x, x_dt, w, false))
    return fail(QMM_ERR_UNSUPPORTED, "fused row-parallel exchange: needs 1<=M<=8, bf16/f16 activations, K a multiple of %d "
                "(M=%lld N=%lld K=%lld bs=%lld)", 512 / wbits, (long long)M, (long long)N, (long long)K, (long long)block_size);
  if (slot_floats < M * N || slot_floats > 0xffffffffLL) return fail(QMM_ERR_WORKSPACE, "fused row-parallel exchange: data slot too small");
  ArParams a = {};
  for (int r = 0; r < world; ++r) {
    if (!peer_bufs[r]) return fail(QMM_ERR_NULL, "fused row-parallel exchange: null buffer of rank %d", r);
    a.data[r] = reinterpret_cast<float*>(peer_bufs[r]);
  }
  a.rank = rank;
  a.world = world;
  a.slot_floats = (uint32_t)slot_floats;
  a.wait_cycles = peer_wait_cycles();
  if (wbits == 4) {
    if (x_dt == QMM_BF16) return launch_nt<4, __nv_bfloat16>(x, w, scale, out, out_dt, M, N, K, block_size, 0, st, &a);
    return launch_nt<4, __half>(x, w, scale, out, out_dt, M, N, K, block_size, 0, st, &a);
  }
  if (x_dt == QMM_BF16) return launch_nt<8, __nv_bfloat16>(x, w, scale, out, out_dt, M, N, K, block_size, 0, st, &a);
  return launch_nt<8, __half>(x, w, scale, out, out_dt, M, N, K, block_size, 0, st, &a);
}

bool decode_mma_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x, int x_dt,
                          const void* w, bool has_zp) {
  if (has_zp) return false;
  if (x_dt != QMM_BF16 && x_dt != QMM_F16) return false;
  if (M < 1 || M > 32 || N < 1 || K < 1) return false;
  const int vps = 512 / wbits;
  if (K % vps != 0) return false;                                 // whole 64-byte steps per weight row
  if (block_size > 0 && block_size % vps != 0) return false;      // a step stays inside one scale block
  if (!aligned(x, 16) || !aligned(w, 16)) return false;
  if (N > 2147483647LL - 16 || K > 2147483647LL) return false;    // 32-bit row and step indices
  return true;
}

int launch_decode_mma(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt,
                      int64_t M, int64_t N, int64_t K, int64_t block_size, cudaStream_t st, int gate_up) {
  if (gate_up && N % 16 != 0)
    return fail(QMM_ERR_BAD_SHAPE, "fused gate/up epilogue: the interleaved weight needs a multiple of 16 rows, got %lld",
                (long long)N);
  if (!decode_mma_supported(wbits, M, N, K, block_size, x, x_dt, w, false))
    return fail(QMM_ERR_UNSUPPORTED,
                "decode kernel: needs bf16/f16 activations, 1<=M<=32, K a multiple of %d, block_size a multiple of %d, "
                "16-byte aligned x/w, no zero point (M=%lld N=%lld K=%lld bs=%lld)",
                512 / wbits, 512 / wbits, (long long)M, (long long)N, (long long)K, (long long)block_size);
  if (wbits == 4) {
    if (x_dt == QMM_BF16) return launch_nt<4, __nv_bfloat16>(x, w, scale, out, out_dt, M, N, K, block_size, gate_up, st);
    return launch_nt<4, __half>(x, w, scale, out, out_dt, M, N, K, block_size, gate_up, st);
  }
  if (x_dt == QMM_BF16) return launch_nt<8, __nv_bfloat16>(x, w, scale, out, out_dt, M, N, K, block_size, gate_up, st);
  return launch_nt<8, __half>(x, w, scale, out, out_dt, M, N, K, block_size, gate_up, st);
}

}  // namespace qmm
