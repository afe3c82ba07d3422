// Weight-only (W8A16 / W4A16) linear for decode and small prefill batches on the integer tensor cores,
// with NO weight conversion on the CUDA cores:
//
//   out[m,n] = sum_b scale[b,n] * (sum_{k in block b} x[m,k] * w[n,k])          (per-channel: one block)
//
// Replaces the reference's mixed-dtype dot and blockwise einsum pair
// (torch_xla/experimental/xla_quantized_matmul.py:113-114, :120-124, :152-170).
//
// Idea.  The weights are already integers; only the activations are floating point.  Each activation row is
// rewritten, exactly, as a fixed-point number relative to the row's largest exponent,
//     x[m,k] = X[m,k] * 2^(e_m - 21),   X integer, |X| < 2^22,   X = l0 + 256*l1 + 65536*l2,  l_i in [-128,127]
// (a bf16/f16 value whose exponent is within 14 of the row maximum is represented exactly; smaller ones are rounded
// at 2^-22 of the row maximum, the error scale of an fp32 accumulation).  The three int8 "limb" rows of a token
// become three columns of the MMA's token operand, so that
//     sum_k x[m,k] w[n,k] = 2^(e_m-21) * ( A0 + 256*A1 + 65536*A2 ),   A_i = sum_k l_i[m,k] * w[n,k]   (int32, exact)
// and the int8 weights go TMA -> shared memory -> tcgen05.mma.kind::i8 untouched.  int4 weights (two's complement
// nibbles, two per byte) only need their nibbles moved into the high half of a byte (value * 16 as int8: three
// integer instructions per eight weights instead of the nine-plus-four of an int4 -> bf16 conversion); the factor
// 16 is folded into the per-token power of two.
//
// Structure.  "Swap-AB": 128 weight rows are the MMA's M side, the limb columns (3 per token, 16..128) its N side.
//   split_rows_kernel   one CTA per token: row maximum, limbs (in the k order the weight operand uses), 2^(e-21)
//   limb_tc_kernel      one CTA per SM, stream-K: the (row tile, 256-value K slot) units are dealt to the CTAs in
//                       equal contiguous shares, so every SM streams the same number of weight bytes whatever N and
//                       K; a tile that spans several CTAs is summed by the CTA that holds its first K range from
//                       fp32 partials the others leave in global scratch (fixed order: deterministic)
//     warp 0            TMA producer of weight bytes (two 128-row x 128-byte tiles per slot, 128-byte swizzle)
//     warp 1            MMA issuer: eight tcgen05.mma.kind::i8 (M128 x N=NCOLS x K32) per slot behind ONE barrier
//                       wait and ONE commit; one TMEM accumulator per scale block, several blocks in flight
//     warp 2            TMA producer of the limb tiles (two NCOLS-row x 128-byte tiles per slot)
//     warps 4..7        drain: tcgen05.ld a block's int32 sums, recombine the limbs in fp32, fold with scale[b,n]
//     warps 8..15       (int4 only) nibble -> byte expansion, raw ring -> operand slots; two groups of four warps
//                       take alternate slots
// Weight bytes in flight per SM = the depth of the TMA ring (64-190 KB), independent of registers and occupancy.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace qmm {

namespace {

constexpr int BMW = 128;                    // weight rows per tile (UMMA M)
constexpr int kTileK = 128;                 // k values per operand tile = one 128-byte swizzle row of int8
constexpr int kSlotK = 256;                 // k values per ring slot: two operand tiles
constexpr int UMMA_K = 32;                  // kind::i8
constexpr uint32_t kATile = BMW * 128;      // 16 KB
constexpr uint32_t kASlot = 2 * kATile;     // 32 KB
constexpr uint32_t kRawBytes = BMW * 128;   // one raw int4 slot: 128 rows x 256 nibbles
constexpr int kDrainWarp0 = 4;
constexpr int kConvWarp0 = 8;
constexpr int kMaxAcc = 8;
constexpr uint32_t kSmemBudget = 227 * 1024 - 1024 /*alignment*/ - 1024 /*barriers*/;

// Optional per-role cycle accounting of CTA 0 (compile with -DQMM_LIMB_DBG; never in the shipped build).
#ifdef QMM_LIMB_DBG
}  // namespace
__device__ long long g_limb_dbg[64];
__device__ long long g_limb_cta[4 * 512];  // per CTA: entry, first slot full, MMAs issued, exit (globaltimer ns)
namespace {
#define DBG_DECL long long dbg_t = 0, dbg_w[4] = {0, 0, 0, 0}; const long long dbg_t0 = clock64(); (void)dbg_t
#define DBG_BEGIN() dbg_t = clock64()
#define DBG_END(i) dbg_w[i] += clock64() - dbg_t
#define DBG_STAMP(i) if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) g_limb_dbg[42 + (i)] = (long long)ptx::globaltimer_ns()
#define DBG_STAMP1(i) if (blockIdx.x == 1 && (threadIdx.x & 31) == 0) g_limb_dbg[42 + (i)] = (long long)ptx::globaltimer_ns()
#define DBG_FLUSH(base)                                                  \
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {                      \
    for (int i_ = 0; i_ < 4; ++i_) g_limb_dbg[(base) + i_] = dbg_w[i_];  \
    g_limb_dbg[(base) + 4] = clock64() - dbg_t0;                         \
  }
#else
#define DBG_DECL
#define DBG_BEGIN()
#define DBG_END(i)
#define DBG_STAMP(i)
#define DBG_STAMP1(i)
#define DBG_FLUSH(base)
#endif

enum LimbErr : uint32_t { kErrPartialWait = 9 };  // owner CTA never saw a partial tile arrive

// How the K axis maps onto accumulators.
enum Mode : int {
  kPerChannel = 0,  // one accumulation per (tile, K range of the CTA)
  kBlock128 = 1,    // scale blocks of 128: two blocks per slot
  kBlockSlots = 2,  // scale blocks of spb whole slots
};

struct Params {
  const float* scale;  // [N] or [S,N]
  const float* pw;     // [M]: 2^(e_m - 21) (times 1/16 for int4 weights)
  void* out;
  int out_dt;
  int M;
  int64_t N;   // weight rows of this launch
  int64_t ld;  // row pitch of `out` and of the scale blocks (the whole layer's N when a launch covers a slice of rows)
  int w_dep;   // the weight operand is written by the kernel before this one (int4 expanded to int8 first)
  int tiles;   // ceil(N / 128)
  int slots;   // K slots per tile
  int spu;     // slots per scheduling unit (= slots per scale block in kBlockSlots mode, else 1)
  int ut;      // units per tile
  int mode;
  int S;       // scale blocks
  long long units;
  float* partial;   // [grid][MT][128] fp32
  uint32_t* flags;  // [grid], zero between launches
  uint32_t* err_word;
  int gate_up;
  int ytiles;    // token tiles per weight tile (1 up to one tile's tokens); a work item is a (weight tile, token tile) pair
  // The schedule: the first `items1` items go to the CTAs whole (CTA c takes items c, c + G, ...); the K units of
  // the remaining items (`units` of them) are dealt in equal contiguous shares to the first `g2` CTAs (stream-K: an
  // item that spans CTAs is summed through the partial tiles).  One token tile: items1 = 0, g2 = the grid.
  long long items1;
  int g2;
  int m0;      // first token of this launch inside the caller's batch (row offset of `out`)
};

// NL = limbs per token: three (22-bit fixed point: fp32-accumulation accuracy), or two (15 bits relative to the row's
// largest value: below the resolution of a 16-bit output) for the widest tiles when the output is bf16 / f16.
template <int WBITS, int NCOLS, int NL = 3>
struct Cfg {
  static constexpr uint32_t kBTile = NCOLS * 128;
  // CTAs per SM.  With int4 weights and up to 48 limb columns a CTA takes at most half of an SM's shared memory, tensor memory and
  // registers, and two run side by side: whenever one pipeline waits (a hand-over between warps, the partial-tile
  // exchange at the end of a K range, its own start-up) the other's MMAs keep the tensor pipe and the weight stream
  // busy, and a kernel's first CTAs overlap the last ones of the kernel before it.
  static constexpr int kOcc = (WBITS == 4 && NCOLS <= 48) ? 2 : 1;
  static constexpr int kTmemCols = 512 / kOcc;
  static constexpr uint32_t kBudget = kOcc == 2 ? 110 * 1024 - 2048 : kSmemBudget;
  // int4 with up to 96 limb columns: the expanded weight operand lives in tensor memory (64 columns per slot, in the
  // upper half of the CTA's columns) and never touches shared memory; the ring slots then hold limb tiles only.
  // (Wider tiles need the columns for accumulators: with two operand slots and three accumulators the large-batch
  // tiles measured 20 % slower than with the operand in shared memory.)
  static constexpr bool kATmem = WBITS == 4 && NCOLS <= 96;
  static constexpr int kATmemSlotCols = 64;
  static constexpr int kATmemSlots = kTmemCols / 2 / kATmemSlotCols;
  static constexpr int kATmemCol0 = kTmemCols - kATmemSlots * kATmemSlotCols;
  static constexpr uint32_t kAInSlot = kATmem ? 0 : kASlot;
  static constexpr uint32_t kSlot = kAInSlot + 2 * kBTile;   // [A tile 0 | A tile 1 |] B tile 0 | B tile 1
  static constexpr int kSlots = kATmem ? kATmemSlots : (WBITS == 4 ? 2 : std::min<int>(6, kBudget / kSlot));
  // expanding warps: two groups of four that take alternate slots, or one group where two CTAs share the SM
  static constexpr int kGroups = WBITS == 4 ? (kOcc == 2 ? 1 : 2) : 0;
  static constexpr int kRawFit = WBITS == 4 ? (int)((kBudget - kSlots * kSlot) / kRawBytes) : 0;
  static constexpr int kRaw = WBITS == 4 ? std::min(10, kGroups == 2 ? (kRawFit & ~1) : kRawFit) : 0;
  static constexpr int kAccCols = kATmem ? kATmemCol0 : kTmemCols;
  static constexpr int kRegions = std::min(2 * kMaxAcc, kAccCols / NCOLS);   // accumulators that fit in TMEM
  // two accumulators of a block-128 slot share one hand-over between MMA issuer and drain warps
  static constexpr bool kPair = kRegions >= 4;
  static constexpr int kTokens = NCOLS / NL;
  // drain warps: four (one per TMEM lane quadrant), or eight for the large-batch tiles, where the two warps of a
  // quadrant take half of the tile's tokens each (the per-block rescaling is what bounds that mode)
  static constexpr int kHalves = NCOLS == 128 ? 2 : 1;
  // tensor-memory loads of the drain double-buffered in registers: tiles of more than 16 tokens, where the register
  // budget allows (the int4 instances of the widest tiles run 640 threads)
  static constexpr bool kPipeDrain = NCOLS >= 96 && !(WBITS == 4 && NCOLS == 128);
  static constexpr int kXDrainWarp0 = 8 + 4 * kGroups;
  static constexpr int kThreads = 256 + 128 * kGroups + 128 * (kHalves - 1);
  static constexpr size_t kSmem = 1024 + (size_t)kRaw * kRawBytes + (size_t)kSlots * kSlot + 1024;
  static_assert(kSlots >= 2 && (WBITS == 8 || kRaw >= 2), "ring depths");
  static_assert(kGroups != 2 || (kSlots % 2 == 0 && kRaw % 2 == 0), "a ring slot always belongs to the same group");
  static_assert(kRegions >= 2, "two accumulators, so that drain and MMA overlap");
  static_assert(kSmem <= (kOcc == 2 ? 110 * 1024 : 227 * 1024), "shared memory budget");
};

// The (item, unit range) fragments of this CTA's share of the schedule, in order.  Item i = (weight tile i / ytiles,
// token tile i % ytiles): the token tiles of one weight tile are neighbours in the order, run on neighbouring CTAs at
// the same time and share the tile's bytes in L2.
struct FragIter {
  long long u, hi;        // this CTA's range of the dealt units (counted from the first dealt item)
  int ut;
  int ytiles, y;          // number of token tiles, token tile of the current item
  long long item;         // the current fragment's item once next() returned true
  long long nxt, items1;  // whole items: the next one of this CTA, their number
  __device__ FragIter(const Params& p) : ut(p.ut), ytiles(p.ytiles), y(0), item(0), nxt(blockIdx.x), items1(p.items1) {
    const long long c = blockIdx.x;
    u = c < p.g2 ? c * p.units / p.g2 : 0;
    hi = c < p.g2 ? (c + 1) * p.units / p.g2 : 0;
  }
  __device__ bool next(int& tile, int& u0, int& u1) {
    if (nxt < items1) {
      item = nxt;
      nxt += gridDim.x;
      u0 = 0;
      u1 = ut;
    } else {
      if (u >= hi) return false;
      const long long rel = u / ut;
      item = items1 + rel;
      u0 = (int)(u - rel * ut);
      const long long rem = hi - u;
      u1 = (int)(rem < (long long)(ut - u0) ? u0 + rem : ut);
      u += u1 - u0;
    }
    tile = (int)(item / ytiles);
    y = (int)(item - (long long)tile * ytiles);
    return true;
  }
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.f + expf(-gate)) * up; }
__device__ __forceinline__ int64_t gate_up_column(int64_t n) { return ((n >> 4) << 3) + (n & 7); }

// ---- activation rows -> int8 limbs -------------------------------------------------------------------------------
// Order of k inside the operand rows.  int8 weights: natural.  int4 weights: the nibble expansion emits, per raw
// 16-byte chunk (32 nibbles, k = 32c + 8j + i), the 16 even-k values and then the 16 odd-k values, so value k sits at
// 32c + 16*(i & 1) + 4j + i/2; the limb rows are written in the same order.
template <typename XT>
__device__ __forceinline__ void load8(const XT* p, float* v);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* v) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* v) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float* v) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&a);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// 2^(q-e) and 2^(e-q) * pw_mul for a row whose largest |x| has the float bits `mx`; a row with a non-finite entry
// gets (0, NaN), an all-zero or denormal row any small exponent.  Three limbs: q = 21 (|X| < 2^22 of the 2^23 that
// balanced limbs hold).  Two limbs: balanced limbs hold -32896..32639, so q = 14 unless the row's largest value
// would round above 32639 (mantissa beyond 32639 / 16384), which takes q = 13.
template <int NL>
__device__ __forceinline__ void row_factors(uint32_t mx, float pw_mul, float& mult, float& pw) {
  int e = (int)(mx >> 23) - 127;
  const bool finite = e < 128;
  if (e < -100) e = -100;
  const int q = NL == 3 ? 21 : ((mx & 0x7fffffu) > 0x7EFE00u ? 13 : 14);
  mult = finite ? __uint_as_float((uint32_t)(q - e + 127) << 23) : 0.f;
  pw = finite ? __uint_as_float((uint32_t)(e - q + 127) << 23) * pw_mul : __uint_as_float(0x7fc00000u);
}

// Eight values -> the bytes of their three limbs, packed in k order (two words per limb).
// X = rint(v * mult) comes out of one FMA against 1.5 * 2^23 (the sum lands where fp32 spacing is 1, so the FMA's
// round-to-nearest-even IS the rint, and X sits in the low mantissa bits).  Balanced limbs l_i in [-128,127] with
// X = l0 + 256 l1 + 65536 l2 are the base-256 digits of X + 0x808080, each minus 128: one integer add puts the digits
// into bytes 0..2, one XOR with 0x808080 turns digit into limb.  Three instructions per value, then byte gathers.
// With two limbs the same holds for X + 0x8080 and bytes 0..1 (l2 is not written).
template <int NL>
__device__ __forceinline__ void split8(const float* v, float mult, uint32_t* l0, uint32_t* l1, uint32_t* l2) {
  constexpr uint32_t kBias = NL == 3 ? 0x808080u : 0x8080u;
  uint32_t z[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    z[i] = (__float_as_uint(fmaf(v[i], mult, 12582912.f)) + (kBias - 0x4B400000u)) ^ kBias;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t a = z[4 * h], b = z[4 * h + 1], c = z[4 * h + 2], d = z[4 * h + 3];
    // byte j of a/b in the low half, of c/d in the high half
    const uint32_t ab0 = __byte_perm(a, b, 0x0040), cd0 = __byte_perm(c, d, 0x0040);
    const uint32_t ab1 = __byte_perm(a, b, 0x0051), cd1 = __byte_perm(c, d, 0x0051);
    l0[h] = __byte_perm(ab0, cd0, 0x5410);
    l1[h] = __byte_perm(ab1, cd1, 0x5410);
    if constexpr (NL == 3) {
      const uint32_t ab2 = __byte_perm(a, b, 0x0062), cd2 = __byte_perm(c, d, 0x0062);
      l2[h] = __byte_perm(ab2, cd2, 0x5410);
    }
  }
}

// One CTA per token row.  xl: [NL*M][K] int8, row NL*m + l = limb l of token m; pw[m] = 2^(e_m - q) * pw_mul.
// A row with a non-finite entry gets pw = NaN (its outputs are NaN); an all-zero row gets zeros.
template <typename XT, int NL>
__global__ void __launch_bounds__(1024) split_rows_kernel(const XT* __restrict__ x, int8_t* __restrict__ xl, float* __restrict__ pw,
                                                          int64_t K, int perm4, float pw_mul) {
  __shared__ uint32_t s_max[32];
  if (blockIdx.x == 0 && threadIdx.x == 0) { DBG_STAMP(10); }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // x may come from the previous kernel of the stream
  if (blockIdx.x == 0 && threadIdx.x == 0) { DBG_STAMP(11); }
  const int m = blockIdx.x;
  const XT* xr = x + (int64_t)m * K;
  const int64_t groups = K >> 3;
  uint32_t mx = 0;
  for (int64_t gi = threadIdx.x; gi < groups; gi += blockDim.x) {
    float v[8];
    load8<XT>(xr + gi * 8, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = max(mx, __float_as_uint(v[i]) & 0x7fffffffu);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x < 32) {
    uint32_t t = threadIdx.x < (blockDim.x >> 5) ? s_max[threadIdx.x] : 0u;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = max(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (threadIdx.x == 0) s_max[0] = t;
  }
  __syncthreads();
  mx = s_max[0];
  float mult, pwv;
  row_factors<NL>(mx, pw_mul, mult, pwv);
  if (threadIdx.x == 0) pw[m] = pwv;
  int8_t* r0 = xl + (int64_t)(NL * m) * K;
  int8_t* r1 = r0 + K;
  int8_t* r2 = r1 + K;
  for (int64_t gi = threadIdx.x; gi < groups; gi += blockDim.x) {
    float v[8];
    load8<XT>(xr + gi * 8, v);
    uint32_t l0[2], l1[2], l2[2] = {0u, 0u};  // bytes of limb l for k = 8*gi + i, packed in k order
    split8<NL>(v, mult, l0, l1, l2);
    if (!perm4) {
      const int64_t o = gi * 8;
      *reinterpret_cast<uint2*>(r0 + o) = make_uint2(l0[0], l0[1]);
      *reinterpret_cast<uint2*>(r1 + o) = make_uint2(l1[0], l1[1]);
      if constexpr (NL == 3) *reinterpret_cast<uint2*>(r2 + o) = make_uint2(l2[0], l2[1]);
    } else {
      // k = 32*c + 8*j + i -> even i at 32*c + 4*j + i/2, odd i at 32*c + 16 + 4*j + i/2
      const int64_t base = (gi >> 2) * 32 + (gi & 3) * 4;
      auto evens = [](const uint32_t* l) { return __byte_perm(l[0], l[1], 0x6420); };
      auto odds = [](const uint32_t* l) { return __byte_perm(l[0], l[1], 0x7531); };
      *reinterpret_cast<uint32_t*>(r0 + base) = evens(l0);
      *reinterpret_cast<uint32_t*>(r0 + base + 16) = odds(l0);
      *reinterpret_cast<uint32_t*>(r1 + base) = evens(l1);
      *reinterpret_cast<uint32_t*>(r1 + base + 16) = odds(l1);
      if constexpr (NL == 3) {
        *reinterpret_cast<uint32_t*>(r2 + base) = evens(l2);
        *reinterpret_cast<uint32_t*>(r2 + base + 16) = odds(l2);
      }
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) { DBG_STAMP(12); }
}

// ---- int4 -> int8 once, for long batches ----
// Packed nibbles [rows, K/2] -> int8 [rows, K] holding value * 16 in natural k order.  Above a couple of hundred tokens
// the per-tile expansion inside the main kernel costs more than this pass over the weights (read N*K/2, write N*K
// bytes at HBM rate) plus the int8 kernel, which runs at more than twice the rate.  Thread = 8 packed bytes at a time
// (loads and 16-byte stores of a warp are contiguous).
__global__ void __launch_bounds__(256) expand_int4_kernel(const uint2* __restrict__ src, uint4* __restrict__ dst, int64_t chunks) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  constexpr int U = 4;  // loads in flight per thread
  uint2 q[U];
#pragma unroll
  for (int u = 0; u < U; ++u) q[u] = i + u * stride < chunks ? __ldcs(src + i + u * stride) : make_uint2(0, 0);
  asm volatile("griddepcontrol.wait;" ::: "memory");  // `dst` may still be read by the kernel before this one
  while (i < chunks) {
    uint2 qn[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t nx = i + (U + u) * stride;
      qn[u] = nx < chunks ? __ldcs(src + nx) : make_uint2(0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (i + u * stride < chunks) {
        const uint32_t lo0 = (q[u].x << 4) & 0xF0F0F0F0u, hi0 = q[u].x & 0xF0F0F0F0u;  // even k, odd k
        const uint32_t lo1 = (q[u].y << 4) & 0xF0F0F0F0u, hi1 = q[u].y & 0xF0F0F0F0u;
        dst[i + u * stride] = make_uint4(__byte_perm(lo0, hi0, 0x5140), __byte_perm(lo0, hi0, 0x7362),
                                         __byte_perm(lo1, hi1, 0x5140), __byte_perm(lo1, hi1, 0x7362));
      }
      q[u] = qn[u];
    }
    i += U * stride;
  }
}

// ---- the stream-K tensor-core kernel -----------------------------------------------------------------------------
// One accumulator (NCOLS int32 columns of this thread's TMEM lane) -> limbs recombined in fp32, times sc, into total.
// SMALL: every int32 sum is below 2^22 in magnitude (scale blocks of at most 256 values), so 256 * A1 + A0 still fits
// an int32 and one conversion serves both low limbs.
template <int NCOLS, int MT, int NL, bool SMALL, typename Release>
__device__ __forceinline__ void fold_region(uint32_t taddr, float sc, float (&total)[MT], bool release_after, Release release) {
  constexpr int CW = 16 * NL;  // columns of a chunk of 16 tokens
  constexpr int kChunks = (NCOLS + CW - 1) / CW;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    uint32_t r[CW];
#pragma unroll
    for (int j = 0; j < NL; ++j)
      if (c * CW + 16 * j < NCOLS) ptx::tmem_ld_32x32b_x16(taddr + c * CW + 16 * j, r + 16 * j);
    ptx::tmem_ld_wait();
    if (c == kChunks - 1 && release_after) release();  // the accumulator's last values are in registers
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      if (c * 16 + t < MT) {
        float lowf;
        if (SMALL) {
          lowf = __int2float_rn((int)r[NL * t + 1] * 256 + (int)r[NL * t]);
        } else {
          lowf = fmaf(__int2float_rn((int)r[NL * t + 1]), 256.f, __int2float_rn((int)r[NL * t]));
        }
        if constexpr (NL == 3) lowf = fmaf(__int2float_rn((int)r[NL * t + 2]), 65536.f, lowf);
        total[c * 16 + t] = fmaf(sc, lowf, total[c * 16 + t]);
      }
    }
  }
}

// The same for NREG accumulators in a row (`stride` columns apart, scale sc[i] each), with the tensor-memory loads of
// the next 16 tokens in flight while the current ones are folded: a load's round trip otherwise sits between every
// two chunks.  Costs a second set of 16 * NL registers.
template <int NCOLS, int MT, int NL, bool SMALL, int NREG, typename Release>
__device__ __forceinline__ void fold_regions_pipelined(uint32_t taddr, uint32_t stride, const float (&sc)[NREG], float (&total)[MT],
                                                       Release release) {
  constexpr int CW = 16 * NL;
  constexpr int kChunks = (NCOLS + CW - 1) / CW;
  constexpr int T = NREG * kChunks;
  if constexpr (NREG == 1 && NCOLS <= 64) {
    // one accumulator of up to 64 columns: all of it in one round trip
    constexpr int L16 = (NCOLS + 15) / 16;
    uint32_t v[16 * L16];
#pragma unroll
    for (int j = 0; j < L16; ++j) ptx::tmem_ld_32x32b_x16(taddr + 16 * j, v + 16 * j);
    ptx::tmem_ld_wait();
    release();
    const float s0 = sc[0];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      float lowf;
      if (SMALL) {
        lowf = __int2float_rn((int)v[NL * t + 1] * 256 + (int)v[NL * t]);
      } else {
        lowf = fmaf(__int2float_rn((int)v[NL * t + 1]), 256.f, __int2float_rn((int)v[NL * t]));
      }
      if constexpr (NL == 3) lowf = fmaf(__int2float_rn((int)v[NL * t + 2]), 65536.f, lowf);
      total[t] = fmaf(s0, lowf, total[t]);
    }
    return;
  }
  uint32_t r[2][CW];
  auto issue = [&](int i, uint32_t* dst) {
    const int reg = i / kChunks, c = i % kChunks;
#pragma unroll
    for (int j = 0; j < NL; ++j)
      if (c * CW + 16 * j < NCOLS) ptx::tmem_ld_32x32b_x16(taddr + reg * stride + c * CW + 16 * j, dst + 16 * j);
  };

  issue(0, r[0]);
#pragma unroll
  for (int i = 0; i < T; ++i) {
    uint32_t* cur = r[i & 1];
    ptx::tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < NL; ++j) ptx::tmem_ld_landed16(cur + 16 * j);
    if (i + 1 < T) issue(i + 1, r[(i + 1) & 1]);
    else release();  // the accumulators' last values are in registers
    const int c = i % kChunks;
    const float s = sc[i / kChunks];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      if (c * 16 + t < MT) {
        float lowf;
        if (SMALL) {
          lowf = __int2float_rn((int)cur[NL * t + 1] * 256 + (int)cur[NL * t]);
        } else {
          lowf = fmaf(__int2float_rn((int)cur[NL * t + 1]), 256.f, __int2float_rn((int)cur[NL * t]));
        }
        if constexpr (NL == 3) lowf = fmaf(__int2float_rn((int)cur[NL * t + 2]), 65536.f, lowf);
        total[c * 16 + t] = fmaf(s, lowf, total[c * 16 + t]);
      }
    }
  }
}

template <int WBITS, int NCOLS, int NL>
__global__ void __launch_bounds__(Cfg<WBITS, NCOLS, NL>::kThreads, Cfg<WBITS, NCOLS, NL>::kOcc)
    limb_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
  using C = Cfg<WBITS, NCOLS, NL>;
  constexpr int kRaw = C::kRaw, kSlots = C::kSlots;
  constexpr uint32_t kBTile = C::kBTile, kSlot = C::kSlot;
  constexpr int MT = C::kTokens;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* raw_base = smem;
  uint8_t* slot_base = raw_base + (size_t)kRaw * kRawBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(slot_base + (size_t)kSlots * kSlot);
  uint64_t* raw_full = bars;                       // [kRaw]    TMA bytes
  uint64_t* raw_empty = raw_full + (kRaw ? kRaw : 1);  // [kRaw]    4 expanding warps
  uint64_t* full = raw_empty + (kRaw ? kRaw : 1);      // [kSlots]  int8: both TMA producers; int4: 4 expanding warps + limb producer
  uint64_t* empty = full + kSlots;                 // [kSlots]  tcgen05.commit
  uint64_t* acc_full = empty + kSlots;             // [kMaxAcc] tcgen05.commit
  uint64_t* acc_empty = acc_full + kMaxAcc;        // [kMaxAcc] 4 drain warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kMaxAcc);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef QMM_LIMB_DBG
  const long long dbg_k0 = clock64();
  const unsigned long long dbg_g0 = ptx::globaltimer_ns();
#endif
  if (threadIdx.x == 0) { DBG_STAMP(0); }
#ifdef QMM_LIMB_DBG
  if (threadIdx.x == 0 && blockIdx.x < 512) g_limb_cta[4 * blockIdx.x] = (long long)ptx::globaltimer_ns();
#endif
  // accumulators per hand-over and hand-over buffers in the TMEM ring
  const int gph = (p.mode == kBlock128 && C::kPair) ? 2 : 1;
  const int nacc = min(kMaxAcc, C::kRegions / gph);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRaw; ++s) {
      ptx::mbar_init(&raw_full[s], 1);
      ptx::mbar_init(&raw_empty[s], 4);
    }
    for (int s = 0; s < kSlots; ++s) {
      // arrivals per slot: the weight side (int8: the TMA producer; int4: the four expanding warps of the slot's group)
      // and the limb tiles' TMA producer
      ptx::mbar_init(&full[s], (WBITS == 4 ? 4 : 1) + 1);
      ptx::mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < kMaxAcc; ++s) {
      ptx::mbar_init(&acc_full[s], 1);
      ptx::mbar_init(&acc_empty[s], 4 * C::kHalves);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_w);
    ptx::prefetch_tensormap(&map_x);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) { DBG_STAMP(1); }
  // The next kernel of the stream may start its own set-up now; it touches nothing of ours before its own wait.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ---------------- weight producer: needs nothing from earlier kernels, so it does not wait for them ----------------
    if (lane == 0) {
      if (p.w_dep) asm volatile("griddepcontrol.wait;" ::: "memory");
      FragIter it(p);
      DBG_DECL;
      int tile, u0, u1, slot = 0;
      uint32_t ph = 0;
      while (it.next(tile, u0, u1)) {
        const int s0 = u0 * p.spu, s1 = min(p.slots, u1 * p.spu);
        for (int s = s0; s < s1; ++s) {
          if constexpr (WBITS == 8) {
            DBG_BEGIN();
            ptx::mbar_wait<32>(&empty[slot], ph ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
            DBG_END(0);
            uint8_t* dst = slot_base + (size_t)slot * kSlot;
            ptx::mbar_expect_tx(&full[slot], kASlot);
            ptx::tma_load_2d(dst, &map_w, &full[slot], s * kSlotK, tile * BMW);
            ptx::tma_load_2d(dst + kATile, &map_w, &full[slot], s * kSlotK + kTileK, tile * BMW);
            if (++slot == kSlots) { slot = 0; ph ^= 1; }
          } else {
            DBG_BEGIN();
            ptx::mbar_wait<32>(&raw_empty[slot], ph ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
            DBG_END(0);
            ptx::mbar_expect_tx(&raw_full[slot], kRawBytes);
            ptx::tma_load_2d(raw_base + (size_t)slot * kRawBytes, &map_w, &raw_full[slot], s * 128, tile * BMW);
            if (++slot == kRaw) { slot = 0; ph ^= 1; }
          }
        }
      }
      DBG_FLUSH(0);
    }
  } else if (warp == 2) {
    // ---------------- limb tile producer ----------------
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");  // the limbs are written by the kernel before this one
      DBG_STAMP(2);
      FragIter it(p);
      DBG_DECL;
      int tile, u0, u1, slot = 0;
      uint32_t ph = 0;
      while (it.next(tile, u0, u1)) {
        const int s0 = u0 * p.spu, s1 = min(p.slots, u1 * p.spu);
        for (int s = s0; s < s1; ++s) {
          DBG_BEGIN();
          ptx::mbar_wait<32>(&empty[slot], ph ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
          DBG_END(0);
          uint8_t* dst = slot_base + (size_t)slot * kSlot + C::kAInSlot;
          ptx::mbar_expect_tx(&full[slot], 2 * kBTile);
          ptx::tma_load_2d(dst, &map_x, &full[slot], s * kSlotK, it.y * (NL * MT));
          ptx::tma_load_2d(dst + kBTile, &map_x, &full[slot], s * kSlotK + kTileK, it.y * (NL * MT));
          if (++slot == kSlots) { slot = 0; ph ^= 1; }
        }
      }
      DBG_FLUSH(8);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: the whole warp walks the loop, lane 0's instructions take effect ----------------
    constexpr uint32_t idesc = ptx::make_idesc(/*s32*/ 2, /*s8*/ 1, /*s8*/ 1, BMW, NCOLS);
    const uint32_t leader = lane == 0 ? 1u : 0u;
    const uint32_t desc_hi = (uint32_t)(ptx::make_sw128_kmajor_desc(0) >> 32);
    const uint32_t lo0 = (uint32_t)ptx::make_sw128_kmajor_desc(ptx::smem_u32(slot_base));
    FragIter it(p);
    DBG_DECL;
    int tile, u0, u1;
    int slot = 0, buf = 0;
    uint32_t ph = 0, pacc = 0;
    uint32_t lo = lo0;
    // the four MMAs of operand tile t of the current slot into accumulator d
    auto issue_tile = [&](uint32_t d, int t, uint32_t accum) {
      const uint32_t a_lo = lo + t * (kATile >> 4), b_lo = lo + (C::kAInSlot >> 4) + t * (kBTile >> 4);
#pragma unroll
      for (int k = 0; k < kTileK / UMMA_K; ++k) {
        const uint64_t bd = ((uint64_t)desc_hi << 32) | (uint64_t)(b_lo + k * (UMMA_K >> 4));
        if constexpr (C::kATmem) {
          // operand rows = TMEM lanes; one K=32 step = 8 columns = one expanded 16-byte chunk of nibbles
          const uint32_t a_tm = tmem_base + C::kATmemCol0 + slot * C::kATmemSlotCols + (4 * t + k) * 8;
          ptx::mma_i8_ts_pred(d, a_tm, bd, idesc, accum | (uint32_t)k, leader);
        } else {
          const uint64_t ad = ((uint64_t)desc_hi << 32) | (uint64_t)(a_lo + k * (UMMA_K >> 4));
          ptx::mma_i8_ss_pred(d, ad, bd, idesc, accum | (uint32_t)k, leader);
        }
      }
    };
    auto wait_acc = [&]() {
      DBG_BEGIN();
      ptx::mbar_wait(&acc_empty[buf], pacc ^ 1, abort_flag, p.err_word, ptx::kErrWaitTmemEmpty);
      DBG_END(0);
      ptx::tcgen05_fence_after();
    };
    auto next_acc = [&]() {
      ptx::mma_commit_pred(&acc_full[buf], leader);
      if (++buf == nacc) { buf = 0; pacc ^= 1; }
    };
    bool dbg_first = true;
    (void)dbg_first;
    auto wait_slot = [&]() {
      DBG_BEGIN();
      ptx::mbar_wait(&full[slot], ph, abort_flag, p.err_word, ptx::kErrWaitFull);
      DBG_END(1);
      if (dbg_first) {
        DBG_STAMP(3);
#ifdef QMM_LIMB_DBG
        if (lane == 0 && blockIdx.x < 512) g_limb_cta[4 * blockIdx.x + 1] = (long long)ptx::globaltimer_ns();
#endif
        dbg_first = false;
      }
      ptx::tcgen05_fence_after();
    };
    auto next_slot = [&]() {
      ptx::mma_commit_pred(&empty[slot], leader);  // frees the slot once the MMAs issued so far have read it
      lo += kSlot >> 4;
      if (++slot == kSlots) { slot = 0; ph ^= 1; lo = lo0; }
    };
    while (it.next(tile, u0, u1)) {
      const int s0 = u0 * p.spu, s1 = min(p.slots, u1 * p.spu);
      if (p.mode == kBlock128) {
        for (int s = s0; s < s1; ++s) {
          if (C::kPair) {
            wait_acc();
            wait_slot();
            const uint32_t d = tmem_base + buf * (2 * NCOLS);
            issue_tile(d, 0, 0);
            issue_tile(d + NCOLS, 1, 0);
            next_slot();
            next_acc();
          } else {
            wait_acc();
            wait_slot();
            issue_tile(tmem_base + buf * NCOLS, 0, 0);
            next_acc();
            wait_acc();
            issue_tile(tmem_base + buf * NCOLS, 1, 0);
            next_slot();
            next_acc();
          }
        }
      } else {
        int s = s0;
        while (s < s1) {
          const int g_end = p.mode == kBlockSlots ? min(s1, s + p.spu) : s1;  // fragments start on block boundaries
          wait_acc();
          const uint32_t d = tmem_base + buf * NCOLS;
          uint32_t accum = 0;
          for (; s < g_end; ++s) {
            wait_slot();
            issue_tile(d, 0, accum);
            issue_tile(d, 1, 1);
            accum = 1;
            next_slot();
          }
          next_acc();
        }
      }
    }
    DBG_STAMP(4);
#ifdef QMM_LIMB_DBG
    if (lane == 0 && blockIdx.x < 512) g_limb_cta[4 * blockIdx.x + 2] = (long long)ptx::globaltimer_ns();
#endif
    DBG_FLUSH(16);
  } else if ((warp >= kDrainWarp0 && warp < kDrainWarp0 + 4) || (C::kHalves == 2 && warp >= C::kXDrainWarp0)) {
    // ---------------- drain: thread = one weight row n (its TMEM lane), all or half of the tile's tokens ----------------
    constexpr int MTD = MT / C::kHalves;                      // tokens per drain thread
    constexpr int DC = C::kHalves == 2 ? 64 : NCOLS;          // accumulator columns a thread loads per block
    const int half = (C::kHalves == 2 && warp >= C::kXDrainWarp0) ? 1 : 0;
    const uint32_t col0 = (uint32_t)(half * NL * MTD);
    constexpr int kDT = 128 * C::kHalves;                     // drain threads
    const bool small = p.mode == kBlock128 || (p.mode == kBlockSlots && p.spu == 1);
    asm volatile("griddepcontrol.wait;" ::: "memory");  // pw, the scratch and `out` belong to earlier kernels until here
    if (warp == kDrainWarp0) { DBG_STAMP(5); }
    const int quad = warp & 3;
    const int rl = quad * 32 + lane;  // row inside the tile
    const int dt = half ? 128 + (int)threadIdx.x - C::kXDrainWarp0 * 32 : (int)threadIdx.x - kDrainWarp0 * 32;  // 0..kDT-1
    auto drain_bar = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(kDT) : "memory"); };
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    FragIter it(p);
    DBG_DECL;
    int tile, u0, u1, buf = 0;
    uint32_t pacc = 0;
    __shared__ int s_npart;
    __shared__ float s_pw[2][64];
    static_assert(MT <= 64, "per-token factors of a tile");
    int frag = 0;
    auto wait_acc = [&]() {
      DBG_BEGIN();
      ptx::mbar_wait_warp<32>(&acc_full[buf], pacc, abort_flag, p.err_word, ptx::kErrWaitTmemFull);
      DBG_END(0);
      ptx::tcgen05_fence_after();
    };
    auto release = [&]() {
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
    };
    auto next_acc = [&]() {
      if (++buf == nacc) { buf = 0; pacc ^= 1; }
    };
    while (it.next(tile, u0, u1)) {
      const int s0 = u0 * p.spu, s1 = min(p.slots, u1 * p.spu);
      const int64_t n = (int64_t)tile * BMW + rl;
      const bool n_ok = n < p.N;
      const bool first = u0 == 0, last = u1 == p.ut;
      const int mt0 = it.y * MT + half * MTD;  // first token this thread owns (0 outside item mode)
      const int mcount = p.M - mt0;          // tokens from there to the end of the batch
      // What the final store needs from global memory is fetched now, under the K loop: the per-channel scale into a
      // register, the tile's per-token factors into shared memory (two buffers: a fragment's barrier separates the
      // readers of one from the writers of its next use).  Fetched at the end they are two L2 round trips per tile.
      float* pw_s = s_pw[frag & 1];
      ++frag;
      const float ps = (p.mode != kPerChannel || !n_ok || !first) ? 1.f : __ldg(p.scale + n);
      if (first && dt < MT) pw_s[dt] = it.y * MT + dt < p.M ? __ldg(p.pw + it.y * MT + dt) : 0.f;
      float total[MTD];
#pragma unroll
      for (int t = 0; t < MTD; ++t) total[t] = 0.f;
      // A tile this CTA starts and others continue: their partial sums are added after this CTA's own K range, in
      // CTA order - always in that order, whenever they land, so that the result does not depend on timing.
      int np = 0;
      auto add_partials = [&]() {
        // two partial tiles in flight at a time (an L2 round trip each), added in CTA order
        const float* src = p.partial + ((size_t)(blockIdx.x + 1) * MT + half * MTD) * BMW + rl;
        constexpr size_t kTile = (size_t)MT * BMW;
        int j = 0;
        for (; C::kThreads <= 512 && j + 1 < np; j += 2) {  // (where the register budget allows)
          float a[MTD], b[MTD];
#pragma unroll
          for (int t = 0; t < MTD; ++t) {
            a[t] = t < mcount ? __ldcg(src + j * kTile + t * BMW) : 0.f;
            b[t] = t < mcount ? __ldcg(src + (j + 1) * kTile + t * BMW) : 0.f;
          }
#pragma unroll
          for (int t = 0; t < MTD; ++t) total[t] = (total[t] + a[t]) + b[t];
        }
        for (; j < np; ++j) {
#pragma unroll
          for (int t = 0; t < MTD; ++t)
            if (t < mcount) total[t] += __ldcg(src + j * kTile + t * BMW);
        }
        drain_bar();
        for (int j = dt; j < np; j += kDT) p.flags[blockIdx.x + 1 + j] = 0u;  // clean for the next launch
      };
      if (first && !last) {
        if (dt == 0) {
          int cnt = 0;
          for (long long c2 = blockIdx.x + 1; c2 < p.g2; ++c2) {
            if (c2 * p.units / p.g2 >= (it.item - p.items1 + 1) * p.ut) break;
            ++cnt;
          }
          s_npart = cnt;
        }
        drain_bar();
        np = s_npart;
      }
      // block scales are fetched four blocks ahead: a load issued in the iteration that uses it would put an L2
      // round trip into every block's drain
      constexpr int kAhead = 4;
      float scq[kAhead];
      int b_next = p.mode == kBlock128 ? 2 * s0 : (p.mode == kBlockSlots ? s0 / p.spu : 0);
      auto fetch_scale = [&]() {
        const float v = (p.mode != kPerChannel && n_ok && b_next < p.S) ? __ldg(p.scale + (int64_t)b_next * p.ld + n) : 0.f;
        ++b_next;
        return v;
      };
      auto pop_scale = [&]() {
        const float v = scq[0];
#pragma unroll
        for (int i = 0; i + 1 < kAhead; ++i) scq[i] = scq[i + 1];
        scq[kAhead - 1] = fetch_scale();
        return v;
      };
#pragma unroll
      for (int i = 0; i < kAhead; ++i) scq[i] = fetch_scale();
      if (p.mode == kBlock128) {
        for (int s = s0; s < s1; ++s) {
          if (C::kPair) {
            wait_acc();
            DBG_BEGIN();
            const uint32_t a = lane_addr + buf * (2 * NCOLS) + col0;
            if constexpr (C::kPipeDrain) {
              const float sc2[2] = {pop_scale(), pop_scale()};
              fold_regions_pipelined<DC, MTD, NL, true, 2>(a, NCOLS, sc2, total, release);
            } else {
              fold_region<DC, MTD, NL, true>(a, pop_scale(), total, false, release);
              fold_region<DC, MTD, NL, true>(a + NCOLS, pop_scale(), total, true, release);
            }
            DBG_END(1);
            next_acc();
          } else {
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
              wait_acc();
              DBG_BEGIN();
              if constexpr (C::kPipeDrain) {
                const float sc1[1] = {pop_scale()};
                fold_regions_pipelined<DC, MTD, NL, true, 1>(lane_addr + buf * NCOLS + col0, 0, sc1, total, release);
              } else {
                fold_region<DC, MTD, NL, true>(lane_addr + buf * NCOLS + col0, pop_scale(), total, true, release);
              }
              DBG_END(1);
              next_acc();
            }
          }
        }
      } else {
        int s = s0;
        while (s < s1) {
          const int g_end = p.mode == kBlockSlots ? min(s1, s + p.spu) : s1;
          const float sc = p.mode == kPerChannel ? 1.f : pop_scale();
          wait_acc();
          DBG_BEGIN();
          if constexpr (C::kPipeDrain) {
            const float sc1[1] = {sc};
            if (small) fold_regions_pipelined<DC, MTD, NL, true, 1>(lane_addr + buf * NCOLS + col0, 0, sc1, total, release);
            else fold_regions_pipelined<DC, MTD, NL, false, 1>(lane_addr + buf * NCOLS + col0, 0, sc1, total, release);
          } else {
            if (small) fold_region<DC, MTD, NL, true>(lane_addr + buf * NCOLS + col0, sc, total, true, release);
            else fold_region<DC, MTD, NL, false>(lane_addr + buf * NCOLS + col0, sc, total, true, release);
          }
          DBG_END(1);
          next_acc();
          s = g_end;
        }
      }
      DBG_BEGIN();
      // ---- end of the fragment ----
      if (!first) {
        // a later K range of a tile that another CTA started: leave the partial sums for that CTA
        float* dst = p.partial + ((size_t)blockIdx.x * MT + half * MTD) * BMW + rl;
        if (warp == kDrainWarp0) { DBG_STAMP1(18); }
#pragma unroll
        for (int t = 0; t < MTD; ++t)
          if (t < mcount) __stcg(dst + t * BMW, total[t]);
        if (warp == kDrainWarp0) { DBG_STAMP1(19); }
        // the barrier orders every drain thread's stores before thread 0's release, which is cumulative at GPU scope
        drain_bar();
        if (warp == kDrainWarp0) { DBG_STAMP1(20); }
        if (dt == 0) {
          __threadfence();
          st_release_gpu(p.flags + blockIdx.x, 1u);
        }
        if (warp == kDrainWarp0) { DBG_STAMP1(21); }
        DBG_END(2);
        continue;
      }
      if (warp == kDrainWarp0) { DBG_STAMP(14); }
      if (!last) {
        // add the partial sums of the CTAs that continue the tile, in CTA order
        for (int j = dt; j < np; j += kDT) {
          const uint32_t* f = p.flags + blockIdx.x + 1 + j;
          const long long t0 = clock64();
          uint32_t spins = 0;
          while (ld_acquire_gpu(f) == 0u) {
            if ((++spins & 0xff) == 0 && (*abort_flag || clock64() - t0 > ptx::kWaitLimitCycles)) {
              *abort_flag = kErrPartialWait;
              if (p.err_word) atomicCAS(p.err_word, 0u, kErrPartialWait | (blockIdx.x << 8));
              break;
            }
          }
        }
        drain_bar();
        if (warp == kDrainWarp0) { DBG_STAMP(15); }
        add_partials();
        if (warp == kDrainWarp0) { DBG_STAMP(16); }
      }
      drain_bar();  // the factors written at the top of the fragment are visible
      float pwv[MTD];
#pragma unroll
      for (int t = 0; t < MTD; ++t) pwv[t] = pw_s[half * MTD + t];
      if (!p.gate_up) {
#pragma unroll
        for (int t = 0; t < MTD; ++t)
          if (t < mcount && n_ok)
            store_from_f32(p.out, (int64_t)(p.m0 + mt0 + t) * p.ld + n, p.out_dt, total[t] * ps * pwv[t]);
      } else {
        // rows come in groups of 16: eight gate rows, then the eight up rows of the same outputs
#pragma unroll
        for (int t = 0; t < MTD; ++t) {
          const float v = t < mcount ? total[t] * ps * pwv[t] : 0.f;
          const float u = __shfl_down_sync(0xffffffffu, v, 8);
          if (t < mcount && n_ok && (rl & 8) == 0)
            store_from_f32(p.out, (int64_t)(p.m0 + mt0 + t) * (p.ld >> 1) + gate_up_column(n), p.out_dt, silu_mul(v, u));
        }
      }
      DBG_END(2);
    }
    if (warp == kDrainWarp0) { DBG_STAMP(6); }
    if (warp == kDrainWarp0) { DBG_FLUSH(24); }
  } else if (WBITS == 4 && warp >= kConvWarp0 && warp < kConvWarp0 + 4 * C::kGroups) {
    // ---------------- int4: nibble -> high half of a byte (value * 16 as int8); lane = row ----------------
    // Two groups of four warps; group g expands the slots g, g+2, ... of the CTA's sequence (ring depths are even,
    // so a ring slot always belongs to the same group).
    const int grp = (warp - kConvWarp0) >> 2, cw = (warp - kConvWarp0) & 3;
    const int r = cw * 32 + lane;
    const uint32_t sw = (uint32_t)(r & 7);
    const uint32_t raw_row = ptx::smem_u32(raw_base) + r * 128;
    const uint32_t a_row = ptx::smem_u32(slot_base) + r * 128;
    FragIter it(p);
    DBG_DECL;
    int tile, u0, u1;
    uint32_t i = 0;  // position in the CTA's slot sequence
    while (it.next(tile, u0, u1)) {
      const int s0 = u0 * p.spu, s1 = min(p.slots, u1 * p.spu);
      for (int s = s0; s < s1; ++s, ++i) {
        if (C::kGroups == 2 && (int)(i & 1) != grp) continue;
        const uint32_t sr = i % kRaw, pr = (i / kRaw) & 1, sa = i % kSlots, pa = (i / kSlots) & 1;
        DBG_BEGIN();
        ptx::mbar_wait_warp<32>(&raw_full[sr], pr, abort_flag, p.err_word, ptx::kErrWaitRaw);
        DBG_END(0);
        uint4 v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = lds128(raw_row + sr * kRawBytes + (((uint32_t)c ^ sw) << 4));
        DBG_BEGIN();
        ptx::mbar_wait_warp<32>(&empty[sa], pa ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
        DBG_END(1);
        if constexpr (C::kATmem) {
          ptx::tcgen05_fence_after();  // the MMAs that read this TMEM slot last have completed (their commit freed it)
          const uint32_t t_row = tmem_base + ((uint32_t)(cw * 32) << 16) + C::kATmemCol0 + sa * C::kATmemSlotCols;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 q = v[c];
            const uint32_t w8[8] = {(q.x << 4) & 0xF0F0F0F0u, (q.y << 4) & 0xF0F0F0F0u, (q.z << 4) & 0xF0F0F0F0u,
                                    (q.w << 4) & 0xF0F0F0F0u, q.x & 0xF0F0F0F0u,        q.y & 0xF0F0F0F0u,
                                    q.z & 0xF0F0F0F0u,        q.w & 0xF0F0F0F0u};
            ptx::tmem_st_32x32b_x8(t_row + 8 * c, w8);
          }
          ptx::tmem_st_wait();
          ptx::tcgen05_fence_before();
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t dst = a_row + sa * kSlot + (c >> 2) * kATile;
            const int cc = c & 3;
            const uint4 q = v[c];
            sts128(dst + (((uint32_t)(2 * cc) ^ sw) << 4), (q.x << 4) & 0xF0F0F0F0u, (q.y << 4) & 0xF0F0F0F0u,
                   (q.z << 4) & 0xF0F0F0F0u, (q.w << 4) & 0xF0F0F0F0u);
            sts128(dst + (((uint32_t)(2 * cc + 1) ^ sw) << 4), q.x & 0xF0F0F0F0u, q.y & 0xF0F0F0F0u, q.z & 0xF0F0F0F0u,
                   q.w & 0xF0F0F0F0u);
          }
          ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to the MMA's async proxy
        }
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(&full[sa]);
          ptx::mbar_arrive(&raw_empty[sr]);
        }
      }
    }
    if (warp == kConvWarp0) { DBG_FLUSH(32); }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
#ifdef QMM_LIMB_DBG
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    g_limb_dbg[40] = clock64() - dbg_k0;
    g_limb_dbg[41] = (long long)(ptx::globaltimer_ns() - dbg_g0);
    DBG_STAMP(7);
  }
  if (threadIdx.x == 0 && blockIdx.x < 512) {
    g_limb_cta[4 * blockIdx.x + 3] = (long long)ptx::globaltimer_ns();
  }
#endif
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Scratch {
  int8_t* limbs;
  float* pw;
  float* partial;
  uint32_t* flags;
  size_t bytes;
};

// How one launch is laid out: limbs per token, limb columns per tile (the template instance), and whether the K axis
// is split over the CTAs (stream-K, one token tile) or the batch runs as (weight tile, token tile) items.
struct Plan {
  int nl, ncols, tile_tokens;
  bool items;
};

// limb_tc_set_limbs(3) keeps three limbs everywhere (process-wide).
std::atomic<int> g_limb_policy{0};

// Limbs per token.  In narrow tiles the MMA costs the same with three limbs as with two, so the exact form is kept
// there.  Wider batches pay per limb column: when the output is a 16-bit type, two limbs (15 bits below the row's
// largest value, error at most 2^-15 of it per activation, under the output's own rounding) carry 64 tokens per
// 128-column tile instead of 42.  fp32 outputs always get three.
Plan plan_for(int wbits, int64_t M, int out_dt) {
  const bool two_ok = g_limb_policy.load(std::memory_order_relaxed) != 3 && (out_dt == QMM_BF16 || out_dt == QMM_F16);
  Plan pl;
  pl.nl = 3;
  pl.items = false;
  if (M <= 5) pl.ncols = 16;
  else if (M <= 10) pl.ncols = 32;
  else if (M <= 16) pl.ncols = 48;
  else if (M <= 32 && !(wbits == 4 && two_ok)) pl.ncols = 96;
  else {
    // 128 columns: 42 tokens of three limbs or 64 of two; one tile is split over K, more run as items
    pl.ncols = 128;
    pl.nl = two_ok ? 2 : 3;
    pl.items = M > (pl.nl == 2 ? 64 : 42);
  }
  pl.tile_tokens = pl.ncols / pl.nl;
  return pl;
}
// tokens per launch above which a batch is chunked (24 tiles of 42, 16 tiles of 64)
int64_t max_rows(int nl) { return nl == 2 ? 1024 : 1008; }

// Layout of the caller's scratch: [flags: 1 KB][pw][limbs][partial tiles]; the flag words come first so that a
// caller who clears only the head of the buffer clears them.  partial_tokens: tokens of a token tile.
Scratch carve(void* base, int64_t M, int64_t K, int nl, int partial_tokens, int max_ctas) {
  Scratch s;
  uint8_t* b = reinterpret_cast<uint8_t*>(base);
  size_t off = 0;
  s.flags = reinterpret_cast<uint32_t*>(b + off);
  off += align_up((size_t)max_ctas * 4, 1024);
  s.pw = reinterpret_cast<float*>(b + off);
  off += align_up((size_t)M * 4, 256);
  s.limbs = reinterpret_cast<int8_t*>(b + off);
  off += align_up((size_t)nl * M * K, 256);
  s.partial = reinterpret_cast<float*>(b + off);
  off += align_up((size_t)max_ctas * partial_tokens * BMW * 4, 256);
  s.bytes = off;
  return s;
}

template <int WBITS, int NCOLS, int NL = 3>
int launch_cfg(const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int grid, cudaStream_t st) {
  using C = Cfg<WBITS, NCOLS, NL>;
  auto kern = limb_tc_kernel<WBITS, NCOLS, NL>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmem);
    if (e != cudaSuccess) return fail(QMM_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_w, map_x, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_LAUNCH, "limb_tc_kernel launch: %s", cudaGetErrorString(e));
  }
  return check_launch("limb_tc_kernel");
}

template <int WBITS>
int launch_ncols(int ncols, int nl, const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& p, int grid, cudaStream_t st) {
  if (nl == 2) return launch_cfg<WBITS, 128, 2>(map_w, map_x, p, grid, st);
  switch (ncols) {
    case 16: return launch_cfg<WBITS, 16>(map_w, map_x, p, grid, st);
    case 32: return launch_cfg<WBITS, 32>(map_w, map_x, p, grid, st);
    case 48: return launch_cfg<WBITS, 48>(map_w, map_x, p, grid, st);
    case 96: return launch_cfg<WBITS, 96>(map_w, map_x, p, grid, st);
    default: return launch_cfg<WBITS, 128>(map_w, map_x, p, grid, st);
  }
}

template <typename XT>
cudaError_t launch_split(const void* x, int8_t* xl, float* pw, int64_t M, int64_t K, int nl, int perm4, float pw_mul, cudaStream_t st) {
  int threads = (int)std::min<int64_t>(1024, std::max<int64_t>(64, align_up((size_t)(K / 8), 32)));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)M);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (nl == 2) return cudaLaunchKernelEx(&cfg, split_rows_kernel<XT, 2>, reinterpret_cast<const XT*>(x), xl, pw, K, perm4, pw_mul);
  return cudaLaunchKernelEx(&cfg, split_rows_kernel<XT, 3>, reinterpret_cast<const XT*>(x), xl, pw, K, perm4, pw_mul);
}

}  // namespace

namespace {

// int4 batches at least this long are expanded to int8 once when the caller gave room: the pass over the weights is
// paid back sooner per channel (the int8 form then runs with no hand-over inside a tile) than with scale blocks
constexpr int64_t kExpandTokens = 384, kExpandTokensBlockwise = 512;

// Work split of one token tile.  Stream-K (equal shares of the tile x K-slot units) keeps every SM streaming, but a
// tile shared by several CTAs costs a partial-tile exchange through L2 at the end of the kernel, worth a few slots of
// streaming.  When handing out whole tiles costs fewer slots per CTA than that, each CTA gets whole tiles and
// nothing is exchanged.  Every CTA should stream at least two slots, or its fixed cost dominates.
struct Split {
  int grid;
  long long cost;  // slots of streaming per SM, exchange included
};
Split split_one_tile(int wbits, const Plan& pl, long long tiles, long long slots, int spu) {
  const long long ut = ceil_div(slots, spu), units = tiles * ut;
  const int occ = (wbits == 4 && pl.ncols <= 48) ? 2 : 1;  // Cfg::kOcc
  const long long ctas_max = std::min<long long>((long long)occ * sm_count(), kLimbMaxCtas);
  const long long min_units = std::max<long long>(1, 2 / spu);
  Split sp;
  sp.grid = (int)std::min<long long>(ctas_max, std::max<long long>(1, units / min_units));
  const long long sk_slots = ceil_div(units, sp.grid) * spu;                  // slots per CTA, stream-K
  const long long per_sm = occ;                                               // CTAs that share an SM's bandwidth
  const long long dp_rounds = ceil_div(tiles, ctas_max);
  const long long dp_slots = dp_rounds * slots;                               // slots per CTA, whole tiles
  // exchange cost in slots of streaming (measured: ~3 us for tiles of 5 tokens, ~13 us for 64); a partial tile is
  // 128 x tokens floats, so it grows with the tile
  // (a slot of the 128-column int4 instance takes three times as long as one of the narrow ones: fewer per exchange)
  const long long exchange = ((wbits == 4 && pl.ncols == 128) ? 3 : (wbits == 4 ? 8 : 4)) * (16 + pl.tile_tokens) / 16;
  // compare per-SM streaming: with whole tiles only ceil(tiles / rounds) CTAs run, spread over the SMs
  const long long dp_ctas = ceil_div(tiles, dp_rounds);
  const long long dp_per_sm = ceil_div(dp_ctas, sm_count());
  const bool fills = occ == 1 || dp_ctas * 4 >= ctas_max * 3;  // two CTAs per SM only pay off when both slots are used
  sp.cost = sk_slots * per_sm + exchange;
  if (fills && dp_slots * dp_per_sm <= sp.cost && tiles <= ctas_max * dp_rounds) {
    sp.cost = dp_slots * dp_per_sm;
    sp.grid = (int)std::min<long long>(tiles, ctas_max);
    // with several rounds the units must still split at tile boundaries: a grid that divides the tile count
    while (tiles % sp.grid != 0) --sp.grid;
  }
  return sp;
}

// One launch of the main kernel over `rows` weight rows at `w` (row pitch K * wbits / 8 bytes).
int launch_main(int wbits, const void* w, int64_t rows, int64_t K, const Plan& pl, Params p, const CUtensorMap& map_x, cudaStream_t st) {
  const int ncols = pl.ncols;
  p.N = rows;
  p.tiles = (int)ceil_div(rows, BMW);
  int grid;
  // (one 128-column token tile over more weight tiles than CTAs is scheduled like several: its exchange is too dear
  // to split every tile, and whole tiles alone leave the last round partly filled)
  if (pl.items || (ncols == 128 && p.tiles > sm_count())) {
    // the CTAs walk the (weight tile, token tile) items, whole items each: nothing is exchanged between them
    const int occ = (wbits == 4 && ncols <= 48) ? 2 : 1;  // Cfg::kOcc
    const long long items = (long long)p.tiles * p.ytiles, ctas = (long long)occ * sm_count();
    grid = (int)std::min<long long>(ctas, items);
    p.items1 = items;
    p.units = 0;
    p.g2 = 0;
    // A partly filled last round (448 items on 148 SMs are four rounds for three rounds' work): the items of that
    // round are split along K over a few CTAs each instead, and summed through the partial tiles like a stream-K
    // tile.  Splitting an item over s CTAs costs item/s plus an exchange that grows with s (one partial tile per
    // CTA, read by the item's first CTA); times in microseconds, per-slot figures measured.
    const long long left = items % ctas;
    if (items > ctas && left != 0) {
      const double item_us = (double)p.slots * (wbits == 4 ? 1.1 : (p.mode == kPerChannel ? 0.55 : 0.9));
      const double per_partial_us = 0.7 * pl.tile_tokens / 64.0;
      double s = std::sqrt(item_us / per_partial_us);  // CTAs per item; need not be whole: the units are dealt evenly
      s = std::min(s, std::min((double)ctas / (double)left, (double)p.ut));
      if (s >= 1.5 && item_us / s + 3.0 + per_partial_us * s < 0.75 * item_us) {
        p.items1 = items - left;
        p.units = left * p.ut;
        p.g2 = (int)std::min<long long>(ctas, (long long)((double)left * s));
      }
    }
  } else {
    const Split sp = split_one_tile(wbits, pl, p.tiles, p.slots, p.spu);
    grid = sp.grid;
    p.items1 = 0;
    p.units = (long long)p.tiles * p.ut;
    p.g2 = grid;
  }
  CUtensorMap map_w;
  const int rc = encode_tmap_2d(&map_w, w, 1, false, (uint64_t)rows, (uint64_t)(K * wbits / 8), BMW, 128);
  if (rc != QMM_OK) return rc;
  return wbits == 4 ? launch_ncols<4>(ncols, pl.nl, map_w, map_x, p, grid, st) : launch_ncols<8>(ncols, pl.nl, map_w, map_x, p, grid, st);
}

}  // namespace

void limb_tc_set_limbs(int limbs) { g_limb_policy.store(limbs == 3 ? 3 : 0, std::memory_order_relaxed); }

size_t limb_tc_workspace_bytes(int64_t M, int64_t K) {
  if (M < 1 || K < 1) return 0;
  // Enough for either limb form (the output type is not known here) and for every batch up to M: the limbs of the
  // longest chunk, and the partial tiles of the widest stream-K batch that is not longer than M.
  return carve(nullptr, std::min(M, max_rows(3)), K, 3, (int)std::min<int64_t>(M, 64), kLimbMaxCtas).bytes;
}

bool limb_tc_shape_ok(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, int x_dt, bool has_zp) {
  if (has_zp) return false;
  if (x_dt != QMM_BF16 && x_dt != QMM_F16 && x_dt != QMM_F32) return false;
  if (M < 1 || N < 1 || K < 128) return false;
  if (wbits == 8 ? (K % 16 != 0) : (K % 32 != 0)) return false;  // TMA row pitches of the weights and the limbs
  // scale blocks of 128 (two per slot) or of whole 256-value slots
  if (block_size > 0 && ((block_size != kTileK && block_size % kSlotK != 0) || K % block_size != 0)) return false;
  // one int32 accumulation runs over a scale block (all of K per-channel): |limb * weight| <= 2^14 per term
  if ((block_size > 0 ? block_size : K) > (1 << 16)) return false;
  if (N > (1LL << 30) || K > (1LL << 24)) return false;
  return true;
}

bool limb_tc_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x, int x_dt, const void* w,
                       bool has_zp) {
  if (!limb_tc_shape_ok(wbits, M, N, K, block_size, x_dt, has_zp)) return false;
  if (!aligned(x, 16) || !aligned(w, 16)) return false;
  return device_is_sm100();
}

bool limb_tc_preferred(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size) {
  // Where the measured table has no entry: this kernel's fixed cost (two launches, the stream-K exchange) is paid
  // back by its streaming rate once the weight is large enough, sooner the larger the batch (thresholds read off
  // the tuner's measurements over the reference's shape families); above 64 tokens it beats the conversion-based
  // tensor-core kernel on every shape measured.
  (void)block_size;
  const int64_t mib = N * K * wbits / 8 >> 20;
  if (M > 64) return N * K >= (1 << 20);
  if (M > 32) return mib >= 24;
  if (M > 8) return mib >= 32;
  return mib >= 48;
}

namespace {

cudaError_t launch_expand(const void* src, void* dst, int64_t rows, int64_t K, cudaStream_t st) {
  const int64_t chunks = rows * K / 16;  // 8 packed bytes each
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)std::min<int64_t>(ceil_div(chunks, 256 * 4), 8LL * sm_count()));
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, expand_int4_kernel, reinterpret_cast<const uint2*>(src), reinterpret_cast<uint4*>(dst), chunks);
}

// pw_mul: factor folded into the per-token power of two (1/16 when the weight bytes hold value * 16); w_dep: the
// weights are written by a kernel earlier in the stream that the weight producer has to wait for.
int launch_limb_impl(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt, int64_t M,
                     int64_t N, int64_t K, int64_t block_size, int gate_up, void* workspace, size_t workspace_bytes,
                     float pw_mul, int w_dep, cudaStream_t st) {
  if (!limb_tc_supported(wbits, M, N, K, block_size, x, x_dt, w, false))
    return fail(QMM_ERR_UNSUPPORTED,
                "split-activation tensor-core kernel: needs an sm_100 device, K >= 128 and a multiple of %d, "
                "block_size 128 or a multiple of 256, 16-byte aligned x/w, no zero point (M=%lld N=%lld K=%lld bs=%lld)",
                wbits == 8 ? 16 : 32, (long long)M, (long long)N, (long long)K, (long long)block_size);
  if (gate_up && N % 16 != 0)
    return fail(QMM_ERR_BAD_SHAPE, "fused gate/up epilogue: the interleaved weight needs a multiple of 16 rows, got %lld", (long long)N);
  const Plan pl = plan_for(wbits, M, out_dt);
  const int nl = pl.nl;
  const size_t need = carve(nullptr, std::min(M, max_rows(nl)), K, nl, pl.tile_tokens, kLimbMaxCtas).bytes;
  if (!workspace || workspace_bytes < need)
    return fail(QMM_ERR_WORKSPACE, "split-activation tensor-core kernel needs %zu bytes of workspace, got %zu", need, workspace_bytes);
  if (!aligned(workspace, 256)) return fail(QMM_ERR_MISALIGNED, "workspace must be 256-byte aligned");
  // int4 and a long batch: with room in the workspace behind the regular scratch, the weights are expanded to int8
  // once and the int8 form of the kernel runs on them (all of them if they fit, else slice by slice, see below)
  const bool widen = wbits == 4 && M >= (block_size > 0 ? kExpandTokensBlockwise : kExpandTokens) && !gate_up;
  const size_t wide_off = align_up(need, 256);
  if (widen && workspace_bytes >= wide_off + (size_t)N * (size_t)K) {
    uint8_t* wide = reinterpret_cast<uint8_t*>(workspace) + wide_off;
    cudaError_t e = launch_expand(w, wide, N, K, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(QMM_ERR_LAUNCH, "expand_int4_kernel launch: %s", cudaGetErrorString(e));
    }
    return launch_limb_impl(8, x, x_dt, wide, scale, out, out_dt, M, N, K, block_size, 0, workspace, wide_off, 0.0625f, 1, st);
  }
  if (M > max_rows(nl)) {
    // long batches run in chunks of whole token tiles that share the scratch (same stream: ordered)
    const int64_t rows = max_rows(nl);
    if (gate_up) return fail(QMM_ERR_UNSUPPORTED, "fused gate/up epilogue: at most %lld tokens per call", (long long)rows);
    const size_t xb = dtype_size(x_dt), ob = dtype_size(out_dt);
    for (int64_t m0 = 0; m0 < M; m0 += rows) {
      const int64_t mc = std::min(rows, M - m0);
      const int rc = launch_limb_impl(wbits, reinterpret_cast<const uint8_t*>(x) + (size_t)m0 * K * xb, x_dt, w, scale,
                                      reinterpret_cast<uint8_t*>(out) + (size_t)m0 * N * ob, out_dt, mc, N, K, block_size, 0, workspace,
                                      workspace_bytes, pw_mul, w_dep, st);
      if (rc != QMM_OK) return rc;
    }
    return QMM_OK;
  }
  const Scratch sc = carve(workspace, M, K, nl, pl.tile_tokens, kLimbMaxCtas);

  // slices of weight rows that fit behind the scratch, expanded and multiplied one after the other
  int64_t slice_rows = 0;
  uint8_t* wide = nullptr;
  if (widen && workspace_bytes > wide_off) {
    wide = reinterpret_cast<uint8_t*>(workspace) + wide_off;
    const size_t room = workspace_bytes - wide_off;
    const int64_t fit = (int64_t)(room / (size_t)K) / BMW * BMW;  // whole weight tiles
    // a slice must still give every SM a few items, or the GEMM's last wave eats the gain
    const int64_t ytiles = ceil_div(M, pl.tile_tokens);
    const int64_t min_rows = std::min<int64_t>(align_up((size_t)N, BMW), ceil_div(3 * (int64_t)sm_count(), ytiles) * BMW);
    if (fit >= min_rows) {
      const int64_t n_slices = ceil_div(N, fit);
      slice_rows = align_up((size_t)ceil_div(N, n_slices), BMW);
    }
  }

  {
    // the limbs are made by a kernel of their own (one CTA per token) and reach the main kernel as TMA tiles; the two
    // are chained with programmatic dependent launch, so the main kernel's set-up and first weight loads run under it
    const int perm4 = wbits == 4 && slice_rows == 0;  // the expanded weights are in natural k order
    cudaError_t e;
    if (x_dt == QMM_F32) e = launch_split<float>(x, sc.limbs, sc.pw, M, K, nl, perm4, pw_mul, st);
    else if (x_dt == QMM_BF16) e = launch_split<__nv_bfloat16>(x, sc.limbs, sc.pw, M, K, nl, perm4, pw_mul, st);
    else e = launch_split<__half>(x, sc.limbs, sc.pw, M, K, nl, perm4, pw_mul, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(QMM_ERR_LAUNCH, "split_rows_kernel launch: %s", cudaGetErrorString(e));
    }
  }
  CUtensorMap map_x;
  int rc = encode_tmap_2d(&map_x, sc.limbs, 1, false, (uint64_t)(nl * M), (uint64_t)K, (uint32_t)pl.ncols, 128);
  if (rc != QMM_OK) return rc;

  Params p;
  p.pw = sc.pw;
  p.out_dt = out_dt;
  p.M = (int)M;
  p.ld = N;
  p.slots = (int)ceil_div(K, kSlotK);
  p.mode = block_size <= 0 ? kPerChannel : (block_size == kTileK ? kBlock128 : kBlockSlots);
  p.S = block_size > 0 ? (int)(K / block_size) : 1;
  p.spu = p.mode == kBlockSlots ? (int)(block_size / kSlotK) : 1;
  p.ut = (int)ceil_div(p.slots, p.spu);
  p.partial = sc.partial;
  p.flags = sc.flags;
  p.err_word = device_error_word();
  p.gate_up = gate_up;
  p.ytiles = pl.items ? (int)ceil_div(M, pl.tile_tokens) : 1;
  p.m0 = 0;
  if (slice_rows == 0) {
    p.scale = scale;
    p.out = out;
    p.w_dep = w_dep;
    return launch_main(wbits, w, N, K, pl, p, map_x, st);
  }
  const size_t ob = dtype_size(out_dt);
  for (int64_t n0 = 0; n0 < N; n0 += slice_rows) {
    const int64_t rows = std::min(slice_rows, N - n0);
    cudaError_t e = launch_expand(reinterpret_cast<const uint8_t*>(w) + (size_t)n0 * (size_t)(K / 2), wide, rows, K, st);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(QMM_ERR_LAUNCH, "expand_int4_kernel launch: %s", cudaGetErrorString(e));
    }
    p.scale = scale + n0;
    p.out = reinterpret_cast<uint8_t*>(out) + (size_t)n0 * ob;
    p.w_dep = 1;
    rc = launch_main(8, wide, rows, K, pl, p, map_x, st);
    if (rc != QMM_OK) return rc;
  }
  return QMM_OK;
}

}  // namespace

int launch_limb_tc(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt, int64_t M,
                   int64_t N, int64_t K, int64_t block_size, int gate_up, void* workspace, size_t workspace_bytes,
                   cudaStream_t st) {
  return launch_limb_impl(wbits, x, x_dt, w, scale, out, out_dt, M, N, K, block_size, gate_up, workspace, workspace_bytes,
                          wbits == 4 ? 0.0625f : 1.f, 0, st);
}

size_t limb_tc_wide_bytes(int wbits, int64_t M, int64_t N, int64_t K) {
  return (wbits == 4 && M >= kExpandTokens) ? 256 + (size_t)N * (size_t)K : 0;
}

}  // namespace qmm

#ifdef QMM_LIMB_DBG
extern "C" __attribute__((visibility("default"))) void qmm_debug_limb_dump() {
  cudaDeviceSynchronize();
  long long h[64];
  cudaMemcpyFromSymbol(h, qmm::g_limb_dbg, sizeof(h));
  const char* names[5] = {"wprod", "bprod", "mma", "drain", "conv"};
  for (int r = 0; r < 5; ++r)
    fprintf(stderr, "[dbg] %-6s w0=%lld w1=%lld w2=%lld w3=%lld total=%lld\n", names[r], h[8 * r], h[8 * r + 1], h[8 * r + 2],
            h[8 * r + 3], h[8 * r + 4]);
  fprintf(stderr, "[dbg] timeline (us after entry): setup %.2f | prev-kernel-done(B) %.2f | first slot full %.2f | MMAs issued %.2f | drain start %.2f | drain end %.2f | exit %.2f || split: entry %.2f wait-done %.2f end %.2f\n",
          (h[43] - h[42]) * 1e-3, (h[44] - h[42]) * 1e-3, (h[45] - h[42]) * 1e-3, (h[46] - h[42]) * 1e-3, (h[47] - h[42]) * 1e-3,
          (h[48] - h[42]) * 1e-3, (h[49] - h[42]) * 1e-3, (h[52] - h[42]) * 1e-3, (h[53] - h[42]) * 1e-3, (h[54] - h[42]) * 1e-3);
  {
    static long long c[4 * 512];
    cudaMemcpyFromSymbol(c, qmm::g_limb_cta, sizeof(c));
    long long t0 = 0;
    int n = 0;
    for (int i = 0; i < 512; ++i)
      if (c[4 * i + 3] > 0) { ++n; if (t0 == 0 || c[4 * i] < t0) t0 = c[4 * i]; }
    fprintf(stderr, "[dbg] per-CTA (us after the first entry): cta entry first-full mma-issued exit\n");
    for (int i = 0; i < n; i += (n > 40 ? n / 20 : 1))
      fprintf(stderr, "[dbg]   %3d %7.2f %7.2f %7.2f %7.2f\n", i, (c[4 * i] - t0) * 1e-3, (c[4 * i + 1] - t0) * 1e-3, (c[4 * i + 2] - t0) * 1e-3,
              (c[4 * i + 3] - t0) * 1e-3);
    double mx = 0, mxe = 0;
    for (int i = 0; i < n; ++i) { mx = std::max(mx, (c[4 * i + 3] - t0) * 1e-3); mxe = std::max(mxe, (c[4 * i] - t0) * 1e-3); }
    fprintf(stderr, "[dbg]   %d CTAs, last entry %.2f, last exit %.2f\n", n, mxe, mx);
  }
  fprintf(stderr, "[dbg] exchange (us after CTA 0's entry): owner CTA 0: K loop folded %.2f | flags seen %.2f | partials added %.2f | stored %.2f || CTA 1: partial ready %.2f | stored %.2f | fenced %.2f | flag set %.2f\n",
          (h[56] - h[42]) * 1e-3, (h[57] - h[42]) * 1e-3, (h[58] - h[42]) * 1e-3, (h[48] - h[42]) * 1e-3, (h[60] - h[42]) * 1e-3,
          (h[61] - h[42]) * 1e-3, (h[62] - h[42]) * 1e-3, (h[63] - h[42]) * 1e-3);
  fprintf(stderr, "[dbg] kernel  cycles=%lld ns=%lld -> %.3f GHz\n", h[40], h[41], h[41] ? (double)h[40] / (double)h[41] : 0.0);
}
#endif
