// W8A8 prefill contraction on the 5th-generation tensor cores:
//   acc[m,n] = sum_k xq[m,k] * w[n,k]   (int8 x int8 -> int32, exact)
//   out[m,n] = ((float)acc * w_scale[n] - (float)rowsum[m] * zp[n]) * x_scale[m]
//
// Replaces the reference's dot_general(int8,int8 -> int32) and its scale multiplications
// (torch_xla/experimental/xla_quantized_matmul.py:107-114,:134-135; Pallas tile body
// torch_xla/experimental/pallas_kernels/quantized_matmul_kernel.py:101-121).
//
// Structure (one persistent CTA per SM, 6 warps):
//   warp 0      TMA producer: xq tile [128 x 128B] and w tile [256 x 128B] per stage, 128B swizzle
//   warp 1      MMA issuer:   4 x tcgen05.mma.kind::i8 (M128 N256 K32) per stage into TMEM
//   warps 2..5  epilogue:     tcgen05.ld the int32 accumulator, dequantise in fp32, store
// Two TMEM accumulators (2 x 256 columns) let the epilogue of one tile overlap the main loop of
// the next.  Both operands are K-major, so no transposition happens anywhere.
#include "common.cuh"
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace qmm {

namespace {

constexpr int BM = 128;       // activation rows per tile  (UMMA M)
constexpr int BN = 256;       // weight rows per tile      (UMMA N)
constexpr int BK = 128;       // int8 elements per stage = one 128-byte swizzle row
constexpr int UMMA_K = 32;    // kind::i8
constexpr int kStages = 3;
constexpr int kAccBufs = 2;
constexpr int kThreads = 192;
constexpr uint32_t kStageA = BM * BK;           // 16 KB
constexpr uint32_t kStageB = BN * BK;           // 32 KB
constexpr uint32_t kStageBytes = kStageA + kStageB;
constexpr uint32_t kTmemCols = kAccBufs * BN;   // 512
constexpr uint32_t kOutBoxCols = 64;                      // 16-bit outputs: 64 columns = one 128-byte swizzle row
constexpr uint32_t kOutBoxBytes = BM * 128;               // 16 KB per [128 x 64] box
constexpr uint32_t kOutStaging = (BN / kOutBoxCols) * kOutBoxBytes;  // 64 KB: the whole 128 x 256 tile
constexpr uint32_t kScaleBytes = 2 * BN * 4;              // w_scale and zero point of the tile's columns
constexpr size_t kSmemBytes = 1024 /*align slack*/ + (size_t)kStages * kStageBytes + kOutStaging + kScaleBytes + 256;

struct Params {
  const float* w_scale;
  const float* zp;
  const float* x_scale;
  const int32_t* rowsum;
  int32_t* acc_out;
  void* out;
  int out_dt;
  int64_t M, N, K;
  int tiles_m, tiles_n, k_blocks;
  int tma_store;  // 16-bit output staged in shared memory and written with TMA
  int out_vec;    // `out` rows may be written with 16-byte stores (base and row pitch 16-byte aligned)
  int acc_vec;    // the same for `acc_out`
  uint32_t* err_word;
};

template <typename OT>
__device__ __forceinline__ void store_row_chunk(OT* dst, const float* v, int ncols, bool vec_ok) {
  constexpr int PER16 = 16 / sizeof(OT);
  if (vec_ok && ncols == 32) {
#pragma unroll
    for (int i = 0; i < 32 / PER16; ++i) {
      OT tmp[PER16];
#pragma unroll
      for (int j = 0; j < PER16; ++j) tmp[j] = from_f32<OT>(v[i * PER16 + j]);
      reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(tmp);
    }
  } else {
    for (int j = 0; j < ncols; ++j) dst[j] = from_f32<OT>(v[j]);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
    w8a8_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_out, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + (size_t)kStages * kStageBytes;               // [4 boxes][128 rows][128 B], swizzled
  float* s_ws = reinterpret_cast<float*>(staging + kOutStaging);         // [BN] weight scales of the tile
  float* s_zp = s_ws + BN;                                               // [BN] zero points (or 0)
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kOutStaging + kScaleBytes);
  uint64_t* full = bars;                       // [kStages]
  uint64_t* empty = bars + kStages;            // [kStages]
  uint64_t* tmem_full = bars + 2 * kStages;    // [kAccBufs]
  uint64_t* tmem_empty = tmem_full + kAccBufs; // [kAccBufs]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + kAccBufs);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < kAccBufs; ++a) {
      ptx::mbar_init(&tmem_full[a], 1);
      ptx::mbar_init(&tmem_empty[a], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&map_x);
    ptx::prefetch_tensormap(&map_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: everything above (barriers, TMEM allocation, descriptor prefetch) may run
  // while the kernel that produces the quantized activations drains; its results are only touched below.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          ptx::mbar_wait(&empty[s], ph ^ 1, abort_flag, p.err_word, ptx::kErrWaitEmpty);
          uint8_t* a_dst = stage_base + (size_t)s * kStageBytes;
          uint8_t* b_dst = a_dst + kStageA;
          ptx::mbar_expect_tx(&full[s], kStageBytes);
          ptx::tma_load_2d(a_dst, &map_x, &full[s], kb * BK, tm * BM);
          ptx::tma_load_2d(b_dst, &map_w, &full[s], kb * BK, tn * BN);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // All 32 lanes walk the loop and wait together; the MMA and commit instructions are predicated on
    // lane 0, so the warp never diverges around them.
    {
      constexpr uint32_t idesc = ptx::make_idesc(/*s32*/ 2, /*s8*/ 1, /*s8*/ 1, BM, BN);
      const uint32_t leader = lane == 0 ? 1u : 0u;
      const uint32_t desc_hi = (uint32_t)(ptx::make_sw128_kmajor_desc(0) >> 32);
      const uint32_t lo0 = (uint32_t)ptx::make_sw128_kmajor_desc(ptx::smem_u32(stage_base));
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
        const int ab = tcount % kAccBufs;
        const uint32_t aph = (tcount / kAccBufs) & 1;
        ptx::mbar_wait(&tmem_empty[ab], aph ^ 1, abort_flag, p.err_word, ptx::kErrWaitTmemEmpty);
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + ab * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          ptx::mbar_wait(&full[s], ph, abort_flag, p.err_word, ptx::kErrWaitFull);
          const uint32_t a_lo = lo0 + (uint32_t)s * (kStageBytes >> 4);
          const uint32_t b_lo = a_lo + (kStageA >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = ((uint64_t)desc_hi << 32) | (uint64_t)(a_lo + k * (UMMA_K >> 4));
            const uint64_t b_desc = ((uint64_t)desc_hi << 32) | (uint64_t)(b_lo + k * (UMMA_K >> 4));
            ptx::mma_i8_ss_pred(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0 ? 1u : 0u, leader);
          }
          ptx::mma_commit_pred(&empty[s], leader);  // frees the stage once these MMAs have read it
        }
        ptx::mma_commit_pred(&tmem_full[ab], leader);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int ab = tcount % kAccBufs;
      const uint32_t aph = (tcount / kAccBufs) & 1;
      ptx::mbar_wait(&tmem_full[ab], aph, abort_flag, p.err_word, ptx::kErrWaitTmemFull);
      ptx::tcgen05_fence_after();
      const int64_t m = (int64_t)tm * BM + quad * 32 + lane;
      const bool row_ok = m < p.M;
      const float xs = (row_ok && p.out) ? p.x_scale[m] : 0.f;
      const int32_t rs = (row_ok && p.rowsum) ? p.rowsum[m] : 0;
      const uint32_t taddr = tmem_base + ab * BN + ((uint32_t)(quad * 32) << 16);
      if (p.tma_store) {
        // ---- 16-bit output: dequantise into a swizzled shared-memory tile, one TMA store per 64 columns ----
        const int e = threadIdx.x - 64;  // 0..127 among the epilogue threads
        if (e == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staging free again
        asm volatile("bar.sync 1, 128;" ::: "memory");
        for (int j = e; j < BN; j += 128) {
          const int64_t n = (int64_t)tn * BN + j;
          s_ws[j] = n < p.N ? __ldg(p.w_scale + n) : 0.f;
          s_zp[j] = (p.zp && n < p.N) ? __ldg(p.zp + n) : 0.f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int rl = quad * 32 + lane;  // row inside the tile
        const uint32_t row_base = ptx::smem_u32(staging) + rl * 128;
        const uint32_t sw = (uint32_t)(rl & 7);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float v0 = w8a8_dequant((int32_t)r[j], s_ws[c * 32 + j], p.zp ? &s_zp[c * 32 + j] : nullptr, rs, xs);
            const float v1 = w8a8_dequant((int32_t)r[j + 1], s_ws[c * 32 + j + 1], p.zp ? &s_zp[c * 32 + j + 1] : nullptr, rs, xs);
            if (p.out_dt == QMM_BF16) {
              __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
              pk[j >> 1] = *reinterpret_cast<uint32_t*>(&h);
            } else {
              __half2 h = __floats2half2_rn(v0, v1);
              pk[j >> 1] = *reinterpret_cast<uint32_t*>(&h);
            }
          }
          // 32 columns = 64 bytes = four 16-byte pieces of box (c / 2), pieces (c & 1) * 4 .. + 3
          const uint32_t box = row_base + (uint32_t)(c >> 1) * kOutBoxBytes;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t piece = (uint32_t)((c & 1) * 4 + i) ^ sw;
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(box + (piece << 4)), "r"(pk[4 * i]),
                         "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                         : "memory");
          }
        }
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&tmem_empty[ab]);
        ptx::fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (e == 0) {
#pragma unroll
          for (int b = 0; b < BN / (int)kOutBoxCols; ++b) {
            const int32_t c0 = tn * BN + b * (int)kOutBoxCols;
            if (c0 < p.N)
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&map_out),
                           "r"(ptx::smem_u32(staging) + b * kOutBoxBytes), "r"(c0), "r"(tm * BM)
                           : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        __syncwarp();  // the TMEM load is warp-collective: reconverge before issuing it
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
        ptx::tmem_ld_wait();
        const int64_t n0 = (int64_t)tn * BN + c * 32;
        const bool live = row_ok && n0 < p.N;
        const int ncols = live ? (int)((p.N - n0 < 32) ? (p.N - n0) : 32) : 0;
        if (live && p.acc_out) {
          int32_t* dst = p.acc_out + m * p.N + n0;
          if (ncols == 32 && p.acc_vec) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          } else {
            for (int j = 0; j < ncols; ++j) dst[j] = (int32_t)r[j];
          }
        }
        if (live && p.out) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int64_t n = (n0 + j < p.N) ? n0 + j : p.N - 1;
            v[j] = w8a8_dequant((int32_t)r[j], __ldg(p.w_scale + n), p.zp ? p.zp + n : nullptr, rs, xs);
          }
          if (p.out_dt == QMM_F32)
            store_row_chunk<float>(reinterpret_cast<float*>(p.out) + m * p.N + n0, v, ncols, p.out_vec != 0);
          else if (p.out_dt == QMM_BF16)
            store_row_chunk<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(p.out) + m * p.N + n0, v, ncols,
                                           p.out_vec != 0);
          else
            store_row_chunk<__half>(reinterpret_cast<__half*>(p.out) + m * p.N + n0, v, ncols, p.out_vec != 0);
        }
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&tmem_empty[ab]);
    }
    // the staging tile must outlive the last TMA store that reads it
    if (p.tma_store && threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

bool w8a8_tc_supported(int64_t M, int64_t N, int64_t K, const void* xq, const void* w) {
  if (M < 1 || N < 1 || K < 16) return false;
  if (K % 16 != 0) return false;  // TMA: row pitch must be a multiple of 16 bytes
  if (!aligned(xq, 16) || !aligned(w, 16)) return false;
  if (M > 2147483647LL / 2 || N > 2147483647LL / 2 || K > 2147483647LL / 2) return false;
  return device_is_sm100();
}

int launch_w8a8_tc(const int8_t* xq, const int8_t* w, const float* w_scale, const float* zp,
                   const float* x_scale, const int32_t* rowsum, int32_t* acc_out, void* out,
                   int out_dt, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  if (!w8a8_tc_supported(M, N, K, xq, w))
    return fail(QMM_ERR_UNSUPPORTED,
                "w8a8 tcgen05 kernel: needs an sm_100 device, K a multiple of 16 and 16-byte aligned "
                "operands (M=%lld N=%lld K=%lld)",
                (long long)M, (long long)N, (long long)K);
  CUtensorMap map_x, map_w;
  int rc = encode_tmap_2d(&map_x, xq, 1, false, (uint64_t)M, (uint64_t)K, BM, BK);
  if (rc != QMM_OK) return rc;
  rc = encode_tmap_2d(&map_w, w, 1, false, (uint64_t)N, (uint64_t)K, BN, BK);
  if (rc != QMM_OK) return rc;

  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBytes);
    if (e != cudaSuccess) return fail(QMM_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  // 16-bit outputs go through a shared-memory tile and TMA stores (row pitch must be a multiple of 16 B)
  const bool tma_store = out && !acc_out && out_dt != QMM_F32 && (N % 8 == 0) && aligned(out, 16);
  CUtensorMap map_out;
  if (tma_store) {
    rc = encode_tmap_2d(&map_out, out, 2, true, (uint64_t)M, (uint64_t)N, BM, kOutBoxCols);
    if (rc != QMM_OK) return rc;
  } else {
    map_out = map_x;  // unused by the kernel on this path
  }
  Params p;
  p.tma_store = tma_store ? 1 : 0;
  // vector stores only where every row start is 16-byte aligned; anything else takes the scalar path
  p.out_vec = (out && aligned(out, 16) && (N * (int64_t)dtype_size(out_dt)) % 16 == 0) ? 1 : 0;
  p.acc_vec = (acc_out && aligned(acc_out, 16) && N % 4 == 0) ? 1 : 0;
  p.w_scale = w_scale;
  p.zp = zp;
  p.x_scale = x_scale;
  p.rowsum = rowsum;
  p.acc_out = acc_out;
  p.out = out;
  p.out_dt = out_dt;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tiles_m = (int)ceil_div(M, BM);
  p.tiles_n = (int)ceil_div(N, BN);
  p.k_blocks = (int)ceil_div(K, BK);
  p.err_word = device_error_word();
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, w8a8_tc_kernel, map_x, map_w, map_out, p);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(QMM_ERR_LAUNCH, "w8a8_tc_kernel launch: %s", cudaGetErrorString(le));
  }
  return check_launch("w8a8_tc_kernel");
}

}  // namespace qmm
