// Internal launcher declarations shared by the translation units of libqmm_b200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace qmm {

// fp32 dequant of one W8A8 accumulator in the reference's operation order
// (torch_xla/experimental/xla_quantized_matmul.py:159, 172-182): every product is rounded
// separately, so the result matches the reference's fp32 output bit for bit.
__device__ __forceinline__ float w8a8_dequant(int32_t acc, float w_scale, const float* zp_n,
                                              int32_t rowsum, float x_scale) {
  float v = __fmul_rn(__int2float_rn(acc), w_scale);
  if (zp_n) v = __fsub_rn(v, __fmul_rn(__int2float_rn(rowsum), *zp_n));
  return __fmul_rn(v, x_scale);
}

// ---- generic.cu ---------------------------------------------------------------------------
int launch_generic_nk(bool packed, const void* x, int x_dt, const void* w, const float* scale,
                      const float* zp, void* out, int out_dt, int64_t M, int64_t N, int64_t K,
                      int64_t block_size, cudaStream_t st);
int launch_generic_sbn(const void* x, int x_dt, const int8_t* w, const float* scale, const float* zp,
                       void* out, int out_dt, int64_t M, int64_t N, int64_t K, int64_t block_size,
                       cudaStream_t st);
int launch_generic_w8a8(const int8_t* xq, const int8_t* w, const float* w_scale, const float* zp,
                        const float* x_scale, const int32_t* rowsum, int32_t* acc_out, void* out,
                        int out_dt, int64_t M, int64_t N, int64_t K, cudaStream_t st);

int launch_stream_read(const void* p, size_t bytes, void* sink, cudaStream_t st);

// ---- gemv.cu ------------------------------------------------------------------------------
// Decode kernels for weights stored [N,K] (int8) or [N,K/2] (packed int4).  block_size == 0
// means per-channel scales.  Returns QMM_ERR_UNSUPPORTED / QMM_ERR_MISALIGNED when the shape
// does not fit (M > 8, row pitch not a multiple of 16 bytes, ...).
bool gemv_nk_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x,
                       int x_dt, const void* w);
int launch_gemv_nk(int wbits, const void* x, int x_dt, const void* w, const float* scale,
                   const float* zp, void* out, int out_dt, int64_t M, int64_t N, int64_t K,
                   int64_t block_size, cudaStream_t st);
// ---- decode_mma.cu ------------------------------------------------------------------------
// Decode kernel: weights dequantised in registers and fed to warp-level MMAs (M <= 32, bf16/f16
// activations, no zero point).  block_size == 0 means per-channel scales.
bool decode_mma_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x, int x_dt,
                          const void* w, bool has_zp);
// gate_up != 0: the weight rows are interleaved gate/up groups of eight and the kernel writes
// silu(gate) * up as [M, N/2].
int launch_decode_mma(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt,
                      int64_t M, int64_t N, int64_t K, int64_t block_size, cudaStream_t st, int gate_up = 0);

// The same kernel for the K-sharded (row-parallel) linear with the sum over ranks fused into its epilogue:
// peer_bufs[r] is rank r's exchange buffer (entry `rank` this GPU's own, the others peer mappings), each laid
// out as two fp32 data slots of slot_floats elements, world * ceil(N/16) flag words, a call counter and a ticket.
int launch_decode_mma_allreduce(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt,
                                int64_t M, int64_t N, int64_t K, int64_t block_size, void* const* peer_bufs, int rank,
                                int world, int64_t slot_floats, cudaStream_t st);

// ---- limb_gemm.cu (tcgen05 kind::i8 on unconverted weights; activations split into int8 limbs) ----------
// Weight-only linear for 1 <= M <= 64 (bf16/f16/f32 activations, no zero point): stream-K over all SMs, needs
// limb_tc_workspace_bytes(M, K) bytes of caller scratch whose first 1024 bytes are zero before the first use (the
// kernel leaves them zero).  gate_up as in launch_decode_mma.
constexpr int kLimbMaxCtas = 320;  // two CTAs per SM on up to 160 SMs
size_t limb_tc_workspace_bytes(int64_t M, int64_t K);
// extra bytes behind the regular scratch that let a long int4 batch expand its weights to int8 once (0: no use for them)
size_t limb_tc_wide_bytes(int wbits, int64_t M, int64_t N, int64_t K);
void limb_tc_set_limbs(int limbs);  // 3: three limbs per token everywhere; anything else: two for 16-bit outputs above 32 tokens
bool limb_tc_shape_ok(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, int x_dt, bool has_zp);
bool limb_tc_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x, int x_dt,
                       const void* w, bool has_zp);
// AUTO's shape rule: true where this kernel is the fastest measured choice.
bool limb_tc_preferred(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size);
int launch_limb_tc(int wbits, const void* x, int x_dt, const void* w, const float* scale, void* out, int out_dt, int64_t M,
                   int64_t N, int64_t K, int64_t block_size, int gate_up, void* workspace, size_t workspace_bytes,
                   cudaStream_t st);

// ---- peer_reduce.cu -----------------------------------------------------------------------
// One-shot all-reduce of fp32 partial results that every rank keeps in peer-mapped memory.
int launch_peer_allreduce(void* const* data_ptrs, void* const* flag_ptrs, int rank, int world, uint32_t epoch, void* out,
                          int out_dt, int64_t count, cudaStream_t st);

// ---- act_quant.cu -------------------------------------------------------------------------
int launch_quantize_activation(const void* x, int x_dt, int8_t* xq, float* x_scale,
                               int32_t* rowsum, int64_t M, int64_t K, int saturate,
                               cudaStream_t st);

// ---- pack.cu ------------------------------------------------------------------------------
int launch_pack_int4_nk(const int8_t* w, uint8_t* wp, int64_t N, int64_t K, cudaStream_t st);
int launch_pack_int4_sbn(const int8_t* w, uint8_t* wp, int64_t S, int64_t bs, int64_t N,
                         cudaStream_t st);
int launch_unpack_int4_nk(const uint8_t* wp, int8_t* w, int64_t N, int64_t K, cudaStream_t st);

// ---- w8a8_gemm.cu (tcgen05 kind::i8) ------------------------------------------------------
bool w8a8_tc_supported(int64_t M, int64_t N, int64_t K, const void* xq, const void* w);
int launch_w8a8_tc(const int8_t* xq, const int8_t* w, const float* w_scale, const float* zp,
                   const float* x_scale, const int32_t* rowsum, int32_t* acc_out, void* out,
                   int out_dt, int64_t M, int64_t N, int64_t K, cudaStream_t st);

// ---- mixed_gemm.cu (tcgen05 kind::f16 after shared-memory dequant) ------------------------
bool mixed_tc_shape_ok(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, int x_dt, bool has_zp);
bool mixed_tc_supported(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, const void* x,
                        int x_dt, const void* w, bool has_zp);
int launch_mixed_tc(int wbits, const void* x, int x_dt, const void* w, const float* scale,
                    void* out, int out_dt, int64_t M, int64_t N, int64_t K, int64_t block_size,
                    cudaStream_t st);

}  // namespace qmm
