/*
 * qmm_b200.h — C ABI of the B200 (sm_100a) weight-quantized linear kernels.
 *
 * The reference (pytorch/xla) has no C ABI for this path: its operator is a PyTorch
 * dispatcher op whose arithmetic runs inside XLA or a TPU Pallas kernel.  The entry points
 * below are what a binding for that operator calls instead; each one names the reference
 * interface it stands in for (paths are inside the pytorch/xla tree).
 *
 * Conventions
 *   - Every pointer is DEVICE memory owned by the caller, except where a parameter is
 *     documented as a host pointer.  Nothing here allocates, frees or synchronises; all work
 *     is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *   - Matrices are dense row-major.  M = number of activation rows (product of x's leading
 *     dims), K = in_features, N = out_features, S = K / block_size.
 *   - Every function returns a qmm_status; 0 is success.  No exception or abort crosses the ABI.
 *     qmm_last_error_string() gives a per-thread description of the last failure.
 *   - There is no CPU fallback: a call that cannot run on the current device fails with a status.
 *   - `variant` picks the kernel family; QMM_VARIANT_AUTO chooses by shape.  A variant that
 *     cannot take the given shape fails with QMM_ERR_UNSUPPORTED rather than running another one.
 */
#ifndef QMM_B200_H_
#define QMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QMM_ABI_VERSION 1

#if defined(__GNUC__)
#define QMM_API __attribute__((visibility("default")))
#else
#define QMM_API
#endif

typedef enum qmm_dtype {
  QMM_F32 = 0,
  QMM_BF16 = 1,
  QMM_F16 = 2,
} qmm_dtype;

typedef enum qmm_status {
  QMM_OK = 0,
  QMM_ERR_BAD_SHAPE = 1,   /* a dimension is negative, zero where it may not be, or inconsistent */
  QMM_ERR_UNSUPPORTED = 2, /* valid request that the chosen variant / this build cannot run */
  QMM_ERR_MISALIGNED = 3,  /* a pointer or row pitch breaks the alignment the variant needs */
  QMM_ERR_LAUNCH = 4,      /* the CUDA runtime rejected a launch or a descriptor */
  QMM_ERR_WORKSPACE = 5,   /* workspace missing or smaller than qmm_workspace_size() says */
  QMM_ERR_NULL = 6,        /* a required pointer is NULL */
  QMM_ERR_DEVICE = 7,      /* current device is not sm_100 or the driver lacks a needed entry */
  QMM_ERR_TIMEOUT = 8,     /* a bounded device-side wait gave up (see qmm_device_error_flag) */
} qmm_status;

typedef enum qmm_variant {
  QMM_VARIANT_AUTO = 0,
  QMM_VARIANT_GENERIC = 1, /* any shape, any alignment; one thread per output element */
  QMM_VARIANT_GEMV = 2,    /* decode: warp-per-row, 128-bit weight loads, M <= 8 */
  QMM_VARIANT_TCGEN05 = 3, /* TMA -> shared memory -> tcgen05.mma with TMEM accumulators */
  QMM_VARIANT_MMA = 4,     /* decode: weights dequantised in registers into warp-level MMAs, M <= 32 */
  /* 5 was a tensor-memory decode variant that lost to QMM_VARIANT_MMA on every shape; the value is not reused */
  QMM_VARIANT_I8TC = 6,    /* activations split into int8 limbs, unconverted weights into tcgen05.mma.kind::i8, stream-K
                              over all SMs, 1 <= M <= 64; only through qmm_weight_only (needs workspace) */
} qmm_variant;

typedef enum qmm_op {
  QMM_OP_W8A16_PERCHANNEL = 0,
  QMM_OP_BLOCKWISE_SBN = 1,
  QMM_OP_W4A16_BLOCKWISE_PACKED = 2,
  QMM_OP_W8A8_PERCHANNEL = 3,
  QMM_OP_W4A16_PERCHANNEL_PACKED = 4,
} qmm_op;

QMM_API int qmm_abi_version(void);
QMM_API const char* qmm_status_string(int status);
QMM_API const char* qmm_last_error_string(void);

/*
 * Per-channel weight-only linear:  out[m,n] = (sum_k x[m,k] * w[n,k]) * scale[n] - (sum_k x[m,k]) * zp[n].
 * Replaces: torch.ops.xla.quantized_matmul with block_size == -1, quantize_activation == False
 *   (torch_xla/experimental/xla_quantized_matmul.py:76-114 XLA key, :139-159 CPU key; the
 *   mixed bf16 x s8 dot it lowers to: torch_xla/csrc/xla_lower_util.cpp:477-481).
 * w: int8 [N,K] (int4 values in an int8 container are the same call); scale: f32 [N];
 * zp: f32 [N] in scaled units, or NULL.  Accumulation is fp32; the scale is applied once, after it.
 */
QMM_API int qmm_w8a16_perchannel(const void* x, int x_dtype, const int8_t* w, const float* scale,
                         const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                         int64_t K, int variant, void* stream);

/*
 * Blockwise weight-only linear on the reference's own weight layout [S, block_size, N] (N minor):
 *   out[m,n] = sum_b scale[b,n] * (sum_c x[m,b*bs+c] * w[b,c,n]) - sum_b (sum_c x[m,b*bs+c]) * zp[b,n].
 * Replaces: torch.ops.xla.quantized_matmul with block_size > 0
 *   (xla_quantized_matmul.py:115-124 and :160-170; layout check :27-53).
 * w: int8 [S,bs,N]; scale, zp: f32 [S,N]; zp may be NULL.
 * Only QMM_VARIANT_AUTO / QMM_VARIANT_GENERIC: this N-minor layout runs on the any-shape kernel (one thread per
 * output).  It is the correctness path; for speed convert the weight once to a K-minor layout (qmm_pack_int4_sbn,
 * or a transposed int8 copy) and call qmm_weight_only - what the operator layer above this ABI does on its own,
 * caching the converted weight per weight tensor.
 */
QMM_API int qmm_blockwise_sbn(const void* x, int x_dtype, const int8_t* w, const float* scale,
                      const float* zp, void* out, int out_dtype, int64_t M, int64_t N, int64_t K,
                      int64_t block_size, int variant, void* stream);

/*
 * Blockwise weight-only linear on int4 weights packed two per byte along K:
 * wp: uint8 [N, K/2], byte j of row n holds k=2j in its low nibble and k=2j+1 in its high
 * nibble, two's complement.  scale, zp: f32 [S,N] as above.  Same formula as qmm_blockwise_sbn.
 * Replaces: the int4 route of the same op, where the reference re-materialises the weight as an
 *   S4 literal on every call (xla_quantized_matmul.py:101-103; torch_xla/csrc/ops/cast_int4.cpp:14-39).
 *   The packed layout itself has no counterpart in the reference (it stores int4 unpacked).
 */
QMM_API int qmm_w4a16_blockwise_packed(const void* x, int x_dtype, const uint8_t* wp, const float* scale,
                               const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                               int64_t K, int64_t block_size, int variant, void* stream);

/*
 * Per-channel weight-only linear on packed int4 weights (wp: uint8 [N,K/2], nibble order as above;
 * scale, zp: f32 [N]).  Same formula as qmm_w8a16_perchannel.
 * Replaces: the int4_weight=True route of the per-channel op (xla_quantized_matmul.py:101-114).
 */
QMM_API int qmm_w4a16_perchannel_packed(const void* x, int x_dtype, const uint8_t* wp, const float* scale,
                                const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                                int64_t K, int variant, void* stream);

/*
 * Blockwise weight-only linear on int8 weights stored K-minor (w: int8 [N,K]; scale, zp: f32 [K/block_size, N]):
 *   out[m,n] = sum_b scale[b,n] * (sum_{k in block b} x[m,k] * w[n,k])  -  sum_b zp[b,n] * sum_{k in block b} x[m,k]
 * The arithmetic of qmm_blockwise_sbn on the layout the decode and tensor-core kernels stream; callers transpose
 * a reference-layout weight [K/bs, bs, N] once (the module does).
 * Replaces: the blockwise einsum pair of the reference (xla_quantized_matmul.py:120-124, :165-170).
 */
QMM_API int qmm_w8a16_blockwise(const void* x, int x_dtype, const int8_t* w, const float* scale, const float* zp,
                        void* out, int out_dtype, int64_t M, int64_t N, int64_t K, int64_t block_size, int variant,
                        void* stream);

/*
 * Any of the four weight-only linears above on K-minor weights, with caller scratch: the one entry point that can
 * run QMM_VARIANT_I8TC, which QMM_VARIANT_AUTO picks where the measured table or its shape rule names it and the
 * workspace suffices (otherwise AUTO chooses as the entry points above do, and the workspace is not touched).
 *   wbits 8: w int8 [N,K];  wbits 4: w uint8 [N,K/2], nibble order as qmm_w4a16_blockwise_packed.
 *   block_size <= 0: per-channel, scale/zp f32 [N];  block_size > 0: scale/zp f32 [K/block_size, N].
 *   workspace: qmm_weight_only_workspace_size(max M, K) bytes of device memory, 256-byte aligned, whose first
 *   1024 bytes are ZERO before the first call (the kernel leaves them zero); calls that share a workspace must be
 *   ordered on the GPU (same stream).  NULL / 0 is allowed and rules the I8TC variant out.  A workspace of
 *   qmm_weight_only_workspace_size_for(wbits, max M, N, K) bytes additionally lets long int4 batches (384 tokens
 *   and more per channel, 512 with scale blocks) expand the weights to int8 once per call (N*K bytes behind the
 *   regular scratch; with less room they are expanded in slices of rows, or per tile inside the kernel as for short
 *   batches): 1.2x faster at 512 tokens per channel (1.05x with scale blocks), 1.1-1.3x at 1024.  Results are bit-identical either way.
 * I8TC computes  sum_k X[m,k] * w[n,k]  exactly in int32, where X is the activation row in 22-bit fixed point
 * relative to the row's largest exponent (exact for bf16/f16 values within 2^-14 of the row maximum, rounded at
 * 2^-22 of it below), then applies scales in fp32: the accuracy of an fp32 accumulation.  (16-bit outputs above 32
 * tokens: 15-bit fixed point, see qmm_set_activation_limbs.)
 * Replaces: torch.ops.xla.quantized_matmul without activation quantization
 *   (torch_xla/experimental/xla_quantized_matmul.py:101-124 XLA key, :152-170 CPU key).
 */
QMM_API size_t qmm_weight_only_workspace_size(int64_t max_M, int64_t K);
QMM_API size_t qmm_weight_only_workspace_size_for(int wbits, int64_t max_M, int64_t N, int64_t K);
/*
 * The kernel family the measured table names for a shape (a QMM_VARIANT_* value), or 0 when the table has no entry
 * and QMM_VARIANT_AUTO falls back to its shape rule.  The table is generated on a B200 by `python -m xla_b200.tune`
 * and compiled in; it is keyed by weight bits, block size (<= 0: per channel), out/in features and the batch
 * bucket M <= 1, 2, 4, 8, 16, 32, 64.
 * Replaces: get_tuned_block_sizes (torch_xla/experimental/pallas_kernels/quantized_matmul_kernel.py:537-555).
 */
QMM_API int qmm_tuned_variant(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size);
/* Name of the kernel family qmm_weight_only's AUTO picks for a shape, given a sufficient workspace (static string). */
QMM_API const char* qmm_weight_only_variant_for(int wbits, int64_t M, int64_t N, int64_t K, int64_t block_size, int has_zp);
QMM_API int qmm_weight_only(int wbits, const void* x, int x_dtype, const void* w, const float* scale, const float* zp,
                    void* out, int out_dtype, int64_t M, int64_t N, int64_t K, int64_t block_size, int variant,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * Fused gate + up projection of a gated MLP for decode batches (1 <= M <= 32, bf16/f16 activations):
 *   out[m, j] = silu(g[m, j]) * u[m, j],   g = x . dequant(Wgate)^T,  u = x . dequant(Wup)^T,  out: [M, N2/2]
 * `w` holds both projections as N2 = 2 * out_features K-minor rows (int8 [N2,K] for wbits == 8, packed int4
 * uint8 [N2,K/2] for wbits == 4) in groups of 16: rows 16i..16i+7 are gate rows 8i..8i+7, rows 16i+8..16i+15
 * the up rows of the same outputs; `scale` (f32 [N2], or [K/block_size, N2] when block_size > 0, else pass 0)
 * follows the same row order.  Both dot products and the activation are computed in fp32 and rounded once.
 * Replaces: nothing in the reference - it issues two quantized_matmul calls and leaves silu(gate) * up to XLA's
 * fusion; the formula per projection is the one of xla_quantized_matmul.py:152-170.
 * Returns QMM_ERR_UNSUPPORTED outside the decode kernels' range (callers then run the two projections as one
 * [N2]-row linear and apply the activation themselves).
 */
QMM_API int qmm_gate_up_decode(int wbits, const void* x, int x_dtype, const void* w, const float* scale, void* out,
                       int out_dtype, int64_t M, int64_t N2, int64_t K, int64_t block_size, void* stream);
/*
 * The same fused operation for any batch up to 1008 tokens on the split-activation kernel (QMM_VARIANT_I8TC), whose
 * drain warps apply silu(gate) * up before the one store: bf16 / f16 / f32 activations, K >= 128 and a multiple of
 * 16 (int8) or 32 (int4), block_size 0, 128 or a multiple of 256.  workspace: as for qmm_weight_only
 * (qmm_weight_only_workspace_size(M, K) bytes, 256-byte aligned, first 1024 bytes zero before the first use).
 * Returns QMM_ERR_UNSUPPORTED outside that range.  No counterpart in the reference (see qmm_gate_up_decode).
 */
QMM_API int qmm_gate_up(int wbits, const void* x, int x_dtype, const void* w, const float* scale, void* out, int out_dtype,
                int64_t M, int64_t N2, int64_t K, int64_t block_size, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Per-token dynamic activation quantizer:
 *   amax = max_k |x[m,k]|; s = amax / 127 (rounded to x's dtype); xq = rint(x / s) (quotient
 *   rounded to x's dtype first) -> int8.
 * Replaces: _quantize_tensor (xla_quantized_matmul.py:56-73) and _quantize_array
 *   (torch_xla/experimental/pallas_kernels/quantized_matmul_kernel.py:10-18).
 * saturate != 0 clamps to [-128,127] (what an XLA device does); saturate == 0 wraps a pre-cast
 * +128 to -128 like the reference's eager CPU conversion.  x_scale: f32 [M] (exact upcast of the
 * scale); xq_rowsum: int32 [M] = sum_k xq[m,k], or NULL.
 */
QMM_API int qmm_quantize_activation(const void* x, int x_dtype, int8_t* xq, float* x_scale,
                            int32_t* xq_rowsum, int64_t M, int64_t K, int saturate, void* stream);

/*
 * W8A8 contraction with int32 accumulation and the fp32 dequant epilogue:
 *   acc[m,n] = sum_k xq[m,k] * w[n,k]                                  (exact, int32)
 *   out[m,n] = ((float)acc * w_scale[n] - (float)xq_rowsum[m] * zp[n]) * x_scale[m]
 * Replaces: _xla_dot_general(int8,int8 -> int32) (torch_xla/csrc/ops/dot_general.cpp:16-37,
 *   xla_quantized_matmul.py:110-111), the CPU twin F.linear(int32,int32) (:153-158), the
 *   scale multiplications (:114,:134-135 / :159,:181-182) and the Pallas tile body
 *   (quantized_matmul_kernel.py:101-121).
 * acc_out (int32 [M,N]) and out may each be NULL, not both.  zp needs xq_rowsum.
 */
QMM_API int qmm_w8a8_gemm(const int8_t* xq, const int8_t* w, const float* w_scale, const float* zp,
                  const float* x_scale, const int32_t* xq_rowsum, int32_t* acc_out, void* out,
                  int out_dtype, int64_t M, int64_t N, int64_t K, int variant, void* stream);

/*
 * The whole quantize_activation=True op: quantizer + contraction + epilogue.
 * Replaces: torch.ops.xla.quantized_matmul(..., quantize_activation=True)
 *   (xla_quantized_matmul.py:107-114,:134-135) and torch.ops.xla.quantized_matmul_int8
 *   (torch_xla/experimental/custom_kernel.py:1066-1106, :1742-1761).
 * workspace: qmm_workspace_size(QMM_OP_W8A8_PERCHANNEL, M, N, K) bytes of device memory, 256-byte
 * aligned, holding the quantized activations between the two kernels.
 */
QMM_API int qmm_w8a8_perchannel(const void* x, int x_dtype, const int8_t* w, const float* w_scale,
                        const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                        int64_t K, int saturate, int variant, void* workspace,
                        size_t workspace_bytes, void* stream);

/*
 * qmm_w8a8_perchannel for callers that cannot hand over device memory of their own: plugins inside
 * a serving process whose framework owns every byte of the GPU, loops that must not hit
 * cudaMalloc's device-wide synchronisation, code bound by a "no allocation after start-up" rule.
 * (No counterpart in the reference: there the XLA runtime owns all temporaries.)
 * The scratch between quantizer and contraction is a fixed array inside the library's device image,
 * QMM_STATIC_SCRATCH_BYTES long, resident on every GPU that loads the library until the process ends.
 *   - Shapes with qmm_workspace_size(QMM_OP_W8A8_PERCHANNEL, M, N, K) > QMM_STATIC_SCRATCH_BYTES are
 *     refused with QMM_ERR_WORKSPACE (M*K up to 8 Mi elements fits, e.g. 2048 x 4096).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call before any stream capture starts.
 *   - All calls share the one array and it keeps the previous call's contents; nothing in it needs
 *     clearing, but two calls whose kernels may overlap on the GPU (other streams, other host
 *     threads) corrupt each other: serialise them.
 * The function itself calls no allocating routine.  Arguments as qmm_w8a8_perchannel.
 */
#define QMM_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u + 64u * 1024u)
QMM_API int qmm_w8a8_perchannel_static(const void* x, int x_dtype, const int8_t* w, const float* w_scale,
                               const float* zp, void* out, int out_dtype, int64_t M, int64_t N,
                               int64_t K, int saturate, int variant, void* stream);

/* Bytes of caller-provided scratch an op needs for the given shape (0 if none). */
QMM_API size_t qmm_workspace_size(int op, int64_t M, int64_t N, int64_t K);

/*
 * int4 packing (device to device).  Values must lie in [-8,7].
 *   qmm_pack_int4_nk : int8 [N,K]      -> uint8 [N,K/2]
 *   qmm_pack_int4_sbn: int8 [S,bs,N]   -> uint8 [N,K/2]   (K = S*bs)
 *   qmm_unpack_int4_nk: uint8 [N,K/2]  -> int8 [N,K]
 * Replaces: _xla_cast_int4 / the CastInt4 IR node (torch_xla/csrc/ops/cast_int4.cpp:14-39), which
 *   narrows an int8 container to 4-bit storage for the device.
 */
QMM_API int qmm_pack_int4_nk(const int8_t* w, uint8_t* wp, int64_t N, int64_t K, void* stream);
QMM_API int qmm_pack_int4_sbn(const int8_t* w, uint8_t* wp, int64_t S, int64_t block_size, int64_t N,
                      void* stream);
QMM_API int qmm_unpack_int4_nk(const uint8_t* wp, int8_t* w, int64_t N, int64_t K, void* stream);

/*
 * Peer-memory buffers and a one-shot all-reduce for the row-parallel (K-sharded) linear on the GPUs of one box.
 * No reference counterpart as code: the reference leaves the all-reduce after a K-sharded matmul to XLA
 * (torch_xla/csrc/cross_replica_reduces.cpp:154; sharding by torch_xla/distributed/spmd/xla_sharding.py:685).
 *
 *   qmm_peer_buffer_create   cudaMalloc's `bytes` on the current device (zero-filled) and returns the pointer
 *                            and a 64-byte CUDA IPC handle for it.  This is the one place the library allocates:
 *                            IPC handles need a whole allocation of their own.
 *   qmm_peer_buffer_open     maps a peer's buffer (its handle, received over any channel) into this process with
 *                            peer access enabled; qmm_peer_buffer_close unmaps it; qmm_peer_buffer_destroy frees
 *                            one's own buffer (after every peer has closed it).
 *   qmm_allreduce_oneshot    out[i] = sum_r data_ptrs[r][i] (fp32 partials, summed in rank order, converted to
 *                            out_dtype), i < count, count % 4 == 0.  data_ptrs / flag_ptrs are HOST arrays of
 *                            `world` device pointers, entry `rank` being this process's own buffers, the others
 *                            peer mappings; flag_ptrs[r] points to 16 zero-initialised uint32 on rank r.  `epoch`
 *                            must increase by one per call, starting at 1, identically on every rank; 0 makes
 *                            the kernel keep the call number itself in flag word 8 (what a launch captured in a
 *                            CUDA graph needs, since its arguments are frozen).  Callers
 *                            alternate between two data regions so that a rank may write call e+1's partial while
 *                            a peer still reads call e's.  Every rank must launch the call (one kernel per GPU,
 *                            the kernels wait for one another through the flags, at most ~1 s: on expiry the
 *                            device error word is set and nothing is reduced).  world <= 8.
 */
QMM_API int qmm_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]);
QMM_API int qmm_peer_buffer_open(const unsigned char handle[64], void** ptr);
QMM_API int qmm_peer_buffer_close(void* ptr);
QMM_API int qmm_peer_buffer_destroy(void* ptr);
QMM_API int qmm_allreduce_oneshot(void* const* data_ptrs, void* const* flag_ptrs, int rank, int world, uint32_t epoch,
                          void* out, int out_dtype, int64_t count, void* stream);

/*
 * Row-parallel (K-sharded) decode linear with the sum over ranks fused into the kernel: every CTA writes its
 * 16 x M partial sums into every rank's exchange buffer (peer stores), flags the tile on every peer, waits (bounded, ~1 s, then the
 * device error word is set) for the same tile of every peer and stores the sum of the `world` partials, added in
 * rank order in fp32 - all ranks end up with bit-identical results and no separate all-reduce runs.
 *   out[m,n] = sum_r sum_b scale_r[b,n] * (sum_{k in block b of rank r's K slice} x_r[m,k] * w_r[n,k])
 * x, w, scale are THIS rank's slices (wbits 4: packed uint8 [N,K/2]; 8: int8 [N,K]; block_size 0 = per-channel
 * scale [N], which every rank applies to its partial).  1 <= M <= 8, bf16/f16 activations.
 * peer_bufs: HOST array of `world` device pointers to exchange buffers of qmm_rowparallel_buffer_bytes(max_M, N,
 * world) bytes each, created zero-filled with qmm_peer_buffer_create on their owners and mapped with
 * qmm_peer_buffer_open elsewhere; slot_floats = max_M * N as passed there.  Every rank must make the same calls in
 * the same order on such a buffer set; a set serves one N.  The call number lives in the buffer, so a launch
 * captured in a CUDA graph stays valid on replay.
 * Replaces: nothing in the reference as code - the K-sharded matmul plus the all-reduce XLA would insert after it
 * (torch_xla/csrc/cross_replica_reduces.cpp:154), per projection the formula of xla_quantized_matmul.py:152-170.
 */
QMM_API size_t qmm_rowparallel_buffer_bytes(int64_t max_M, int64_t N, int world);
QMM_API int qmm_rowparallel_decode(int wbits, const void* x, int x_dtype, const void* w, const float* scale, void* out,
                           int out_dtype, int64_t M, int64_t N, int64_t K, int64_t block_size,
                           void* const* peer_bufs, int rank, int world, int64_t slot_floats, void* stream);

/*
 * Host-buffer front end of the weight-only linears: one call copies the activations in from HOST memory, runs
 * the linear and copies the result out to HOST memory, on three streams of the pipeline's own that overlap the
 * copies of neighbouring calls with the kernel.  The reference has no such call: a user of the reference moves
 * the activation to the XLA device (`x.to(xla_device)`, torch_xla/csrc/tensor_util.cpp), runs
 * torch.ops.xla.quantized_matmul on it (torch_xla/experimental/xla_quantized_matmul.py:79-114, :133-170) and
 * reads the result back (`y.cpu()`); this entry is that round trip as one enqueue.
 *
 *   qmm_host_pipeline_create   allocates, on the current device, `depth` (1..64) staging slots of max_x_bytes +
 *                              max_out_bytes and the streams and events; nothing is allocated afterwards.
 *   qmm_host_weight_only       enqueues one linear.  x_host [M,K] and out_host [M,N] are HOST pointers (page-locked
 *                              for the copies to overlap); w, scale, zp are DEVICE pointers in the layout `layout`
 *                              names, with the meaning they have in the device entry point of that layout.  Returns
 *                              once the work is enqueued; when more than `depth` calls are in flight it first waits
 *                              for the oldest.  out_host is valid after qmm_host_pipeline_sync.
 *   qmm_host_pipeline_wait_stream  makes every linear submitted from now on wait for the work that `stream` holds at
 *                              this moment: call it after preparing weights or scales on another stream (packing,
 *                              an upload) - the pipeline's own streams are not ordered after the caller's otherwise.
 *   qmm_host_pipeline_sync     blocks until every result submitted so far is in its host buffer.
 *   qmm_host_pipeline_destroy  waits for the pipeline's streams and frees everything.
 * A pipeline is used by one host thread at a time, on the device it was created on.  x_host must stay untouched
 * until the call's copy-in has run (at the latest: qmm_host_pipeline_sync).
 */
typedef enum qmm_host_layout {
  QMM_HOST_W4_BLOCKWISE_PACKED = 0,  /* as qmm_w4a16_blockwise_packed */
  QMM_HOST_W4_PERCHANNEL_PACKED = 1, /* as qmm_w4a16_perchannel_packed (block_size ignored) */
  QMM_HOST_W8_PERCHANNEL = 2,        /* as qmm_w8a16_perchannel (block_size ignored) */
  QMM_HOST_W8_BLOCKWISE_KMINOR = 3,  /* as qmm_w8a16_blockwise */
} qmm_host_layout;
QMM_API int qmm_host_pipeline_create(size_t max_x_bytes, size_t max_out_bytes, int depth, void** pipeline);
QMM_API int qmm_host_weight_only(void* pipeline, int layout, const void* x_host, int x_dtype, const void* w,
                                 const float* scale, const float* zp, void* out_host, int out_dtype, int64_t M,
                                 int64_t N, int64_t K, int64_t block_size, int variant);
QMM_API int qmm_host_pipeline_wait_stream(void* pipeline, void* stream);
QMM_API int qmm_host_pipeline_sync(void* pipeline);
QMM_API int qmm_host_pipeline_destroy(void* pipeline);

/*
 * Device-side error word of the current device.  Kernels that wait on hardware barriers give up
 * after a bounded number of polls and record a non-zero code here instead of hanging.
 * Reads the word back (this call synchronises `stream`), stores it in *flag (HOST pointer) and
 * clears it.  Returns QMM_ERR_TIMEOUT if it was non-zero.
 */
QMM_API int qmm_device_error_flag(uint32_t* flag, void* stream);

/*
 * Precision of the split-activation kernel (QMM_VARIANT_I8TC) above 32 tokens.  It rewrites every activation row as
 * fixed point below the row's largest value and multiplies int8 "limbs" of it with the integer weights exactly.
 * Three limbs (22 bits) give the accuracy of an fp32 accumulation and are used for fp32 outputs and for every batch
 * of up to 32 tokens.  limbs = 0 (default): bf16 / f16 outputs above 32 tokens use two limbs, i.e. each activation
 * carries an error of at most 2^-15 of its row's largest |x| - ~1e-4 of the output's scale for N(0,1) rows, ~1e-3
 * when 1 % of the entries are 20 times larger, under the 2^-9 rounding of a bf16 output; a third fewer tensor-core
 * columns per token.  limbs = 3: three limbs everywhere.  Process-wide; applies to launches made after the call.
 * The reference multiplies bf16 activations with the up-cast weights in bf16 x bf16 -> fp32
 * (torch_xla/experimental/xla_quantized_matmul.py:113-114, :120-124); it has no such knob.
 */
QMM_API int qmm_set_activation_limbs(int limbs);

/*
 * How long the kernels that wait for another GPU (qmm_allreduce_oneshot, qmm_rowparallel_decode) keep waiting
 * before they give up: `seconds` of SM clock at about 2 GHz, in (0, 60]; the default is about one second.  On
 * expiry the kernel sets the device error word (code 7: all-reduce kernel, 8: fused decode exchange; the peer's
 * rank in bits 8 and up), fills its result with NaN and returns; the context stays usable.  Process-wide; applies
 * to launches made after the call.  Stands in for the reference's collective timeouts, which live in the PJRT
 * runtime (torch_xla/csrc/runtime/), not in this operator.
 */
QMM_API int qmm_set_peer_wait_limit(double seconds);

/*
 * Measurement aid: reads `bytes` of device memory at `p` (16-byte aligned) once with streaming loads and discards them;
 * `sink` is 4 bytes of device memory.  The time of this kernel is what a decode linear whose weights are those bytes
 * could reach at best on the same launch path.  No counterpart in the reference.
 */
QMM_API int qmm_stream_read(const void* p, size_t bytes, void* sink, void* stream);

/* Name of the kernel family the AUTO heuristic picks (static string, for logs and tests). */
QMM_API const char* qmm_variant_for(int op, int64_t M, int64_t N, int64_t K, int64_t block_size,
                            int has_zp);

#ifdef __cplusplus
}
#endif

#endif /* QMM_B200_H_ */
