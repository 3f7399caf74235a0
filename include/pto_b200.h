/*
 * pto_b200.h - C ABI of the B200 (sm_100a) implementation of the PTO tile library's GEMM hot path.
 *
 * Every entry point enqueues work on the caller's CUDA stream and returns immediately (no implicit
 * synchronisation), like the reference launchers that take `void* stream`. All matrix pointers are
 * device pointers passed as uint8_t*, as in the reference (`uint8_t* out, uint8_t* src0, uint8_t* src1`).
 * The caller owns every buffer; the library allocates no device memory.
 *
 * Return value: 0 on success, otherwise a PTO_B200_E* code (see pto_b200_error_string). Argument
 * errors are reported before anything is launched; nothing aborts or traps.
 *
 * Storage conventions (reference: include/pto/common/pto_tile.hpp Layout::ND / Layout::DN):
 *   A    : M x K, row-major (ND), leading dimension lda >= K                       (elements)
 *   B    : PTO_B200_B_DN  - column-major K x N, i.e. stored N x K row-major, ldb >= K
 *          PTO_B200_B_ND  - row-major K x N, ldb >= N (16-bit inputs only)
 *   C    : M x N, row-major (ND), ldc >= N
 * Base addresses of A and B must be 16-byte aligned and lda/ldb * element size multiples of 16 bytes
 * (TMA requirement); C has no alignment requirement (aligned C takes the vector-store path).
 */
#ifndef PTO_B200_H
#define PTO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    PTO_B200_F16 = 0,  /* IEEE half            (reference `half`)          */
    PTO_B200_BF16 = 1, /* bfloat16             (reference `bfloat16_t`)    */
    PTO_B200_F32 = 2,  /* float                                              */
    PTO_B200_S8 = 3,   /* int8_t                                             */
    PTO_B200_S32 = 4,  /* int32_t                                            */
    PTO_B200_E4M3 = 5, /* float8_e4m3_t (fn variant: no inf, 0x7f NaN)      */
    PTO_B200_E5M2 = 6, /* float8_e5m2_t                                      */
    PTO_B200_E2M1 = 7, /* float4_e2m1x2_t: two 4-bit values per byte, the even element in the low nibble */
    PTO_B200_U8 = 8,   /* uint8_t (destination of the 8-bit pre-quant stores)     */
    PTO_B200_S16 = 9   /* int16_t (destination of the shifting pre-quant store)   */
} pto_b200_dtype;

typedef enum {
    PTO_B200_B_DN = 0, /* B column-major (stored N x K); gemm_performance, mxfp8, gemm_ar */
    PTO_B200_B_ND = 1  /* B row-major (stored K x N); demos/cpu/gemm_demo              */
} pto_b200_b_layout;

enum {
    PTO_B200_OK = 0,
    PTO_B200_EINVAL = 1,      /* null pointer, non-positive size, ld smaller than the row length  */
    PTO_B200_EALIGN = 2,      /* A/B base or leading dimension breaks the 16-byte TMA rule        */
    PTO_B200_EDTYPE = 3,      /* dtype / layout combination outside CheckMadValid's table          */
    PTO_B200_EWORKSPACE = 4,  /* workspace missing, misaligned or too small                        */
    PTO_B200_ECUDA = 5,       /* a CUDA runtime / driver call failed (see pto_b200_last_cuda_error)*/
    PTO_B200_EDEVICE = 6,     /* current device is not compute capability 10.0                     */
    PTO_B200_ETIMEOUT = 7,    /* a kernel gave up on a bounded wait (see pto_b200_device_status)   */
    PTO_B200_ESCRATCH = 8     /* problem needs more than PTO_B200_MX_STATIC_SCRATCH_BYTES of built-in scratch */
};

/*
 * Dense GEMM, C = A * B, fp32 (or int32) accumulate over the whole K: the tile loop
 * TLOAD -> TEXTRACT -> TMATMUL (k == 0) / TMATMUL_ACC (k > 0) -> TSTORE.
 * Replaces: RunGemmE2E / LaunchGEMME2E<T>, kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:170-273
 * (which hard-codes m = n = k = 6144; sizes are run-time arguments here).
 *   in_dtype F16 or BF16 -> out_dtype F32, BF16 or F16 (cast = round to nearest even, TSTORE's static_cast,
 *                           include/pto/cpu/TStore.hpp:187-198)
 *   in_dtype S8          -> out_dtype S32 (exact accumulators, include/pto/cpu/TMatmul.hpp:104-106)
 * K-split use (gemm_ar `k_per_rank`, kernels/manual/a2a3/gemm_ar/gemm_compute_kernel.cpp:150-165): pass the
 * rank's slice pointers with lda = ldb = full K, k = K / ranks and out_dtype F32 to get the fp32 partial.
 */
int pto_b200_gemm(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n, int k,
                  long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype, int b_layout);

/*
 * pto_b200_gemm with the number of thread blocks capped, the `launch_block_count` argument of the reference's
 * launchGemmCompute (kernels/manual/a2a3/gemm_ar/gemm_compute_kernel.cpp:254-259): the GEMM then occupies at most
 * that many SMs and leaves the rest to a communication kernel running beside it on another stream
 * (kernels/manual/a2a3/gemm_ar/README.md:327 describes the same trade). 0 = use every SM.
 */
int pto_b200_gemm_ex(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n, int k,
                     long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype, int b_layout,
                     int launch_block_count);

/*
 * pto_b200_gemm_ex with an optional workspace for the last, partly filled wave of tiles. The reference assigns each
 * core a fixed sub-matrix (InitGMOffsets, gemm_performance_kernel.cpp:48-67) and has no counterpart; on 148 SMs a
 * 4096^3 problem leaves the last wave 46 % full, so with a workspace each leftover tile is cut into two K halves
 * that run on two CTA pairs at once and then swap: each pair parks the 32-bit accumulators of the 128 columns the
 * other pair finishes in the workspace, adds the other's half to its own and stores. Results differ from the unsplit
 * chain only by the fp32 summation order (int32: exact).
 *   workspace : device memory of pto_b200_gemm_workspace_bytes() bytes, 16-byte aligned, ZERO before its first use,
 *               or NULL = never split. One workspace must not be used by two launches that can overlap on the GPU
 *               (use one per stream). The split is skipped when launch_block_count caps the blocks: the two pairs of
 *               a tile wait for each other inside the kernel, so all blocks of the launch must be on the GPU at once.
 */
size_t pto_b200_gemm_workspace_bytes(void);
int pto_b200_gemm_ws(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n, int k,
                     long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype, int b_layout,
                     int launch_block_count, uint8_t* workspace, size_t workspace_bytes);

/*
 * pto_b200_gemm with a bias row: C[i][j] = (sum_k A[i][k] * B[k][j]) + bias[j], cast to out_dtype afterwards.
 * Replaces: TMATMUL_BIAS(c, a, b, bias) as the first step of the K loop followed by TMATMUL_ACC
 * (include/pto/common/pto_instr.hpp:1000-1015; arithmetic include/pto/cpu/TMatmul.hpp:219-230: the matmul result,
 * then bias added per column in the accumulator's type, CheckBiasValid :159-167).
 *   bias : n values of the accumulator type in device memory, 4-byte aligned: fp32 for F16 / BF16 inputs,
 *          int32 for S8 inputs (out_dtype S32).
 * The bias is added once to the finished accumulator: identical to the reference for int32; for fp32 the reference
 * adds it after the first baseK chunk of the chain, one fp32 rounding apart (inside the dense tolerance).
 */
int pto_b200_gemm_bias(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, const uint8_t* bias,
                       int m, int n, int k, long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype,
                       int b_layout);

/*
 * int8 x int8 -> int32 GEMM with the dequantising store fused:
 *   out[i][j] = bf16( (float(acc[i][j]) * s_col[j]) * s_row[i] ),  two separately rounded fp32 multiplies.
 * Replaces: TMATMUL/TMATMUL_ACC on int8 tiles + TSTORE_FP per-column dequant
 * (kernels/manual/a2a3/dispatch_mega_combine/op_kernel/utils/pto_gmm_preload_async_fixpipe_quant.hpp:75-124,409-411;
 * scale arithmetic include/pto/cpu/common.hpp:139-185) followed by the per-token row scale
 * (op_kernel/swiglu.h:101,113). s_col is used as a full fp32 value; to match the reference's 19-bit
 * per-column scale encoding bit for bit, pass s_col with the low 13 mantissa bits zero.
 * B is PTO_B200_B_DN. s_row has m floats, s_col n floats (device memory).
 */
int pto_b200_gemm_s8_dequant(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                             const float* s_row, const float* s_col, int m, int n, int k, long long lda,
                             long long ldb, long long ldc);

/*
 * GEMM whose store applies a pre-quant scale word: out[i][j] = cast16( relu?( clamp( float(acc[i][j]) * scale_j ) ) ).
 * Replaces: TMATMUL / TMATMUL_ACC followed by TSTORE(dst, acc, uint64_t preQuantScalar) (include/pto/common/
 * pto_instr.hpp:441-462) or by TSTORE(dst, acc, fpTile) / TSTORE_FP (:464-518), with the mode the overloads pick
 * (GetScalarPreQuantMode / GetVectorPreQuantMode, include/pto/cpu/common.hpp:58-108) and the arithmetic of
 * quantize_element (:139-185); kernel usage kernels/manual/a2a3/dispatch_mega_combine/op_kernel/utils/
 * pto_gmm_preload_async_fixpipe_quant.hpp:75-124.
 *   in_dtype S8 (int32 accumulators: QS322BF16_PRE / VQS322BF16_PRE, DEQF16 / VDEQF16) or F16 / BF16 (fp32
 *   accumulators: QF322BF16_PRE / VQF322BF16_PRE, QF322F16_PRE / VQF322F16_PRE); out_dtype BF16 or F16, or S8 / U8
 *   (REQ8 / VREQ8 for int32 accumulators, QF322B8_PRE / VQF322B8_PRE for fp32 ones: out = relu?( clamp( rint(
 *   float(acc) * scale_j + offset ) ) ) as one byte, offset = the 9-bit field in bits [45:37] of the word, clamp range
 *   -128..127 when bit 46 of the word is set, else 0..255; S8 and U8 store the same byte); B is PTO_B200_B_DN.
 *   fp_words == NULL : scalar form, scale = the fp32 value in bits [31:0] of pre_quant_scalar for every column
 *   fp_words != NULL : vector form, n 64-bit words in device memory (8-byte aligned), one per column; the scale is the
 *                      19-bit float (sign, 8 exponent, 10 mantissa bits) in bits [31:13] of the word, i.e. fp32 with
 *                      the low 13 mantissa bits ignored (extract_m1_from_quant, common.hpp:116-137)
 *   relu != 0        : ReluPreMode::NormalRelu, applied after the scaling
 *   out_dtype S16 (in_dtype S8 only; SHIFTS322S16 / VSHIFTS322S16): out = relu?( int16( acc >> (1 + bits [35:32] of the
 *   word) ) ), an arithmetic shift and the wrapping cast of the reference; no scale is applied.
 * Half outputs are clamped to +-65504 as the reference does.
 */
int pto_b200_gemm_quant(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n, int k,
                        long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype,
                        unsigned long long pre_quant_scalar, const unsigned long long* fp_words, int relu);

/*
 * MX block-scaled fp8 GEMM: C[i][j] = sum_k A[i][k] * B[k][j] * 2^(SA[i][k/32]-127) * 2^(SB[j][k/32]-127).
 * Replaces: RunMxMatmul / LaunchMxMatmul (uint8_t* out, src0, src1, src2, src3, void* stream),
 * kernels/manual/a5/matmul_mxfp8_performance/mxmatmul_performance_kernel.cpp:284-380; arithmetic
 * TMATMUL_MX, include/pto/cpu/TMatmul.hpp:169-205.
 *   src2 : e8m0 scales of A, M x K/32 row-major (Layout::MX_A_ND), leading dimension ld_sfa bytes
 *   src3 : e8m0 scales of B, N x K/32 row-major (Layout::MX_B_DN), leading dimension ld_sfb bytes
 *   a_dtype / b_dtype : E4M3 or E5M2 (any mix), or both E2M1 (MXFP4: kernels/manual/a5/matmul_mxfp4_performance,
 *                       float4_e2m1x2_t of include/pto/cpu/MXTypes.hpp:316-359; lda / ldb still count ELEMENTS, a row
 *                       holds k / 2 bytes; bases 32-byte aligned, lda and ldb multiples of 64, k a multiple of 128);
 *                       out_dtype BF16 or F32; B is PTO_B200_B_DN; k % 32 == 0.
 *   workspace : device scratch of at least pto_b200_gemm_mx_workspace_bytes(m, n, k) bytes, 16-byte aligned;
 *               the scales are re-tiled into it by a small kernel on the same stream before the GEMM. With
 *               pto_b200_gemm_workspace_bytes() MORE bytes (zero before their first use) the CTA-pair kernel also cuts a
 *               partly filled last wave of tiles into K halves, as pto_b200_gemm_ws does, under the same rule: such a
 *               workspace must not be used by two launches that can overlap. The same holds for the tiled_scales
 *               buffer of pto_b200_mx_retile_scales / pto_b200_gemm_mx_pretiled.
 * Scale byte 0xFF (NaN in the e8m0 encoding) is outside the supported input domain.
 */
int pto_b200_gemm_mx(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, const uint8_t* src2,
                     const uint8_t* src3, uint8_t* workspace, size_t workspace_bytes, int m, int n, int k,
                     long long lda, long long ldb, long long ldc, long long ld_sfa, long long ld_sfb, int a_dtype,
                     int b_dtype, int out_dtype);

size_t pto_b200_gemm_mx_workspace_bytes(int m, int n, int k);

/*
 * pto_b200_gemm_mx in two steps, for scales that do not change between calls (the weights' scales) or that a producer
 * can write in the tiled form directly: pto_b200_mx_retile_scales fills the workspace from the reference-layout scale
 * tensors (one small re-tile kernel, about 3 % of a 16384 x 8192 x 8192 call), pto_b200_gemm_mx_pretiled multiplies
 * with a workspace that was filled earlier for the same m, n, k. The reference's counterpart are its pre-tiled scale
 * layouts, Layout::MX_A_ZZ / Layout::MX_B_NN (include/pto/common/pto_tile.hpp:849-881,943-975), whose fractal order
 * belongs to its L0 scale buffers; here the order is the one tcgen05.cp copies into tensor memory: 512-byte atoms
 * (k_block of 128, 128-row block), byte (r % 32) * 16 + (r / 32) * 4 + j for row r and K group j; all A atoms first
 * (2 * ceil(m / 256) row blocks per k_block), then B's (2 * ceil(n / 256)); rows and groups past the end hold 127.
 */
int pto_b200_mx_retile_scales(void* stream, uint8_t* workspace, size_t workspace_bytes, const uint8_t* src2,
                              const uint8_t* src3, int m, int n, int k, long long ld_sfa, long long ld_sfb);
int pto_b200_gemm_mx_pretiled(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                              const uint8_t* tiled_scales, size_t tiled_bytes, int m, int n, int k, long long lda,
                              long long ldb, long long ldc, int a_dtype, int b_dtype, int out_dtype);

/*
 * pto_b200_gemm_mx with an fp32 bias row added to the finished accumulator: the six-operand TMATMUL_MX
 * (c, a, a_scale, b, b_scale, bias), include/pto/common/pto_instr.hpp:918-942, include/pto/cpu/TMatmul.hpp:271-292.
 * bias : n floats in device memory.
 */
int pto_b200_gemm_mx_bias(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, const uint8_t* src2,
                          const uint8_t* src3, const uint8_t* bias, uint8_t* workspace, size_t workspace_bytes, int m,
                          int n, int k, long long lda, long long ldb, long long ldc, long long ld_sfa,
                          long long ld_sfb, int a_dtype, int b_dtype, int out_dtype);

/*
 * pto_b200_gemm_mx without a workspace argument. No counterpart in the reference (its launchers never need
 * scratch); it exists for callers that have no way to obtain device memory at the moment of the call:
 *   - code that keeps the reference's exact launcher shape, LaunchMxMatmul(out, src0, src1, src2, src3, stream),
 *     and therefore has nowhere to pass a sixth buffer;
 *   - processes whose device memory was handed out in full at start-up (a serving process that reserves the whole
 *     HBM for its own pool), where a cudaMalloc made later fails or stalls the device.
 * The re-tiled scale factors go into an array that lives inside this library's device image
 * (PTO_B200_MX_STATIC_SCRATCH_BYTES, held on every GPU that loads the library until the process exits), so this
 * call allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.
 *
 * Limits and rules:
 *   - pto_b200_gemm_mx_workspace_bytes(m, n, k) must not exceed PTO_B200_MX_STATIC_SCRATCH_BYTES, otherwise the call
 *     returns PTO_B200_ESCRATCH and launches nothing (8 MiB covers 16384 x 8192 x 8192 and 6144^3).
 *   - The first call on each device looks up the array's device address (one cudaGetSymbolAddress with that device
 *     current). Make that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left there. Each call
 *     rewrites every byte it later reads, so nothing has to be cleared; but two calls whose kernels can overlap on
 *     the GPU (different streams, no event between them) race on it. Serialise them, or use pto_b200_gemm_mx with
 *     separate workspaces.
 * Arguments, results and error codes are otherwise those of pto_b200_gemm_mx.
 */
#define PTO_B200_MX_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
int pto_b200_gemm_mx_static(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                            const uint8_t* src2, const uint8_t* src3, int m, int n, int k, long long lda,
                            long long ldb, long long ldc, long long ld_sfa, long long ld_sfb, int a_dtype,
                            int b_dtype, int out_dtype);

/*
 * fp32 -> bf16 cast (round to nearest even) of `count` contiguous elements: the TSTORE cast applied to the
 * reduced K-split partials (gemm_ar: reduced_output -> fp16/bf16 result, kernels/manual/a2a3/gemm_ar/README.md:33-46).
 */
int pto_b200_cast_f32_to_bf16(void* stream, uint8_t* out, const uint8_t* in, long long count);

/*
 * One left row: out[j] = sum_k a[k] * B[k][j] (+ bias[j]).
 * Replaces: TGEMV / TGEMV_BIAS (include/pto/common/pto_instr.hpp:1019-1060; include/pto/cpu/TMatmul.hpp:232-252,
 * the TMATMUL arithmetic with a one-row left tile; reference cases tests/cpu/st/testcase/tmatmul case_gemm_*).
 *   src0 : the left row, k elements, 16-byte aligned
 *   src1 : B column-major (PTO_B200_B_DN), n runs of k elements, leading dimension ldb elements (rows 16-byte aligned)
 *   bias : n values of the accumulator type (fp32, or int32 for S8 inputs), or null
 *   in_dtype F16 / BF16 (out F32 / BF16 / F16) or S8 (out S32).
 * Bandwidth-bound: B is streamed once with plain loads, no tensor-core tile. The fp32 sum is formed from 32 partial
 * sums, not as the reference's single chain: within the dense tolerance; int32 is exact.
 */
int pto_b200_gemv(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, const uint8_t* bias, int n,
                  int k, long long ldb, int in_dtype, int out_dtype);

/*
 * One left row against a block-scaled fp8 matrix:
 *   out[j] = sum_k a[k] * B[k][j] * 2^(SA[k/32] - 127) * 2^(SB[j][k/32] - 127)  (+ bias[j]).
 * Replaces: TGEMV_MX (include/pto/common/pto_instr.hpp:797-862: plain, accumulating and bias forms;
 * include/pto/cpu/TMatmul.hpp:294-326, the TMATMUL_MX arithmetic with a one-row left tile).
 *   src0 : the left row, k fp8 bytes, 16-byte aligned;      src2 : its k / 32 e8m0 scales
 *   src1 : B column-major (n runs of k bytes, leading dimension ldb, a multiple of 16); src3 : its scales [n][ld_sfb]
 *   bias : n floats or null; a_dtype / b_dtype E4M3 or E5M2 (any mix); out_dtype F32 or BF16; k % 32 == 0.
 * Bandwidth-bound like pto_b200_gemv: B and its scales are streamed once, no tensor-core tile.
 */
int pto_b200_gemv_mx(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, const uint8_t* src2,
                     const uint8_t* src3, const uint8_t* bias, int n, int k, long long ldb, long long ld_sfb, int a_dtype,
                     int b_dtype, int out_dtype);

/*
 * OCP MX quantisation of fp32 rows into e4m3 bytes and e8m0 block scales (one per 32 elements along k): the
 * producer of pto_b200_gemm_mx's src0 / src2 (or src1 / src3) operands.
 * Replaces: TQUANT<QuantType::MXFP8> with the OCP scale rule (include/pto/common/pto_instr.hpp:2981-3035;
 * include/pto/cpu/TQuant.hpp:178-190 shared exponent, :226-237 scaling, :118-153 e4m3fn encoding, :461-494 grouping).
 *   src    : rows x k floats, leading dimension ld_src elements (multiple of 4), 16-byte aligned, finite values
 *   data   : rows x k bytes, leading dimension ld_data bytes (multiple of 4), 4-byte aligned
 *   scales : rows x k/32 bytes, leading dimension ld_scales bytes
 *   k % 32 == 0. Bit-identical to the reference for finite input.
 */
int pto_b200_mx_quantize_e4m3(void* stream, uint8_t* data, uint8_t* scales, const uint8_t* src, int rows, int k,
                              long long ld_src, long long ld_data, long long ld_scales);

/*
 * The same with the scale rule as an argument: QuantScaleAlg::OCP or QuantScaleAlg::NV (include/pto/common/type.hpp:205-208).
 * NV (include/pto/cpu/TQuant.hpp:33-37,194-211,239-248, the NV form of EncodeE4M3Fn :118-131): the block scale is the
 * smallest power of two that brings absmax to at most 448 (e8m0 = biased exponent of absmax / 448, rounded up), and
 * scaled values below 2^-10 in magnitude are stored as zeros that keep their sign. Bit-identical to the reference for
 * finite input.
 */
typedef enum { PTO_B200_SCALE_OCP = 0, PTO_B200_SCALE_NV = 1 } pto_b200_scale_alg;
int pto_b200_mx_quantize_e4m3_ex(void* stream, uint8_t* data, uint8_t* scales, const uint8_t* src, int rows, int k,
                                 long long ld_src, long long ld_data, long long ld_scales, int scale_alg);

/*
 * TQUANT to MXFP4: fp32 rows into packed float4_e2m1x2_t bytes and e8m0 block scales (one per 32 elements along k),
 * the producer of the PTO_B200_E2M1 operands of pto_b200_gemm_mx. Replaces TQUANT<QuantType::MXFP4_E2M1> with a float
 * source under either scale rule, include/pto/cpu/TQuant.hpp:280-372 (group maximum :280-305 - the OCP rule takes it
 * over the values truncated to bf16 -, shared exponent :210-221 (OCP: biased exponent - 2) / :194-208 with the e2m1 spec
 * :39-45 (NV: absmax / 6 rounded up to a power of two), scaling :226-248, element code EncodeE2M1Magic :155-176: round
 * to nearest even on the e2m1 grid, saturating at 6, sign kept on zeros).
 *   src    : rows x k floats, leading dimension ld_src elements (multiple of 4), 16-byte aligned, finite values
 *   data   : rows x k/2 bytes (element 2i in the low nibble of byte i), leading dimension ld_data bytes (even), 2-byte aligned
 *   scales : rows x k/32 bytes, leading dimension ld_scales bytes
 *   k % 32 == 0; scale_alg PTO_B200_SCALE_OCP or PTO_B200_SCALE_NV. Bit-identical to the reference for finite input.
 */
int pto_b200_mx_quantize_e2m1(void* stream, uint8_t* data, uint8_t* scales, const uint8_t* src, int rows, int k,
                              long long ld_src, long long ld_data, long long ld_scales, int scale_alg);

/*
 * K-split reduction over peer memory: the reduce-scatter / all-gather half of the reference's GEMM + AllReduce
 * (kernels/manual/a2a3/gemm_ar/comm_kernel.cpp:165-210 reduce-scatter into the owner's window, :377-400 all-gather,
 * :111-123 and :528-590 the TNOTIFY / TWAIT counters), one process per GPU, buffers mapped into every rank
 * (the reference's HCCL windows; here any peer-mapped allocation, e.g. torch symmetric memory). All pointer arrays
 * are HOST arrays of `world` device pointers, entry r = rank r's buffer as mapped in this process. Flag arrays hold
 * PTO_B200_KSPLIT_FLAG_STRIDE ints per slot and must be zero before the first step; epochs start at 1 and only grow.
 *
 *   pto_b200_ksplit_signal : on the GEMM's stream after the GEMM of one row panel; stores ready[slot][rank] = epoch
 *                            into every rank's ready-flag array.
 *   pto_b200_ksplit_reduce : waits (bounded) until ready[slot][r] >= epoch for every r in this rank's array, then
 *                            for rows [row0, row0 + rows) - this rank's shard of the panel - sums the fp32 partials
 *                            of all ranks in rank order, casts to bf16 (round to nearest even) and stores the result
 *                            into every rank's output; finally stores done[slot][rank] = epoch into every rank's
 *                            done-flag array. launch_block_count = thread blocks to use (0 = 32).
 *                            multicast_partial / multicast_out: NVSwitch multicast addresses of the same partial /
 *                            output buffers (NVLS), or null. With them the sum is formed inside the switch
 *                            (multimem.ld_reduce, the switch's own fixed order) and the result is broadcast with one
 *                            multimem.st; without them plain peer loads are summed in rank order and stored per rank.
 *   pto_b200_ksplit_wait   : waits (bounded) until done[slot][r] >= epoch for slots [slot0, slot0 + slots), all r.
 * A wait that gives up records a code in the status word (pto_b200_device_status) and the kernel returns.
 */
#define PTO_B200_KSPLIT_MAX_RANKS 8
#define PTO_B200_KSPLIT_FLAG_STRIDE 8
int pto_b200_ksplit_signal(void* stream, void* const* flag_arrays, int world, int rank, int slot, int epoch);
int pto_b200_ksplit_reduce(void* stream, void* const* partial_ptrs, void* const* out_ptrs, void* const* done_arrays,
                           const int* ready_local, int* cta_counters_local, int world, int rank, int slot, int epoch,
                           long long row0, int rows, int n, long long ld_partial, long long ld_out,
                           int launch_block_count, const void* multicast_partial, void* multicast_out);
int pto_b200_ksplit_wait(void* stream, const int* done_local, int world, int slot0, int slots, int epoch);

/*
 * One rank's whole step of the K-split GEMM + allreduce in ONE kernel launch: this rank's GEMM over its K slice,
 * row panel by row panel into its fp32 partial, and - by extra warps of the same kernel - the exchange of every
 * finished panel over peer memory: wait for all ranks' partials of the panel, sum this rank's row shard of it (NVSwitch
 * multimem.ld_reduce when multicast addresses are given, else plain peer loads in rank order), cast to bf16, store into
 * every rank's output, and finally wait until every rank has delivered every panel into this rank's output.
 * Replaces: launchGemmCompute + launchGemmCommAll running on two streams (kernels/manual/a2a3/gemm_ar/
 * gemm_compute_kernel.cpp:150-259 tile loop that fills the ready queue, comm_kernel.cpp:165-210 reduce-scatter,
 * :377-400 all-gather, :528-590 queue consumer, :725 launcher; main.cpp:761-800 the two-stream step).
 *   src0 / src1   : this rank's K slice of A [m, k_local] (lda) and of column-major B [n, k_local] (ldb), F16 or BF16
 *   partial_ptrs  : every rank's fp32 partial [m, ld_partial] of THIS step (double-buffer across steps: a slow peer may
 *                   still be reading the previous step's partial); entry `rank` is written by this launch
 *   out_ptrs      : every rank's bf16 output [m, ld_out]
 *   ready_arrays / done_arrays : every rank's flag arrays (PTO_B200_KSPLIT_FLAG_STRIDE ints per slot, zero before the
 *                   first step); slots [slot0, slot0 + panels) are used, with panels = ceil(m / panel_rows)
 *   panel_counters_local / exchange_counters_local : this rank's scratch, one int per slot, zero before the first step
 *   epoch         : 1, 2, 3, ... one per step, the same on every rank
 *   panel_rows    : rows of a panel, a multiple of 256
 *   multicast_partial / multicast_out : NVSwitch multicast addresses of the same partial / output buffers, or null
 *   launch_block_count : cap on thread blocks, 0 = every SM
 * All ranks must launch the same step at about the same time: a rank waits at most the wait limit
 * (pto_b200_set_wait_limit) for the others, then records a code in the status word and returns. The launch must be
 * able to hold all its thread blocks on the GPU at once (nothing else resident that takes whole SMs), because blocks
 * wait for panels that other blocks of the same launch complete. No TMA load and no multicast load reads peer memory:
 * peers are reached by the exchange warps' own loads and stores only. Every rank receives identical bits.
 */
int pto_b200_ksplit_gemm_allreduce(void* stream, const uint8_t* src0, const uint8_t* src1, int m, int n, int k_local,
                                   long long lda, long long ldb, int in_dtype, void* const* partial_ptrs,
                                   void* const* out_ptrs, void* const* ready_arrays, void* const* done_arrays,
                                   int* panel_counters_local, int* exchange_counters_local, int world, int rank,
                                   int slot0, int epoch, int panel_rows, long long ld_partial, long long ld_out,
                                   const void* multicast_partial, void* multicast_out, int launch_block_count);

/*
 * One rank's whole step of AllGather + GEMM in ONE kernel launch: every rank holds an M slice of A, B is replicated,
 * every rank ends with the whole C = A * B. Extra warps of the GEMM kernel push this rank's slice, 256-row block by
 * block, into every rank's copy of A (one NVSwitch multicast store per 16 bytes when a multicast address is given,
 * else one store per peer) and publish a flag per block; the tile loop starts with this rank's own rows and waits for
 * the flag of a remote block before its first load from it, so multiplication starts before the gather completes.
 * Replaces: launchRingCommStreaming + launchAllGatherGemmComputeStreaming on two streams
 * (kernels/manual/a2a3/allgather_gemm/allgather_gemm_comm_kernel.cpp:255, allgather_gemm_compute_kernel.cpp:393;
 * pipeline described in kernels/manual/a2a3/allgather_gemm/README.md:28-110).
 *   a_ptrs        : every rank's copy of A [m, lda] as mapped in this process; rank r owns rows [r m/world, (r+1) m/world)
 *                   and must have written them into ITS copy before the launch; the other rows are filled by the peers
 *   src1          : B, column-major [n, k] (ldb), the same on every rank; in_dtype F16 or BF16
 *   out           : this rank's C [m, n] (ldc), out_dtype F32, BF16 or F16
 *   flag_arrays   : every rank's flag array, ceil(m / 256) + PTO_B200_KSPLIT_MAX_RANKS ints, zero before the first step
 *   block_counters_local : this rank's scratch, m / (256 world) ints, zero before the first step
 *   done_counter_local   : this rank's scratch, one int, zero before the first step
 *   epoch         : 1, 2, 3, ... one per step, the same on every rank
 *   multicast_a   : NVSwitch multicast address of the A copies, or null
 * m must be a multiple of 256 * world and k of 8. A step's pushes wait (bounded) until every rank has finished
 * reading the previous step's rows. As for pto_b200_ksplit_gemm_allreduce, all ranks launch the same step at about the
 * same time and the launch must be able to hold all its thread blocks on the GPU at once. TMA loads read this GPU's
 * own copy of A only; peers are reached by plain or multimem stores.
 */
int pto_b200_allgather_gemm(void* stream, uint8_t* out, void* const* a_ptrs, const uint8_t* src1, int m, int n, int k,
                            long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype,
                            void* const* flag_arrays, int* block_counters_local, int* done_counter_local, int world,
                            int rank, int epoch, void* multicast_a, int launch_block_count);

/*
 * Cycles a kernel of this library waits on one barrier or flag before it gives up (records a code in the status
 * word, see pto_b200_device_status, and returns without trapping). Default 4e9 (about two seconds); cycles <= 0
 * restores the default. Applies to launches made after the call; returns the previous value. The reference has no
 * counterpart (its TWAIT spins without a limit, kernels/manual/a2a3/gemm_ar/comm_kernel.cpp:528-590).
 */
long long pto_b200_set_wait_limit(long long cycles);

/*
 * Fixed-shape launchers with the reference's exact signatures.
 * call_kernel: demos/torch_jit/gemm/gemm_kernel.cpp:263-266 (fp16 6144^3, B column-major, fp32 out; blockDim ignored).
 */
void call_kernel(uint32_t blockDim, void* stream, uint8_t* out, uint8_t* src0, uint8_t* src1);

/*
 * Synchronises the current device and returns the kernel status word in *status (0 = every bounded wait
 * completed; non-zero = the first wait that gave up) and clears it. Returns PTO_B200_ETIMEOUT if non-zero.
 */
int pto_b200_device_status(int* status);

const char* pto_b200_error_string(int code);
/* Text of the last CUDA error seen by the calling thread inside this library ("" if none). */
const char* pto_b200_last_cuda_error(void);
/* Kernels launched by this library since it was loaded (all threads). */
unsigned long long pto_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* PTO_B200_H */
