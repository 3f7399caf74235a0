// OCP MX quantisation on the device: fp32 [rows][k] -> e4m3fn bytes [rows][k] + one e8m0 scale per 32 elements of K.
//
// Follows TQUANT<QuantType::MXFP8> with the OCP scale rule (include/pto/cpu/TQuant.hpp: group maximum and shared
// exponent ComputeSharedExponent :178-190, scaling factor ComputeMxScalingFromExponent :226-237, element encoding
// EncodeE4M3Fn :118-153, grouping of 32 along the row QuantizeMxTile :461-494; MX_BLOCK_SIZE = 32,
// include/pto/common/constants.hpp:42):
//   e8m0    = max(biased_exponent(absmax of the 32 values) - 8, 0)
//   scaling = 2^(127 - e8m0)
//   byte    = nearest e4m3fn code of clamp(x * scaling, +-448), ties to the even code; a result that rounds to zero
//             is stored as +0 (0x00) whatever its sign.
// With the NV scale rule (ComputeNvSharedExponent with the e4m3 spec, TQuant.hpp:33-37,194-211; scaling :239-248; the
// NV form of EncodeE4M3Fn :118-131):
//   e8m0    = biased exponent of absmax / 448, plus one unless absmax / 448 is a power of two (0 for an all-zero block)
//   byte    = as above, except that a scaled value below 2^-10 in magnitude is stored as a zero WITH its sign.
// Inputs must be finite (a NaN or infinity in a block is outside the supported domain).
//
// HBM-bound: 4 bytes read and 1 + 1/32 bytes written per element. Eight consecutive lanes own one block of 32
// values (one 16-byte load each), share the maximum with three shuffles and store 4 bytes each, so a warp reads 512
// contiguous bytes and writes 128.
#pragma once
#include <cuda_fp8.h>

#include <cstdint>

namespace pto_b200 {

constexpr int kQuantThreads = 256;

// Two floats -> two e4m3fn codes (low byte = first value), round to nearest even, saturating at +-448.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t drop_negative_zero(uint32_t four_codes)
{
    // a byte that is exactly 0x80 (negative zero) becomes 0x00; other bytes stay
    const uint32_t magnitude = four_codes & 0x7F7F7F7Fu;
    const uint32_t nonzero = ((magnitude + 0x7F7F7F7Fu) | magnitude) & 0x80808080u; // 0x80 per byte with magnitude != 0
    return magnitude | (four_codes & nonzero);
}

constexpr int kQuantItems = 4; // 16-byte loads in flight per thread

// src: [rows][ld_src] floats (16-byte aligned rows); data: [rows][ld_data] bytes (4-byte aligned rows);
// scales: [rows][ld_scales] bytes. k % 32 == 0.
enum MxScaleAlg : int { MX_SCALE_OCP = 0, MX_SCALE_NV = 1 };

template <int ALG>
__global__ void __launch_bounds__(kQuantThreads) mx_quantize_e4m3_kernel(const float* __restrict__ src,
                                                                          uint8_t* __restrict__ data,
                                                                          uint8_t* __restrict__ scales, int rows, int k,
                                                                          long long ld_src, long long ld_data,
                                                                          long long ld_scales)
{
    const int k4 = k / 4;
    const long long total = static_cast<long long>(rows) * k4; // 16-byte items; a multiple of 8 per row
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const unsigned group_mask = 0xFFu << (threadIdx.x & 24u);
    // (row, column) of the running item index, advanced by one stride per item: one division per thread, none per item
    const long long row_step = stride / k4;
    const int col_step = static_cast<int>(stride - row_step * k4);
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    long long cur_row = i / k4;
    int cur_c4 = static_cast<int>(i - cur_row * k4);
    // total and stride are multiples of 8, so the eight lanes of a group hold items of one 32-value block that are
    // all in range or all out of range: the group's shuffles below are executed by all eight lanes or by none
    while (i < total) {
        float4 v[kQuantItems];
        long long row[kQuantItems];
        int c4[kQuantItems];
#pragma unroll
        for (int u = 0; u < kQuantItems; ++u) {
            row[u] = -1;
            if (i < total) {
                row[u] = cur_row;
                c4[u] = cur_c4;
                v[u] = __ldcs(reinterpret_cast<const float4*>(src + cur_row * ld_src) + cur_c4);
            }
            i += stride;
            cur_row += row_step;
            cur_c4 += col_step;
            if (cur_c4 >= k4) {
                cur_c4 -= k4;
                cur_row += 1;
            }
        }
#pragma unroll
        for (int u = 0; u < kQuantItems; ++u) {
            if (row[u] < 0) {
                continue;
            }
            float amax = fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w)));
            amax = fmaxf(amax, __shfl_xor_sync(group_mask, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(group_mask, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(group_mask, amax, 4));
            uint32_t e8m0;
            if constexpr (ALG == MX_SCALE_OCP) {
                const uint32_t exponent = (__float_as_uint(amax) & 0x7F800000u) >> 23;
                e8m0 = exponent <= 8u ? 0u : exponent - 8u;
            } else {
                const uint32_t bits = __float_as_uint(__fmul_rn(amax, 1.0f / 448.0f));
                const uint32_t exponent = (bits & 0x7F800000u) >> 23;
                const uint32_t mantissa = bits & 0x007FFFFFu;
                const bool round_up = mantissa > 0u && !(exponent == 0u && mantissa <= 0x00400000u);
                e8m0 = (amax == 0.0f) ? 0u : exponent + (round_up ? 1u : 0u);
            }
            const float scaling = __uint_as_float((254u - e8m0) << 23); // e8m0 <= 246 for finite input: never zero
            const float y0 = __fmul_rn(v[u].x, scaling), y1 = __fmul_rn(v[u].y, scaling);
            const float y2 = __fmul_rn(v[u].z, scaling), y3 = __fmul_rn(v[u].w, scaling);
            const uint32_t lo = cvt_e4m3x2(y0, y1);
            const uint32_t hi = cvt_e4m3x2(y2, y3);
            uint32_t packed = lo | (hi << 16);
            if constexpr (ALG == MX_SCALE_OCP) {
                packed = drop_negative_zero(packed);
            } else {
                // values below 2^-10 keep their sign as +-0 (what the conversion gives); a value of exactly -2^-10 is a
                // tie that the reference's search resolves to +0
                constexpr float kTie = -0.0009765625f;
                packed &= ~((y0 == kTie ? 0x80u : 0u) | (y1 == kTie ? 0x8000u : 0u) | (y2 == kTie ? 0x800000u : 0u) |
                            (y3 == kTie ? 0x80000000u : 0u));
            }
            *reinterpret_cast<uint32_t*>(data + row[u] * ld_data + static_cast<long long>(c4[u]) * 4) = packed;
            if ((c4[u] & 7) == 0) {
                scales[row[u] * ld_scales + (c4[u] >> 3)] = static_cast<uint8_t>(e8m0);
            }
        }
    }
}

// TQUANT to MXFP4: fp32 [rows][k] -> float4_e2m1x2_t bytes [rows][k / 2] (element 2i in the low nibble) + one e8m0
// scale per 32 elements of K (include/pto/cpu/TQuant.hpp: group maximum ComputeMxGroupMax :280-305, shared exponent
// ComputeE2M1SharedExponent :210-221 / ComputeNvSharedExponent with the e2m1 spec :39-45,:194-208, scaling :226-248,
// element code EncodeE2M1Magic :155-176):
//   OCP: amax = the largest |x| of the block TRUNCATED to bf16; e8m0 = max(biased_exponent(amax) - 2, 0)
//   NV:  e8m0 = biased exponent of amax / 6, plus one unless amax / 6 is a power of two (0 for an all-zero block)
//   scaling = 2^(127 - e8m0); code = sign | magnitude code of |x * scaling| rounded to nearest even on the e2m1 grid
//   (steps of 0.5 below 2, 1 below 4, 2 above; 6 is the largest), the sign kept on a zero as well.
// Inputs must be finite. Same thread layout as the e4m3 kernel: eight lanes own a block, a lane stores two bytes.
// Two floats -> two e2m1 codes in one byte (low nibble = first value): round to nearest even on the e2m1 grid,
// saturating at +-6, the sign kept on zeros - what EncodeE2M1Magic computes with its power-of-two addition.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi)
{
    uint16_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; mov.b16 %0, {t, 0}; }" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// src: [rows][ld_src] floats (16-byte aligned rows); data: [rows][ld_data] bytes (2-byte aligned rows, k / 2 used);
// scales: [rows][ld_scales] bytes. k % 32 == 0.
template <int ALG>
__global__ void __launch_bounds__(kQuantThreads) mx_quantize_e2m1_kernel(const float* __restrict__ src,
                                                                          uint8_t* __restrict__ data,
                                                                          uint8_t* __restrict__ scales, int rows, int k,
                                                                          long long ld_src, long long ld_data,
                                                                          long long ld_scales)
{
    const int k4 = k / 4;
    const long long total = static_cast<long long>(rows) * k4; // 16-byte items; a multiple of 8 per row
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const unsigned group_mask = 0xFFu << (threadIdx.x & 24u);
    const long long row_step = stride / k4;
    const int col_step = static_cast<int>(stride - row_step * k4);
    long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    long long cur_row = i / k4;
    int cur_c4 = static_cast<int>(i - cur_row * k4);
    // total and stride are multiples of 8: the eight lanes of a group are all in range or all out of range
    while (i < total) {
        float4 v[kQuantItems];
        long long row[kQuantItems];
        int c4[kQuantItems];
#pragma unroll
        for (int u = 0; u < kQuantItems; ++u) {
            row[u] = -1;
            if (i < total) {
                row[u] = cur_row;
                c4[u] = cur_c4;
                v[u] = __ldcs(reinterpret_cast<const float4*>(src + cur_row * ld_src) + cur_c4);
            }
            i += stride;
            cur_row += row_step;
            cur_c4 += col_step;
            if (cur_c4 >= k4) {
                cur_c4 -= k4;
                cur_row += 1;
            }
        }
#pragma unroll
        for (int u = 0; u < kQuantItems; ++u) {
            if (row[u] < 0) {
                continue;
            }
            // the maximum as a bit pattern without the sign: for finite floats the integer order is the value order
            uint32_t amax_bits = max(max(__float_as_uint(v[u].x) & 0x7FFFFFFFu, __float_as_uint(v[u].y) & 0x7FFFFFFFu),
                                     max(__float_as_uint(v[u].z) & 0x7FFFFFFFu, __float_as_uint(v[u].w) & 0x7FFFFFFFu));
            amax_bits = max(amax_bits, __shfl_xor_sync(group_mask, amax_bits, 1));
            amax_bits = max(amax_bits, __shfl_xor_sync(group_mask, amax_bits, 2));
            amax_bits = max(amax_bits, __shfl_xor_sync(group_mask, amax_bits, 4));
            uint32_t e8m0;
            if constexpr (ALG == MX_SCALE_OCP) {
                const uint32_t exponent = amax_bits >> 23; // truncation to bf16 keeps the exponent field
                e8m0 = exponent <= 2u ? 0u : exponent - 2u;
            } else {
                const uint32_t bits = __float_as_uint(__fmul_rn(__uint_as_float(amax_bits), 1.0f / 6.0f));
                const uint32_t exponent = (bits & 0x7F800000u) >> 23;
                const uint32_t mantissa = bits & 0x007FFFFFu;
                const bool round_up = mantissa > 0u && !(exponent == 0u && mantissa <= 0x00400000u);
                e8m0 = (amax_bits == 0u) ? 0u : exponent + (round_up ? 1u : 0u);
            }
            const float scaling = __uint_as_float((254u - e8m0) << 23); // e8m0 <= 252 for finite input: never zero
            const uint32_t codes = cvt_e2m1x2(__fmul_rn(v[u].x, scaling), __fmul_rn(v[u].y, scaling)) |
                                   (cvt_e2m1x2(__fmul_rn(v[u].z, scaling), __fmul_rn(v[u].w, scaling)) << 8);
            *reinterpret_cast<uint16_t*>(data + row[u] * ld_data + static_cast<long long>(c4[u]) * 2) =
                static_cast<uint16_t>(codes);
            if ((c4[u] & 7) == 0) {
                scales[row[u] * ld_scales + (c4[u] >> 3)] = static_cast<uint8_t>(e8m0);
            }
        }
    }
}

} // namespace pto_b200
