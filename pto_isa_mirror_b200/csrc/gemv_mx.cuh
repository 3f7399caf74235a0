// TGEMV_MX on sm_100a: one left row against a block-scaled fp8 matrix,
//   out[j] = sum_k a[k] * B[k][j] * 2^(SA[k/32] - 127) * 2^(SB[j][k/32] - 127)   (+ bias[j]).
//
// The reference runs TGEMV_MX through the arithmetic of TMATMUL_MX with a one-row left tile
// (include/pto/cpu/TMatmul.hpp:294-326 -> TMatmulMX :169-205; declarations include/pto/common/pto_instr.hpp:797-862).
// As for TGEMV there is nothing to reuse with one row: every byte of B and of its scales is read once, the bound is
// HBM bandwidth, and a 128-row block-scaled MMA tile would waste 127/128 of its work. One warp per output column
// (a contiguous K-run of the column-major B): each lane takes 16 consecutive fp8 values per 16-byte load - they lie
// inside one 32-element scale block - converts both operands with the hardware fp8 -> half conversion, sums the 16
// products in fp32 and multiplies the partial sum by the two block scales; a shuffle reduction, bias, cast, one store.
//
// Algorithmic bytes per launch: n * k (B) + n * k / 32 (its scales) + k + k / 32 (the row, re-read from L2 by every
// warp) + n * sizeof(out). Summation order differs from the reference's sequential chain: within the MX tolerance,
// exact for integer-valued inputs with power-of-two scales.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <cstdint>

#include "gemv.cuh"

namespace pto_b200 {

// Two fp8 bytes (low 16 bits of `two`) -> two floats.
template <bool E5M2>
__device__ __forceinline__ float2 fp8x2_to_float2(uint32_t two)
{
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two & 0xFFFFu), E5M2 ? __NV_E5M2 : __NV_E4M3);
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// 2^(e - 127) for an e8m0 byte (0 -> 2^-127, a subnormal float; 255 is outside the input domain).
__device__ __forceinline__ float e8m0_to_float(uint32_t e)
{
    return __uint_as_float(e == 0u ? 0x00400000u : (e << 23));
}

// a: [k] fp8 bytes, 16-byte aligned; sa: [k / 32] e8m0 bytes. b: [n][ldb] fp8 bytes (column-major K x N), rows
// 16-byte aligned; sb: [n][ld_sfb] e8m0 bytes. bias: n floats or null. out: [n] floats or bf16. k % 32 == 0.
template <bool A_E5M2, bool B_E5M2, int OUT>
__global__ void __launch_bounds__(kGemvThreads) gemv_mx_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ sa,
                                                               const uint8_t* __restrict__ b, const uint8_t* __restrict__ sb,
                                                               const float* __restrict__ bias, void* __restrict__ out, int n,
                                                               int k, long long ldb, long long ld_sfb)
{
    const int lane = threadIdx.x & 31;
    const int warps_per_block = kGemvThreads / 32;
    const int kv = k / 16; // 16-byte loads per column
    const uint4* av = reinterpret_cast<const uint4*>(a);
    for (long long col = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); col < n;
         col += static_cast<long long>(gridDim.x) * warps_per_block) {
        const uint4* brow = reinterpret_cast<const uint4*>(b + col * ldb);
        const uint8_t* sbrow = sb + col * ld_sfb;
        float acc = 0.0f;
#pragma unroll 2
        for (int i = lane; i < kv; i += 32) {
            const uint4 bv = ld_stream_u4(brow + i);
            const uint4 xv = __ldg(av + i);
            const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
            float part0 = 0.0f, part1 = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 b0 = fp8x2_to_float2<B_E5M2>(bw[w]);
                const float2 b1 = fp8x2_to_float2<B_E5M2>(bw[w] >> 16);
                const float2 x0 = fp8x2_to_float2<A_E5M2>(xw[w]);
                const float2 x1 = fp8x2_to_float2<A_E5M2>(xw[w] >> 16);
                part0 = fmaf(x0.x, b0.x, part0);
                part1 = fmaf(x0.y, b0.y, part1);
                part0 = fmaf(x1.x, b1.x, part0);
                part1 = fmaf(x1.y, b1.y, part1);
            }
            const int group = i >> 1; // 16 values per load, 32 per scale block
            const float scale = e8m0_to_float(__ldg(sa + group)) * e8m0_to_float(__ldg(sbrow + group));
            acc = fmaf(part0 + part1, scale, acc);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
        }
        if (lane == 0) {
            if (bias != nullptr) {
                acc += __ldg(bias + col);
            }
            if constexpr (OUT == GEMV_OUT_F32) {
                static_cast<float*>(out)[col] = acc;
            } else {
                static_cast<__nv_bfloat16*>(out)[col] = __float2bfloat16_rn(acc);
            }
        }
    }
}

} // namespace pto_b200
