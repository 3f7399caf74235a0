// TGEMV_MX on sm_100a: one left row against a block-scaled fp8 matrix,
//   out[j] = sum_k a[k] * B[k][j] * 2^(SA[k/32] - 127) * 2^(SB[j][k/32] - 127)   (+ bias[j]).
//
// The reference runs TGEMV_MX through the arithmetic of TMATMUL_MX with a one-row left tile
// (include/pto/cpu/TMatmul.hpp:294-326 -> TMatmulMX :169-205; declarations include/pto/common/pto_instr.hpp:797-862).
// As for TGEMV there is nothing to reuse with one row: every byte of B and of its scales is read once and the bound is
// HBM bandwidth - provided the fp8 bytes become floats cheaply enough. A first version converted the matrix AND the
// left row in every warp and stopped at 0.59 of the copy bandwidth.
//
// gemv_mx_kernel (K up to kGemvMxSmemK): the block converts the left row once into shared memory as floats (laid out so
// that a warp's 16-byte reads are conflict-free) together with its block scales; after that only the matrix bytes are
// converted. One warp per output column (a contiguous K-run of the column-major B): each lane takes 16 consecutive fp8
// values per 16-byte load - they lie inside one 32-element scale block - sums the 16 products in fp32 and multiplies
// the partial sum by the two block scales; a shuffle reduction, bias, cast, one store. 0.64-0.66 of the copy
// bandwidth on a 32768 x 8192 matrix (64.5 us). Tried on the same matrix and slower or equal: the matrix bytes turned
// into scaled floats with integer shifts and masks instead of conversion instructions (71.5 us), half of them each way
// (65.5 us), the left row in registers with K cut over the warps of a block (83-90 us), four loads in flight per lane
// instead of two (75 us).
//
// gemv_mx_mma_kernel (any K): no shared memory and no conversion at all: the 32 products of a scale block are formed
// by a warp-level fp8 MMA (mma.sync m16n8k32, fp32 accumulate) straight from the bytes. The MMA's 16 x 32 row operand
// holds eight consecutive scale blocks (256 contiguous bytes) of one column of B in rows 0-7 and of the next column in
// rows 8-15; its 32 x 8 column operand holds the same eight blocks of the left row, one block per column. The
// products wanted are the diagonal ones, D[g][g] and D[g+8][g]; each is multiplied by its two block scales and added
// in fp32. This warp-level fp8 MMA issues slowly on this GPU (measured 3.1 TB/s, below the conversion kernel), so it
// serves the rows too long for shared memory.
//
// Algorithmic bytes per launch: n * k (B) + n * k / 32 (its scales) + k + k / 32 (the row) + n * sizeof(out).
// Summation order differs from the reference's sequential chain: within the MX tolerance, exact for integer-valued
// inputs with power-of-two scales.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <cstdint>

#include "gemv.cuh"

namespace pto_b200 {

// 2^(e - 127) for an e8m0 byte (0 -> 2^-127, a subnormal float; 255 is outside the input domain).
__device__ __forceinline__ float e8m0_to_float(uint32_t e)
{
    return __uint_as_float(e == 0u ? 0x00400000u : (e << 23));
}

// Eight bytes of a row of B, read once: kept out of L1 so that the left row and the scales stay cached there.
__device__ __forceinline__ uint2 ld_stream_u2(const void* ptr)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr));
    return v;
}

// D (16 x 8, fp32) = A (16 x 32 fp8, row-major fragment) * B (32 x 8 fp8, column fragment), accumulator zero.
// Thread (g = lane / 4, t = lane % 4) holds A[g][4t..4t+3], A[g+8][4t..], A[g][16+4t..], A[g+8][16+4t..] and
// B[4t..4t+3][g], B[16+4t..][g]; it receives D[g][2t], D[g][2t+1], D[g+8][2t], D[g+8][2t+1].
template <bool A_E5M2, bool B_E5M2>
__device__ __forceinline__ void mma_fp8_16x8x32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1)
{
    d[0] = d[1] = d[2] = d[3] = 0.0f;
    if constexpr (!A_E5M2 && !B_E5M2) {
        asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else if constexpr (!A_E5M2 && B_E5M2) {
        asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e5m2.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else if constexpr (A_E5M2 && !B_E5M2) {
        asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e5m2.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e5m2.e5m2.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

constexpr int kGemvMxColsPerWarp = 2;

// a: [k] fp8 bytes, 16-byte aligned; sa: [k / 32] e8m0 bytes. b: [n][ldb] fp8 bytes (column-major K x N), rows
// 16-byte aligned; sb: [n][ld_sfb] e8m0 bytes. bias: n floats or null. out: [n] floats or bf16. k % 32 == 0.
// A_E5M2 / B_E5M2 name the left row's and the matrix's format; the matrix is the MMA's row operand.
template <bool A_E5M2, bool B_E5M2, int OUT>
__global__ void __launch_bounds__(kGemvThreads) gemv_mx_mma_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ sa,
                                                               const uint8_t* __restrict__ b, const uint8_t* __restrict__ sb,
                                                               const float* __restrict__ bias, void* __restrict__ out, int n,
                                                               int k, long long ldb, long long ld_sfb)
{
    constexpr int kWarps = kGemvThreads / 32;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2; // MMA row group: scale block g of the eight this step covers
    const int t = lane & 3;  // bytes 8t..8t+7 of that block
    const int k_blocks = k / 32;
    const bool diagonal = (t == (g >> 1)); // this thread receives D[g][g] (register g & 1) and D[g+8][g]
    const long long pairs = (static_cast<long long>(n) + 1) / 2;
    for (long long pair = static_cast<long long>(blockIdx.x) * kWarps + warp; pair < pairs;
         pair += static_cast<long long>(gridDim.x) * kWarps) {
        const long long c0 = pair * 2;
        const long long c1 = (c0 + 1 < n) ? c0 + 1 : c0; // an odd n: the last column twice, the second sum dropped
        const uint8_t* b0 = b + c0 * ldb + 8 * lane;     // lane 4g + t: block g, bytes 8t.. -> 256 contiguous bytes
        const uint8_t* b1 = b + c1 * ldb + 8 * lane;
        const uint8_t* xs = a + 8 * lane;
        const uint8_t* s0 = sb + c0 * ld_sfb + g;
        const uint8_t* s1 = sb + c1 * ld_sfb + g;
        const uint8_t* sx = sa + g;
        float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll 4
        for (int blk0 = 0; blk0 < k_blocks; blk0 += 8) {
            uint2 m0 = make_uint2(0u, 0u), m1 = make_uint2(0u, 0u), xv = make_uint2(0u, 0u);
            uint32_t e0 = 127u, e1 = 127u, ex = 127u;
            if (blk0 + g < k_blocks) { // past the end of K: zero operands
                m0 = ld_stream_u2(b0 + blk0 * 32);
                m1 = ld_stream_u2(b1 + blk0 * 32);
                xv = __ldg(reinterpret_cast<const uint2*>(xs + blk0 * 32));
                e0 = __ldg(s0 + blk0);
                e1 = __ldg(s1 + blk0);
                ex = __ldg(sx + blk0);
            }
            float d[4];
            mma_fp8_16x8x32<B_E5M2, A_E5M2>(d, m0.x, m1.x, m0.y, m1.y, xv.x, xv.y);
            const float scale_x = e8m0_to_float(ex);
            acc0 = fmaf((g & 1) ? d[1] : d[0], scale_x * e8m0_to_float(e0), acc0);
            acc1 = fmaf((g & 1) ? d[3] : d[2], scale_x * e8m0_to_float(e1), acc1);
        }
        acc0 = diagonal ? acc0 : 0.0f;
        acc1 = diagonal ? acc1 : 0.0f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            acc0 += __shfl_xor_sync(0xFFFFFFFFu, acc0, off);
            acc1 += __shfl_xor_sync(0xFFFFFFFFu, acc1, off);
        }
        if (lane < 2 && c0 + lane < n) {
            float acc = lane == 0 ? acc0 : acc1;
            const long long col = c0 + lane;
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

// Two fp8 bytes (low 16 bits of `two`) -> two floats, through the conversion instructions.
template <bool E5M2>
__device__ __forceinline__ float2 fp8x2_to_float2(uint32_t two)
{
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two & 0xFFFFu), E5M2 ? __NV_E5M2 : __NV_E4M3);
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

constexpr int kGemvMxSmemK = 40960; // longest left row kept in shared memory: 160 KiB of floats + 5 KiB of scales

// Position (in float4 units) of the j-th float4 of the 16-value group q of the left row: the 32 lanes of a warp read
// groups q = 32 c + lane, so for a fixed j their float4s are consecutive.
__device__ __forceinline__ int gemv_mx_x_slot(int q, int j) { return ((q >> 5) * 4 + j) * 32 + (q & 31); }

// Same operands as gemv_mx_mma_kernel; dynamic shared memory: ceil(k / 512) * 512 floats + k / 32 floats.
template <bool A_E5M2, bool B_E5M2, int OUT>
__global__ void __launch_bounds__(kGemvThreads) gemv_mx_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ sa,
                                                               const uint8_t* __restrict__ b, const uint8_t* __restrict__ sb,
                                                               const float* __restrict__ bias, void* __restrict__ out, int n,
                                                               int k, long long ldb, long long ld_sfb)
{
    extern __shared__ float4 gemv_mx_smem[];
    float4* x4 = gemv_mx_smem;                                             // the left row as floats, slot order
    float* sx = reinterpret_cast<float*>(gemv_mx_smem + ((k + 511) / 512) * 128); // 2^(SA - 127) per scale block
    for (int w = threadIdx.x; w < k / 4; w += kGemvThreads) {              // four values per thread and step
        const uint32_t four = __ldg(reinterpret_cast<const uint32_t*>(a) + w);
        const float2 lo = fp8x2_to_float2<A_E5M2>(four);
        const float2 hi = fp8x2_to_float2<A_E5M2>(four >> 16);
        x4[gemv_mx_x_slot(w >> 2, w & 3)] = make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    for (int g = threadIdx.x; g < k / 32; g += kGemvThreads) {
        sx[g] = e8m0_to_float(__ldg(sa + g));
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warps_per_block = kGemvThreads / 32;
    const int kv = k / 16; // 16-byte loads per column
    for (long long col = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); col < n;
         col += static_cast<long long>(gridDim.x) * warps_per_block) {
        const uint4* brow = reinterpret_cast<const uint4*>(b + col * ldb);
        const uint8_t* sbrow = sb + col * ld_sfb;
        float acc = 0.0f;
#pragma unroll 2
        for (int i = lane; i < kv; i += 32) {
            const uint4 bv = ld_stream_u4(brow + i);
            const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
            float part0 = 0.0f, part1 = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float4 x = x4[gemv_mx_x_slot(i, w)];
                const float2 m0 = fp8x2_to_float2<B_E5M2>(bw[w]);
                const float2 m1 = fp8x2_to_float2<B_E5M2>(bw[w] >> 16);
                part0 = fmaf(x.x, m0.x, part0);
                part1 = fmaf(x.y, m0.y, part1);
                part0 = fmaf(x.z, m1.x, part0);
                part1 = fmaf(x.w, m1.y, part1);
            }
            const int group = i >> 1; // 16 values per load, 32 per scale block
            const float part = part0 + part1;
            acc = fmaf(part, sx[group] * e8m0_to_float(__ldg(sbrow + group)), acc);
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
