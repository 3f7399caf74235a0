// TGEMV on sm_100a: out[j] = sum_k a[k] * B[k][j] (+ bias[j]) for one left row (m = 1).
//
// The reference runs TGEMV / TGEMV_ACC / TGEMV_BIAS through the same arithmetic as TMATMUL with a one-row left
// tile (include/pto/cpu/TMatmul.hpp:232-252; declarations include/pto/common/pto_instr.hpp:1019-1060). With one
// row there is nothing to reuse: every byte of B is read once and used once, so the bound is HBM bandwidth, not the
// tensor pipe, and a 128-row MMA tile would waste 127/128 of its work. This kernel therefore streams B with plain
// 16-byte loads: one warp per output column (a contiguous K-run of the column-major B), lanes striding over K,
// fp32 (int32 for int8) partial sums per lane, a shuffle reduction, then bias, cast and one store.
//
// Algorithmic bytes per launch: n * k * sizeof(element) (B) + k * sizeof(element) (a, re-read from L2 by every
// warp) + n * sizeof(out). Summation order differs from the reference's sequential chain (32 lane partials, tree
// reduced): exact for int8, within the dense tolerance for 16-bit inputs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace pto_b200 {

enum GemvIn : int { GEMV_F16 = 0, GEMV_BF16 = 1, GEMV_S8 = 2 };
enum GemvOut : int { GEMV_OUT_F32 = 0, GEMV_OUT_BF16 = 1, GEMV_OUT_F16 = 2, GEMV_OUT_S32 = 3 };

constexpr int kGemvThreads = 256;

// B is read exactly once: keep it out of L1 so that the left row stays cached there.
__device__ __forceinline__ uint4 ld_stream_u4(const uint4* ptr)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
    return v;
}

template <int IN>
__device__ __forceinline__ float2 unpack2(uint32_t u)
{
    if constexpr (IN == GEMV_BF16) {
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
    } else {
        return __half22float2(*reinterpret_cast<const __half2*>(&u));
    }
}

template <int IN>
__device__ __forceinline__ float scalar_to_float(const void* base, long long idx)
{
    if constexpr (IN == GEMV_BF16) {
        return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    } else {
        return __half2float(static_cast<const __half*>(base)[idx]);
    }
}

// a: [k] elements, 16-byte aligned. b: [n][ldb] elements (column-major K x N), rows 16-byte aligned.
// bias: n values of the accumulator type or null. out: [n] of the OUT type.
// At most 32 registers per thread: eight 256-thread blocks per SM, so that 8192 columns (1024 blocks) are all
// resident at once on 148 SMs instead of running as one full wave and a 38 % wave.
template <int IN, int OUT>
__global__ void __launch_bounds__(kGemvThreads, 8) gemv_kernel(const void* __restrict__ a, const void* __restrict__ b,
                                                             const void* __restrict__ bias, void* __restrict__ out,
                                                             int n, int k, long long ldb)
{
    constexpr int kElemBytes = (IN == GEMV_S8) ? 1 : 2;
    constexpr int kVec = 16 / kElemBytes; // elements per 16-byte load
    const int lane = threadIdx.x & 31;
    const int warps_per_block = kGemvThreads / 32;
    const int kv = k / kVec;
    const uint4* av = static_cast<const uint4*>(a);
    for (long long col = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); col < n;
         col += static_cast<long long>(gridDim.x) * warps_per_block) {
        const char* brow_bytes = static_cast<const char*>(b) + col * ldb * kElemBytes;
        const uint4* brow = reinterpret_cast<const uint4*>(brow_bytes);
        if constexpr (IN == GEMV_S8) {
            int acc0 = 0, acc1 = 0;
#pragma unroll 2
            for (int i = lane; i < kv; i += 32) {
                const uint4 bv = ld_stream_u4(brow + i);
                const uint4 xv = __ldg(av + i);
                acc0 = __dp4a(static_cast<int>(xv.x), static_cast<int>(bv.x), acc0);
                acc1 = __dp4a(static_cast<int>(xv.y), static_cast<int>(bv.y), acc1);
                acc0 = __dp4a(static_cast<int>(xv.z), static_cast<int>(bv.z), acc0);
                acc1 = __dp4a(static_cast<int>(xv.w), static_cast<int>(bv.w), acc1);
            }
            int acc = acc0 + acc1;
            for (int kk = kv * kVec + lane; kk < k; kk += 32) {
                acc += static_cast<int>(static_cast<const int8_t*>(a)[kk]) *
                       static_cast<int>(reinterpret_cast<const int8_t*>(brow_bytes)[kk]);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
            }
            if (lane == 0) {
                if (bias != nullptr) {
                    acc = static_cast<int>(static_cast<uint32_t>(acc) +
                                           static_cast<uint32_t>(__ldg(static_cast<const int*>(bias) + col)));
                }
                static_cast<int*>(out)[col] = acc;
            }
        } else {
            float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll 2
            for (int i = lane; i < kv; i += 32) {
                const uint4 bv = ld_stream_u4(brow + i);
                const uint4 xv = __ldg(av + i);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float2 bf = unpack2<IN>(bw[w]);
                    const float2 xf = unpack2<IN>(xw[w]);
                    acc0 = fmaf(xf.x, bf.x, acc0);
                    acc1 = fmaf(xf.y, bf.y, acc1);
                }
            }
            float acc = acc0 + acc1;
            for (int kk = kv * kVec + lane; kk < k; kk += 32) {
                acc = fmaf(scalar_to_float<IN>(a, kk), scalar_to_float<IN>(brow_bytes, kk), acc);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
            }
            if (lane == 0) {
                if (bias != nullptr) {
                    acc += __ldg(static_cast<const float*>(bias) + col);
                }
                if constexpr (OUT == GEMV_OUT_F32) {
                    static_cast<float*>(out)[col] = acc;
                } else if constexpr (OUT == GEMV_OUT_BF16) {
                    static_cast<__nv_bfloat16*>(out)[col] = __float2bfloat16_rn(acc);
                } else {
                    static_cast<__half*>(out)[col] = __float2half_rn(acc);
                }
            }
        }
    }
}

} // namespace pto_b200
