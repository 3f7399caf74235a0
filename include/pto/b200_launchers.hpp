// b200_launchers.hpp - the reference's GEMM launcher functions, with their exact signatures, over the B200 C ABI.
//
//   LaunchGEMME2E<T>    kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:250-273 (decl main.cpp:16-17)
//   LaunchMxMatmul      kernels/manual/a5/matmul_mxfp8_performance/mxmatmul_performance_kernel.cpp:361-380
//   launchGemmCompute   kernels/manual/a2a3/gemm_ar/gemm_compute_kernel.cpp:254-259
// The reference fixes the problem size in template constants of each launcher; the same constants are the defaults
// here and a GemmShape argument overrides them at run time. All pointers are device pointers; `stream` is a
// cudaStream_t. Launchers return void like the reference's; a rejected launch is reported through pto::b200::fail.
#ifndef PTO_B200_LAUNCHERS_HPP
#define PTO_B200_LAUNCHERS_HPP

#include "pto-inst.hpp"

namespace pto {
namespace b200 {
struct GemmShape {
    int m, n, k;
};
} // namespace b200
} // namespace pto

// fp16 x fp16 -> fp32, A [m, k] row-major, B column-major (stored [n, k]); T = uint16_t as in the reference.
template <typename T>
inline void LaunchGEMME2E(uint8_t* out, uint8_t* src0, uint8_t* src1, void* stream,
                          pto::b200::GemmShape shape = {6144, 6144, 6144})
{
    static_assert(sizeof(T) == 2, "LaunchGEMME2E is instantiated for 16-bit inputs (uint16_t in the reference)");
    const int rc = pto_b200_gemm(stream, out, src0, src1, shape.m, shape.n, shape.k, shape.k, shape.k, shape.n,
                                 PTO_B200_F16, PTO_B200_F32, PTO_B200_B_DN);
    if (rc != PTO_B200_OK) {
        pto::b200::fail("LaunchGEMME2E", rc);
    }
}

// e5m2 x e5m2 with e8m0 scales (src2: [m, k/32], src3: [n, k/32]) -> bf16. Six arguments as in the reference:
// the scale re-tiling scratch is the library's built-in array (pto_b200_gemm_mx_static). The MXFP4 kernel of the same
// name (kernels/manual/a5/matmul_mxfp4_performance/mxmatmul_performance_kernel.cpp:446-463: float4_e2m1x2_t operands,
// two per byte, 2040 x 8100 x 8192) is this call with operand_dtype = PTO_B200_E2M1 and shape {2040, 8100, 8192}.
inline void LaunchMxMatmul(uint8_t* out, uint8_t* src0, uint8_t* src1, uint8_t* src2, uint8_t* src3, void* stream,
                           pto::b200::GemmShape shape = {6144, 6144, 6144}, int operand_dtype = PTO_B200_E5M2)
{
    const int rc = pto_b200_gemm_mx_static(stream, out, src0, src1, src2, src3, shape.m, shape.n, shape.k, shape.k,
                                           shape.k, shape.n, shape.k / 32, shape.k / 32, operand_dtype, operand_dtype,
                                           PTO_B200_BF16);
    if (rc != PTO_B200_OK) {
        pto::b200::fail("LaunchMxMatmul", rc);
    }
}

// Per-rank GEMM of the GEMM + allreduce pipeline: src0 [m, k_per_rank] and src1 [n, k_per_rank] are this rank's
// packed K slices, gemm_output [m, n] is fp16 as in the reference. launch_block_count caps the thread blocks (SMs) the
// GEMM occupies, as it caps the cores in the reference (0 = all). queue_set and rank belong to the reference's
// device-side tile queue and are not used: completion is stream-ordered.
inline void launchGemmCompute(uint8_t* gemm_output, uint8_t* src0, uint8_t* src1, uint8_t* queue_set, int rank,
                              void* stream, int launch_block_count, uint32_t k_per_rank,
                              pto::b200::GemmShape shape = {5416, 1408, 6144}, int out_dtype = PTO_B200_F16)
{
    (void)queue_set;
    (void)rank;
    const int k = static_cast<int>(k_per_rank);
    const int rc = pto_b200_gemm_ex(stream, gemm_output, src0, src1, shape.m, shape.n, k, k, k, shape.n, PTO_B200_F16,
                                    out_dtype, PTO_B200_B_DN, launch_block_count > 0 ? launch_block_count : 0);
    if (rc != PTO_B200_OK) {
        pto::b200::fail("launchGemmCompute", rc);
    }
}

#endif // PTO_B200_LAUNCHERS_HPP
