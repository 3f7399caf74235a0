// gemm_tile_program.cpp - the reference's GEMM tile programs written against include/pto/pto-inst.hpp and run
// on a B200: (1) the CPU demo's TLOAD / TMOV / TMATMUL / TSTORE sequence (demos/cpu/gemm_demo/gemm_demo.cpp:83-121,
// B row-major), (2) the gemm_performance K loop with TEXTRACT slices and TMATMUL / TMATMUL_ACC
// (kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:69-131, B column-major), (3) the fixed-signature
// launcher, (4) the bias form of the K loop (TMATMUL_BIAS then TMATMUL_ACC, tests/cpu/st/testcase/tmatmul/
// tmatmul_kernel.cpp:86-96), (5) a one-row TGEMV_BIAS, (6) the int8 K loop stored with a per-column scaling tile
// (TSTORE_FP), with one pre-quant scalar plus ReLU and requantised to int8 (kernels/manual/a2a3/dispatch_mega_combine/op_kernel/utils/
// pto_gmm_preload_async_fixpipe_quant.hpp:75-124), (7) the block-scaled K loop with MX_A_ND / MX_B_DN scale tensors
// (kernels/manual/a5/matmul_mxfp8_performance/mxmatmul_performance_kernel.cpp:153-344), (8) LaunchMxMatmul on e5m2
// operands and (9) on float4_e2m1x2_t operands, two per byte (kernels/manual/a5/matmul_mxfp4_performance). Inputs are small integers so the fp32 results are exact; the program checks them against host loops and
// prints "tile programs ok".
//
// Build (one line): g++ -std=c++17 -I include -I /usr/local/cuda/include examples/gemm_tile_program.cpp
//   -L pto_isa_mirror_b200/lib -lpto_b200 -L /usr/local/cuda/lib64 -lcudart -o examples/gemm_tile_program
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include <cuda_runtime.h>

#include "pto/b200_launchers.hpp"

using namespace pto;

static uint16_t f32_to_f16_small_int(int v)
{ // exact for |v| <= 2048
    if (v == 0) return 0;
    uint16_t sign = v < 0 ? 0x8000 : 0;
    unsigned a = v < 0 ? -v : v;
    int e = 0;
    while ((a >> (e + 1)) != 0) ++e;
    unsigned man = (a << (10 - e)) & 0x3FF;
    return sign | static_cast<uint16_t>((e + 15) << 10) | static_cast<uint16_t>(man);
}

static uint16_t f32_to_bf16_rne(float f)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}

// small integers |v| <= 4 as fp8: e4m3 (bias 7, 3 mantissa bits) and e5m2 (bias 15, 2 mantissa bits)
static uint8_t int_to_e4m3(int v)
{
    static const uint8_t mag[5] = {0x00, 0x38, 0x40, 0x44, 0x48};
    return static_cast<uint8_t>((v < 0 ? 0x80 : 0) | mag[v < 0 ? -v : v]);
}
static uint8_t int_to_e5m2(int v)
{
    static const uint8_t mag[5] = {0x00, 0x3C, 0x40, 0x42, 0x44};
    return static_cast<uint8_t>((v < 0 ? 0x80 : 0) | mag[v < 0 ? -v : v]);
}
static uint8_t int_to_e2m1(int v)
{ // 4-bit codes of 0, 1, 2, 3, 4
    static const uint8_t mag[5] = {0x0, 0x2, 0x4, 0x5, 0x6};
    return static_cast<uint8_t>((v < 0 ? 0x8 : 0) | mag[v < 0 ? -v : v]);
}

template <typename T>
static T* to_device(const std::vector<T>& h)
{
    T* d = nullptr;
    cudaMalloc(&d, h.size() * sizeof(T));
    cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}

int main()
{
    constexpr int M = 128, K = 256, N = 256, baseK = 64;
    std::vector<int> ai(M * K), bi(K * N);
    for (int i = 0; i < M * K; ++i) ai[i] = (i * 7 + 3) % 9 - 4;
    for (int i = 0; i < K * N; ++i) bi[i] = (i * 5 + 1) % 7 - 3;
    std::vector<float> ref(M * N, 0.f);
    for (int i = 0; i < M; ++i)
        for (int k = 0; k < K; ++k)
            for (int j = 0; j < N; ++j) ref[i * N + j] += static_cast<float>(ai[i * K + k] * bi[k * N + j]);

    std::vector<uint16_t> a16(M * K), b_nd(K * N), b_dn(N * K);
    for (int i = 0; i < M * K; ++i) a16[i] = f32_to_f16_small_int(ai[i]);
    for (int k = 0; k < K; ++k)
        for (int j = 0; j < N; ++j) {
            b_nd[k * N + j] = f32_to_f16_small_int(bi[k * N + j]);
            b_dn[j * K + k] = b_nd[k * N + j];
        }
    half* dA = reinterpret_cast<half*>(to_device(a16));
    half* dBnd = reinterpret_cast<half*>(to_device(b_nd));
    half* dBdn = reinterpret_cast<half*>(to_device(b_dn));
    float* dC = nullptr;
    cudaMalloc(&dC, M * N * sizeof(float));
    std::vector<float> out(M * N);
    int bad = 0;
    auto check = [&](const char* what) {
        cudaDeviceSynchronize();
        cudaMemcpy(out.data(), dC, out.size() * sizeof(float), cudaMemcpyDeviceToHost);
        int n = 0;
        for (size_t i = 0; i < out.size(); ++i) n += (out[i] != ref[i]);
        std::printf("%s: %d mismatches\n", what, n);
        bad += n;
        cudaMemset(dC, 0, M * N * sizeof(float));
    };

    { // (1) the CPU demo's program, B row-major
        using GlobalA = GlobalTensor<half, Shape<1, 1, 1, M, K>, Stride<M * K, M * K, M * K, K, 1>>;
        using GlobalB = GlobalTensor<half, Shape<1, 1, 1, K, N>, Stride<K * N, K * N, K * N, N, 1>>;
        using GlobalC = GlobalTensor<float, Shape<1, 1, 1, M, N>, Stride<M * N, M * N, M * N, N, 1>>;
        GlobalA aGlobal(dA);
        GlobalB bGlobal(dBnd);
        GlobalC cGlobal(dC);
        using TileMatA = Tile<TileType::Mat, half, M, K, BLayout::ColMajor, M, K, SLayout::RowMajor, 512>;
        using TileMatB = Tile<TileType::Mat, half, K, N, BLayout::ColMajor, K, N, SLayout::RowMajor, 512>;
        TileMatA aMat;
        TileMatB bMat;
        TileLeft<half, M, K, M, K> aTile;
        TileRight<half, K, N, K, N> bTile;
        TileAcc<float, M, N, M, N> cTile;
        TASSIGN(aMat, 0x0);
        TASSIGN(bMat, 0x10000);
        TLOAD(aMat, aGlobal);
        TLOAD(bMat, bGlobal);
        TMOV(aTile, aMat);
        TMOV(bTile, bMat);
        TMATMUL(cTile, aTile, bTile);
        TSTORE(cGlobal, cTile);
        check("demo program (TLOAD/TMOV/TMATMUL/TSTORE, B row-major)");
    }
    { // (2) the gemm_performance K loop, B column-major, stepK = 2 panels sliced with TEXTRACT
        constexpr int stepK = 2;
        using GlobalDataSrcA = GlobalTensor<half, TileShape2D<half, M, baseK * stepK, Layout::ND>,
                                            BaseShape2D<half, M, K, Layout::ND>, Layout::ND>;
        using GlobalDataSrcB = GlobalTensor<half, TileShape2D<half, baseK * stepK, N, Layout::DN>,
                                            BaseShape2D<half, K, N, Layout::DN>, Layout::DN>;
        using GlobalDataOut = GlobalTensor<float, TileShape2D<float, M, N, Layout::ND>, BaseShape2D<float, M, N, Layout::ND>,
                                           Layout::ND>;
        using TileMatA = Tile<TileType::Mat, half, M, baseK * stepK, BLayout::ColMajor, M, baseK * stepK, SLayout::RowMajor>;
        using TileMatB = Tile<TileType::Mat, half, baseK * stepK, N, BLayout::RowMajor, baseK * stepK, N, SLayout::ColMajor>;
        TileMatA aMatTile[2];
        TileMatB bMatTile[2];
        TileLeft<half, M, baseK, M, baseK> aTile[2];
        TileRight<half, baseK, N, baseK, N> bTile[2];
        TileAcc<float, M, N, M, N> cTile;
        int db = 0;
        for (int kIter = 0; kIter < K / baseK; ++kIter) {
            if (kIter % stepK == 0) {
                GlobalDataSrcA gmA(dA + kIter * baseK);
                GlobalDataSrcB gmB(dBdn + kIter * baseK);
                TLOAD(aMatTile[db], gmA);
                TLOAD(bMatTile[db], gmB);
                db ^= 1;
            }
            const int cur = db ^ 1;
            TEXTRACT(aTile[kIter & 1], aMatTile[cur], 0, (kIter % stepK) * baseK);
            TEXTRACT(bTile[kIter & 1], bMatTile[cur], (kIter % stepK) * baseK, 0);
            if (kIter == 0) {
                TMATMUL(cTile, aTile[kIter & 1], bTile[kIter & 1]);
            } else {
                TMATMUL_ACC(cTile, cTile, aTile[kIter & 1], bTile[kIter & 1]);
            }
        }
        GlobalDataOut dstGlobal(dC);
        TSTORE(dstGlobal, cTile);
        check("gemm_performance K loop (TEXTRACT/TMATMUL/TMATMUL_ACC, B column-major)");
    }
    { // (3) the launcher with the reference's signature (run-time shape instead of 6144^3)
        LaunchGEMME2E<uint16_t>(reinterpret_cast<uint8_t*>(dC), reinterpret_cast<uint8_t*>(dA),
                                reinterpret_cast<uint8_t*>(dBdn), nullptr, {M, N, K});
        check("LaunchGEMME2E<uint16_t>");
    }
    { // (4) TMATMUL_BIAS on the first K chunk, TMATMUL_ACC on the rest (tests/cpu/st/testcase/tmatmul bias cases)
        std::vector<float> bias(N);
        for (int j = 0; j < N; ++j) bias[j] = static_cast<float>((j * 3) % 11 - 5);
        float* dBias = to_device(bias);
        for (int i = 0; i < M; ++i)
            for (int j = 0; j < N; ++j) ref[i * N + j] += bias[j];
        using GlobalA = GlobalTensor<half, TileShape2D<half, M, baseK, Layout::ND>, BaseShape2D<half, M, K, Layout::ND>>;
        using GlobalB = GlobalTensor<half, TileShape2D<half, baseK, N, Layout::DN>, BaseShape2D<half, K, N, Layout::DN>,
                                     Layout::DN>;
        using GlobalBias = GlobalTensor<float, Shape<1, 1, 1, 1, N>, Stride<N, N, N, N, 1>>;
        using GlobalC = GlobalTensor<float, Shape<1, 1, 1, M, N>, Stride<M * N, M * N, M * N, N, 1>>;
        TileLeft<half, M, baseK, M, baseK> aTile;
        TileRight<half, baseK, N, baseK, N> bTile;
        TileAcc<float, M, N, M, N> cTile;
        Tile<TileType::Bias, float, 1, N, BLayout::RowMajor, 1, N> biasTile;
        GlobalBias biasGlobal(dBias);
        TLOAD(biasTile, biasGlobal);
        for (int kIter = 0; kIter < K / baseK; ++kIter) {
            GlobalA gmA(dA + kIter * baseK);
            GlobalB gmB(dBdn + kIter * baseK);
            TLOAD(aTile, gmA);
            TLOAD(bTile, gmB);
            if (kIter == 0) {
                TMATMUL_BIAS(cTile, aTile, bTile, biasTile);
            } else {
                TMATMUL_ACC(cTile, cTile, aTile, bTile);
            }
        }
        GlobalC cGlobal(dC);
        TSTORE(cGlobal, cTile);
        check("bias program (TMATMUL_BIAS/TMATMUL_ACC, B column-major)");
        { // (5) TGEMV_BIAS: the first row alone, streamed without tensor-core tiles; compare with row 0 of (4)
            using GlobalRow = GlobalTensor<half, Shape<1, 1, 1, 1, K>, Stride<K, K, K, K, 1>>;
            using GlobalMatB = GlobalTensor<half, TileShape2D<half, K, N, Layout::DN>, BaseShape2D<half, K, N, Layout::DN>,
                                            Layout::DN>;
            using GlobalRowOut = GlobalTensor<float, Shape<1, 1, 1, 1, N>, Stride<N, N, N, N, 1>>;
            TileLeft<half, 1, K, 1, K> xTile;
            TileRight<half, K, N, K, N> wTile;
            TileAcc<float, 1, N, 1, N> yTile;
            GlobalRow xGlobal(dA);
            GlobalMatB wGlobal(dBdn);
            GlobalRowOut yGlobal(dC);
            TLOAD(xTile, xGlobal);
            TLOAD(wTile, wGlobal);
            TGEMV_BIAS(yTile, xTile, wTile, biasTile);
            TSTORE(yGlobal, yTile);
            cudaDeviceSynchronize();
            cudaMemcpy(out.data(), dC, N * sizeof(float), cudaMemcpyDeviceToHost);
            int n = 0;
            for (int j = 0; j < N; ++j) n += (out[j] != ref[j]);
            std::printf("one-row program (TGEMV_BIAS): %d mismatches\n", n);
            bad += n;
        }
        cudaFree(dBias);
    }
    { // (6) int8 K loop, stored through the fixpipe quant forms: per-column scaling tile, then one scalar with ReLU
        std::vector<int8_t> a8(M * K), b8(N * K);
        std::vector<int> acc(M * N, 0);
        for (int i = 0; i < M * K; ++i) a8[i] = static_cast<int8_t>(ai[i] * 9);
        for (int k = 0; k < K; ++k)
            for (int j = 0; j < N; ++j) b8[j * K + k] = static_cast<int8_t>(bi[k * N + j] * 11);
        for (int i = 0; i < M; ++i)
            for (int k = 0; k < K; ++k)
                for (int j = 0; j < N; ++j) acc[i * N + j] += static_cast<int>(a8[i * K + k]) * b8[j * K + k];
        // scale words: fp32 bits in [31:0]; the vector form reads [31:13], so these values carry low mantissa bits
        std::vector<uint64_t> words(N);
        std::vector<float> col_scale(N);
        for (int j = 0; j < N; ++j) {
            const float sc = 0.001f * static_cast<float>(1 + j % 7) * (j % 5 == 0 ? -1.0f : 1.0f);
            uint32_t bits;
            std::memcpy(&bits, &sc, 4);
            words[j] = bits;
            bits &= 0xFFFFE000u;
            std::memcpy(&col_scale[j], &bits, 4);
        }
        const float scalar = 0.00314159f;
        uint32_t scalar_bits;
        std::memcpy(&scalar_bits, &scalar, 4);
        int8_t* dA8 = to_device(a8);
        int8_t* dB8 = to_device(b8);
        uint64_t* dWords = to_device(words);
        uint16_t* dOut16 = nullptr;
        cudaMalloc(&dOut16, M * N * sizeof(uint16_t));
        using GlobalA = GlobalTensor<int8_t, TileShape2D<int8_t, M, baseK, Layout::ND>, BaseShape2D<int8_t, M, K, Layout::ND>>;
        using GlobalB = GlobalTensor<int8_t, TileShape2D<int8_t, baseK, N, Layout::DN>, BaseShape2D<int8_t, K, N, Layout::DN>,
                                     Layout::DN>;
        using GlobalOut = GlobalTensor<bfloat16_t, Shape<1, 1, 1, M, N>, Stride<M * N, M * N, M * N, N, 1>>;
        using GlobalScale = GlobalTensor<uint64_t, Shape<1, 1, 1, 1, N>, Stride<N, N, N, N, 1>>;
        using ScaleMatTile = Tile<TileType::Mat, uint64_t, 1, N, BLayout::RowMajor, 1, N, SLayout::NoneBox>;
        using ScalingTile = Tile<TileType::Scaling, uint64_t, 1, N, BLayout::RowMajor, 1, N, SLayout::NoneBox>;
        using AccTile = TileAcc<int32_t, M, N, M, N>;
        TileLeft<int8_t, M, baseK, M, baseK> aTile;
        TileRight<int8_t, baseK, N, baseK, N> bTile;
        AccTile cTile;
        for (int kIter = 0; kIter < K / baseK; ++kIter) {
            GlobalA gmA(dA8 + kIter * baseK);
            GlobalB gmB(dB8 + kIter * baseK);
            TLOAD(aTile, gmA);
            TLOAD(bTile, gmB);
            if (kIter == 0) {
                TMATMUL(cTile, aTile, bTile);
            } else {
                TMATMUL_ACC(cTile, cTile, aTile, bTile);
            }
        }
        ScaleMatTile scaleMat;
        ScalingTile scalingTile;
        GlobalScale scaleGlobal(dWords);
        TLOAD(scaleMat, scaleGlobal);
        TMOV(scalingTile, scaleMat);
        GlobalOut outGlobal(reinterpret_cast<bfloat16_t*>(dOut16));
        std::vector<uint16_t> out16(M * N);
        TSTORE_FP<AccTile, GlobalOut, ScalingTile>(outGlobal, cTile, scalingTile);
        cudaDeviceSynchronize();
        cudaMemcpy(out16.data(), dOut16, out16.size() * 2, cudaMemcpyDeviceToHost);
        int n6 = 0;
        for (int i = 0; i < M; ++i)
            for (int j = 0; j < N; ++j)
                n6 += (out16[i * N + j] != f32_to_bf16_rne(static_cast<float>(acc[i * N + j]) * col_scale[j]));
        std::printf("int8 program (TMATMUL/TMATMUL_ACC + TSTORE_FP per-column scale): %d mismatches\n", n6);
        bad += n6;
        TSTORE<AccTile, GlobalOut, AtomicType::AtomicNone, ReluPreMode::NormalRelu>(outGlobal, cTile,
                                                                                   static_cast<uint64_t>(scalar_bits));
        cudaDeviceSynchronize();
        cudaMemcpy(out16.data(), dOut16, out16.size() * 2, cudaMemcpyDeviceToHost);
        n6 = 0;
        for (int i = 0; i < M * N; ++i) {
            float r = static_cast<float>(acc[i]) * scalar;
            r = r > 0.0f ? r : 0.0f;
            n6 += (out16[i] != f32_to_bf16_rne(r));
        }
        std::printf("int8 program (TSTORE with a pre-quant scalar and ReLU): %d mismatches\n", n6);
        bad += n6;
        // the same accumulators requantised to int8 (REQ8): scale 0.25, offset 3 in bits [45:37], signed clamp (bit 46)
        using GlobalOut8 = GlobalTensor<int8_t, TileShape2D<int8_t, M, N, Layout::ND>, BaseShape2D<int8_t, M, N, Layout::ND>,
                                        Layout::ND>;
        int8_t* dOut8 = nullptr;
        cudaMalloc(&dOut8, M * N);
        GlobalOut8 out8Global(dOut8);
        const float quarter = 0.25f;
        uint32_t quarter_bits;
        std::memcpy(&quarter_bits, &quarter, 4);
        const uint64_t word8 = static_cast<uint64_t>(quarter_bits) | (3ull << 37) | (1ull << 46);
        TSTORE(out8Global, cTile, word8);
        cudaDeviceSynchronize();
        std::vector<int8_t> out8(M * N);
        cudaMemcpy(out8.data(), dOut8, out8.size(), cudaMemcpyDeviceToHost);
        n6 = 0;
        for (int i = 0; i < M * N; ++i) {
            float r = std::nearbyint(static_cast<float>(acc[i]) * quarter + 3.0f);
            r = r < -128.0f ? -128.0f : (r > 127.0f ? 127.0f : r);
            n6 += (out8[i] != static_cast<int8_t>(r));
        }
        std::printf("int8 program (TSTORE to int8 with a pre-quant scalar, offset and signed clamp): %d mismatches\n", n6);
        bad += n6;
        cudaFree(dOut8);
        cudaFree(dA8);
        cudaFree(dB8);
        cudaFree(dWords);
        cudaFree(dOut16);
    }
    { // (7) block-scaled K loop: e4m3 operands, e8m0 scales in MX_A_ND / MX_B_DN tensors; (8) LaunchMxMatmul on e5m2
        constexpr int mxK = 128, KG = K / 32;
        std::vector<uint8_t> a43(M * K), b43(N * K), a52(M * K), b52(N * K), sfa(M * KG), sfb(N * KG);
        for (int i = 0; i < M * K; ++i) {
            a43[i] = int_to_e4m3(ai[i]);
            a52[i] = int_to_e5m2(ai[i]);
        }
        for (int k = 0; k < K; ++k)
            for (int j = 0; j < N; ++j) {
                b43[j * K + k] = int_to_e4m3(bi[k * N + j]);
                b52[j * K + k] = int_to_e5m2(bi[k * N + j]);
            }
        for (int i = 0; i < M * KG; ++i) sfa[i] = static_cast<uint8_t>(127 + (i * 3) % 3);
        for (int i = 0; i < N * KG; ++i) sfb[i] = static_cast<uint8_t>(126 + (i * 5) % 3);
        std::vector<float> ref_mx(M * N, 0.f);
        for (int i = 0; i < M; ++i)
            for (int k = 0; k < K; ++k)
                for (int j = 0; j < N; ++j) {
                    const float sc = std::ldexp(1.0f, sfa[i * KG + k / 32] - 127) * std::ldexp(1.0f, sfb[j * KG + k / 32] - 127);
                    ref_mx[i * N + j] += static_cast<float>(ai[i * K + k] * bi[k * N + j]) * sc;
                }
        auto* dA43 = reinterpret_cast<float8_e4m3_t*>(to_device(a43));
        auto* dB43 = reinterpret_cast<float8_e4m3_t*>(to_device(b43));
        auto* dSfa = reinterpret_cast<float8_e8m0_t*>(to_device(sfa));
        auto* dSfb = reinterpret_cast<float8_e8m0_t*>(to_device(sfb));
        using GlobalA = GlobalTensor<float8_e4m3_t, TileShape2D<float8_e4m3_t, M, mxK, Layout::ND>,
                                     BaseShape2D<float8_e4m3_t, M, K, Layout::ND>, Layout::ND>;
        using GlobalB = GlobalTensor<float8_e4m3_t, TileShape2D<float8_e4m3_t, mxK, N, Layout::DN>,
                                     BaseShape2D<float8_e4m3_t, K, N, Layout::DN>, Layout::DN>;
        using GlobalSA = GlobalTensor<float8_e8m0_t, TileShape2D<float8_e8m0_t, M, mxK / 32, Layout::MX_A_ND>,
                                      BaseShape2D<float8_e8m0_t, M, KG, Layout::MX_A_ND>, Layout::MX_A_ND>;
        using GlobalSB = GlobalTensor<float8_e8m0_t, TileShape2D<float8_e8m0_t, mxK / 32, N, Layout::MX_B_DN>,
                                      BaseShape2D<float8_e8m0_t, KG, N, Layout::MX_B_DN>, Layout::MX_B_DN>;
        using GlobalC = GlobalTensor<float, Shape<1, 1, 1, M, N>, Stride<M * N, M * N, M * N, N, 1>>;
        TileLeft<float8_e4m3_t, M, mxK, M, mxK> aTile;
        TileRight<float8_e4m3_t, mxK, N, mxK, N> bTile;
        TileLeftScale<float8_e8m0_t, M, mxK / 32, M, mxK / 32> aScale;
        TileRightScale<float8_e8m0_t, mxK / 32, N, mxK / 32, N> bScale;
        TileAcc<float, M, N, M, N> cTile;
        for (int kIter = 0; kIter < K / mxK; ++kIter) {
            GlobalA gmA(dA43 + kIter * mxK);
            GlobalB gmB(dB43 + kIter * mxK);
            GlobalSA gmSA(dSfa + kIter * (mxK / 32));
            GlobalSB gmSB(dSfb + kIter * (mxK / 32));
            TLOAD(aTile, gmA);
            TLOAD(aScale, gmSA);
            TLOAD(bTile, gmB);
            TLOAD(bScale, gmSB);
            if (kIter == 0) {
                TMATMUL_MX(cTile, aTile, aScale, bTile, bScale);
            } else {
                TMATMUL_MX(cTile, cTile, aTile, aScale, bTile, bScale);
            }
        }
        GlobalC cGlobal(dC);
        TSTORE(cGlobal, cTile);
        ref.swap(ref_mx);
        check("block-scaled program (TLOAD scales / TMATMUL_MX K loop / TSTORE)");
        // (8) the six-argument launcher: e5m2 operands, bf16 result (the integers here stay exact in bf16 only when
        // small, so compare after the same rounding)
        uint8_t* dA52 = to_device(a52);
        uint8_t* dB52 = to_device(b52);
        uint16_t* dOut16 = nullptr;
        cudaMalloc(&dOut16, M * N * sizeof(uint16_t));
        LaunchMxMatmul(reinterpret_cast<uint8_t*>(dOut16), dA52, dB52, reinterpret_cast<uint8_t*>(dSfa),
                       reinterpret_cast<uint8_t*>(dSfb), nullptr, {M, N, K});
        cudaDeviceSynchronize();
        std::vector<uint16_t> out16(M * N);
        cudaMemcpy(out16.data(), dOut16, out16.size() * 2, cudaMemcpyDeviceToHost);
        int n8 = 0;
        for (int i = 0; i < M * N; ++i) n8 += (out16[i] != f32_to_bf16_rne(ref[i]));
        std::printf("LaunchMxMatmul (e5m2, bf16 out): %d mismatches\n", n8);
        bad += n8;
        // (9) the same launcher on packed 4-bit operands: element 2i in the low nibble of byte i, element 2i+1 high
        std::vector<uint8_t> a4(M * K / 2), b4(N * K / 2);
        for (int i = 0; i < M * K / 2; ++i)
            a4[i] = static_cast<uint8_t>(int_to_e2m1(ai[2 * i]) | (int_to_e2m1(ai[2 * i + 1]) << 4));
        for (int j = 0; j < N; ++j)
            for (int k = 0; k < K; k += 2)
                b4[(j * K + k) / 2] = static_cast<uint8_t>(int_to_e2m1(bi[k * N + j]) | (int_to_e2m1(bi[(k + 1) * N + j]) << 4));
        uint8_t* dA4 = to_device(a4);
        uint8_t* dB4 = to_device(b4);
        cudaMemset(dOut16, 0xFF, M * N * sizeof(uint16_t));
        LaunchMxMatmul(reinterpret_cast<uint8_t*>(dOut16), dA4, dB4, reinterpret_cast<uint8_t*>(dSfa),
                       reinterpret_cast<uint8_t*>(dSfb), nullptr, {M, N, K}, PTO_B200_E2M1);
        cudaDeviceSynchronize();
        cudaMemcpy(out16.data(), dOut16, out16.size() * 2, cudaMemcpyDeviceToHost);
        int n9 = 0;
        for (int i = 0; i < M * N; ++i) n9 += (out16[i] != f32_to_bf16_rne(ref[i]));
        std::printf("LaunchMxMatmul (float4_e2m1x2, bf16 out): %d mismatches\n", n9);
        bad += n9;
        cudaFree(dA4);
        cudaFree(dB4);
        ref.swap(ref_mx);
        cudaFree(dA43);
        cudaFree(dB43);
        cudaFree(dSfa);
        cudaFree(dSfb);
        cudaFree(dA52);
        cudaFree(dB52);
        cudaFree(dOut16);
    }
    int status = 0;
    pto_b200_device_status(&status);
    if (bad == 0 && status == 0) {
        std::printf("tile programs ok\n");
        return 0;
    }
    return 1;
}
