// gemm_tile_program.cpp - the reference's two GEMM tile programs written against include/pto/pto-inst.hpp and run
// on a B200: (1) the CPU demo's TLOAD / TMOV / TMATMUL / TSTORE sequence (demos/cpu/gemm_demo/gemm_demo.cpp:83-121,
// B row-major), (2) the gemm_performance K loop with TEXTRACT slices and TMATMUL / TMATMUL_ACC
// (kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:69-131, B column-major), (3) the fixed-signature
// launcher, (4) the bias form of the K loop (TMATMUL_BIAS then TMATMUL_ACC, tests/cpu/st/testcase/tmatmul/
// tmatmul_kernel.cpp:86-96) and (5) a one-row TGEMV_BIAS. Inputs are small integers so the fp32 results are exact;
// the program checks them against a host loop and prints "tile programs ok".
//
// Build (one line): g++ -std=c++17 -I include -I /usr/local/cuda/include examples/gemm_tile_program.cpp
//   -L pto_isa_mirror_b200/lib -lpto_b200 -L /usr/local/cuda/lib64 -lcudart -o examples/gemm_tile_program
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
    int status = 0;
    pto_b200_device_status(&status);
    if (bad == 0 && status == 0) {
        std::printf("tile programs ok\n");
        return 0;
    }
    return 1;
}
