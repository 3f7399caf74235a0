// ref_shim.cpp - thin extern "C" entry points into the REFERENCE's own CPU simulator.
//
// TEST INFRASTRUCTURE ONLY. This file contains no arithmetic of its own: it includes the reference's headers
// and its gemm_performance tile loop from the reference tree (given on the command line as REF, never copied
// into this repository) and instantiates them for the tile shapes the parity tests and fixtures use. The
// result, oracle/_ref/libpto_ref.so, validates the C restatement in pto_gemm_oracle.c, generates the fixtures
// under tests/golden/, and is the CPU baseline of the benchmark (kind "reference").
//
// Build: see oracle/Makefile (g++ -std=c++23 with __cplusplus forced to 202302L so that the simulator's
// bfloat16_t is the real std::bfloat16_t, -O2 -D__CPU_SIM -include stdint.h -include stddef.h).
#include <pto/pto-inst.hpp>
#include <pto/common/constants.hpp>
#include <pto/cpu/MXTypes.hpp>
#include <pto/cpu/TQuant.hpp>

#include <cstdint>
#include <cstring>

// The reference tile loop RunGemmE2E (kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:170-235).
// Its <<<>>> launcher is guarded by #ifndef __COSTMODEL, the same way the reference's own host-side test pulls
// the file in (tests/costmodel/st/testcase/gemm_perf_sim/main.cpp:16-31).
#define __COSTMODEL
#include REF_GEMM_KERNEL_CPP
#undef __COSTMODEL

using namespace pto;

namespace {

template <int K>
void run_f16_tile(float* out, const uint16_t* a, const uint16_t* b_dn)
{
    RunGemmE2E<float, half, half, float, 1, 128, K, 256, 128, K, 256, 128, K, 256, 128, 64, 256, 1, 4, 4, 1>(
        out, reinterpret_cast<half*>(const_cast<uint16_t*>(a)), reinterpret_cast<half*>(const_cast<uint16_t*>(b_dn)));
}

// fp32 operands (bf16-representable values feed the same cast-to-float + fma arithmetic, cpu/TMatmul.hpp:101-104).
// baseN = 128 and stepK = 2 keep the 4-byte panels inside the simulated L1 / L0B capacities.
template <int K>
void run_f32_tile(float* out, const float* a, const float* b_dn)
{
    RunGemmE2E<float, float, float, float, 1, 128, K, 256, 128, K, 256, 128, K, 256, 128, 64, 128, 1, 2, 2, 1>(
        out, const_cast<float*>(a), const_cast<float*>(b_dn));
}

template <int K>
void run_s8_tile(int32_t* out, const int8_t* a, const int8_t* b_dn)
{
    RunGemmE2E<int32_t, int8_t, int8_t, int32_t, 1, 128, K, 256, 128, K, 256, 128, K, 256, 128, 64, 256, 1, 4, 4, 1>(
        out, const_cast<int8_t*>(a), const_cast<int8_t*>(b_dn));
}

// Raw code of element idx of a row of k elements: a byte for the fp8 types; for the packed 4-bit types two elements
// share a byte, the even one in the low nibble (GetProperDataPart, include/pto/cpu/MXTypes.hpp:351-359).
template <typename T>
uint8_t mx_raw_code(const uint8_t* base, size_t row, int k, int idx)
{
    if constexpr (IsTwinType<T>()) {
        const uint8_t byte = base[row * static_cast<size_t>(k / 2) + static_cast<size_t>(idx / 2)];
        return (idx & 1) ? static_cast<uint8_t>(byte >> 4) : static_cast<uint8_t>(byte & 0xF);
    } else {
        return base[row * static_cast<size_t>(k) + static_cast<size_t>(idx)];
    }
}

template <typename AT, typename BT>
void run_mx_tile(float* out, const uint8_t* a, const uint8_t* b_dn, const uint8_t* sfa, const uint8_t* sfb, int k,
                 const float* bias = nullptr)
{
    constexpr int M = 128, N = 256, KC = 128, KS = KC / 32;
    NPU_MEMORY_INIT(NPUArch::A5);
    using LeftTile = TileLeft<AT, M, KC, M, KC>;
    using RightTile = TileRight<BT, KC, N, KC, N>;
    using LeftScaleTile = TileLeftScale<float8_e8m0_t, M, KS, M, KS>;
    using RightScaleTile = TileRightScale<float8_e8m0_t, KS, N, KS, N>;
    using AccTile = TileAcc<float, M, N, M, N>;
    LeftTile aTile;
    RightTile bTile;
    LeftScaleTile saTile;
    RightScaleTile sbTile;
    AccTile cTile;
    TASSIGN(aTile, 0x0);
    TASSIGN(bTile, 0x0);
    TASSIGN(saTile, GetScaleAddr(aTile.data()));
    TASSIGN(sbTile, GetScaleAddr(bTile.data()));
    TASSIGN(cTile, 0x0);
    using BiasTile = Tile<TileType::Bias, float, 1, N, BLayout::RowMajor, 1, N>;
    BiasTile biasTile;
    TASSIGN(biasTile, 0x0);
    if (bias != nullptr) {
        for (int j = 0; j < N; ++j) {
            biasTile.SetElement(0, j, bias[j]);
        }
    }
    const int kg = k / 32;
    for (int k0 = 0; k0 < k; k0 += KC) {
        for (int i = 0; i < M; ++i) {
            for (int kk = 0; kk < KC; ++kk) {
                aTile.SetElement(i, kk, AT::FromRaw(mx_raw_code<AT>(a, i, k, k0 + kk)));
            }
            for (int g = 0; g < KS; ++g) {
                saTile.SetElement(i, g, float8_e8m0_t::FromRaw(sfa[static_cast<size_t>(i) * kg + k0 / 32 + g]));
            }
        }
        for (int j = 0; j < N; ++j) {
            for (int kk = 0; kk < KC; ++kk) {
                bTile.SetElement(kk, j, BT::FromRaw(mx_raw_code<BT>(b_dn, j, k, k0 + kk)));
            }
            for (int g = 0; g < KS; ++g) {
                sbTile.SetElement(g, j, float8_e8m0_t::FromRaw(sfb[static_cast<size_t>(j) * kg + k0 / 32 + g]));
            }
        }
        if (k0 == 0 && bias != nullptr) {
            TMATMUL_MX(cTile, aTile, saTile, bTile, sbTile, biasTile);
        } else if (k0 == 0) {
            TMATMUL_MX(cTile, aTile, saTile, bTile, sbTile);
        } else {
            TMATMUL_MX(cTile, cTile, aTile, saTile, bTile, sbTile);
        }
    }
    for (int i = 0; i < M; ++i) {
        for (int j = 0; j < N; ++j) {
            out[static_cast<size_t>(i) * N + j] = cTile.GetElement(i, j);
        }
    }
}

// One 128 x 256 tile through TMATMUL_BIAS on the first 64-deep K chunk and TMATMUL_ACC on the rest, the way a K loop
// uses the bias form (tests/cpu/st/testcase/tmatmul/tmatmul_kernel.cpp:86-96 for the single-chunk case).
template <typename AccT, typename InT, typename RawT>
void run_bias_tile(AccT* out, const RawT* a, const RawT* b_dn, const AccT* bias, int k)
{
    constexpr int M = 128, N = 256, KC = 64;
    using LeftTile = TileLeft<InT, M, KC, M, KC>;
    using RightTile = TileRight<InT, KC, N, KC, N>;
    using AccTile = TileAcc<AccT, M, N, M, N>;
    using BiasTile = Tile<TileType::Bias, AccT, 1, N, BLayout::RowMajor, 1, N>;
    LeftTile aTile;
    RightTile bTile;
    AccTile cTile;
    BiasTile biasTile;
    TASSIGN(aTile, 0x0);
    TASSIGN(bTile, 0x0);
    TASSIGN(cTile, 0x0);
    TASSIGN(biasTile, 0x0);
    for (int j = 0; j < N; ++j) {
        biasTile.SetElement(0, j, bias[j]);
    }
    const InT* at = reinterpret_cast<const InT*>(a);
    const InT* bt = reinterpret_cast<const InT*>(b_dn);
    for (int k0 = 0; k0 < k; k0 += KC) {
        for (int i = 0; i < M; ++i) {
            for (int kk = 0; kk < KC; ++kk) {
                aTile.SetElement(i, kk, at[static_cast<size_t>(i) * k + k0 + kk]);
            }
        }
        for (int j = 0; j < N; ++j) {
            for (int kk = 0; kk < KC; ++kk) {
                bTile.SetElement(kk, j, bt[static_cast<size_t>(j) * k + k0 + kk]);
            }
        }
        if (k0 == 0) {
            TMATMUL_BIAS(cTile, aTile, bTile, biasTile);
        } else {
            TMATMUL_ACC(cTile, cTile, aTile, bTile);
        }
    }
    for (int i = 0; i < M; ++i) {
        for (int j = 0; j < N; ++j) {
            out[static_cast<size_t>(i) * N + j] = cTile.GetElement(i, j);
        }
    }
}

} // namespace

extern "C" {

// 128 x 256 output tile, bias form: TMATMUL_BIAS on k in [0, 64), TMATMUL_ACC afterwards. k % 64 == 0.
int ref_tile_f16_bias(float* out, const uint16_t* a, const uint16_t* b_dn, const float* bias, int k)
{
    if (k <= 0 || k % 64 != 0) {
        return -1;
    }
    run_bias_tile<float, half, uint16_t>(out, a, b_dn, bias, k);
    return 0;
}

// e4m3 x e4m3 MX tile with the six-operand TMATMUL_MX (bias) on the first 128-deep chunk. k % 128 == 0.
int ref_tile_mx_bias(float* out, const uint8_t* a, const uint8_t* b_dn, const uint8_t* sfa, const uint8_t* sfb,
                     const float* bias, int k)
{
    if (k <= 0 || k % 128 != 0 || bias == nullptr) {
        return -1;
    }
    run_mx_tile<float8_e4m3_t, float8_e4m3_t>(out, a, b_dn, sfa, sfb, k, bias);
    return 0;
}

int ref_tile_s8_bias(int32_t* out, const int8_t* a, const int8_t* b_dn, const int32_t* bias, int k)
{
    if (k <= 0 || k % 64 != 0) {
        return -1;
    }
    run_bias_tile<int32_t, int8_t, int8_t>(out, a, b_dn, bias, k);
    return 0;
}

// 1 if this build has the simulator's real bfloat16_t (std::bfloat16_t), 0 if it is the _Float16 placeholder.
int ref_has_real_bf16()
{
#if defined(__STDCPP_BFLOAT16_T__) && __cplusplus >= 202302L
    return 1;
#else
    return 0;
#endif
}

// One 128 x 256 output tile with the full K, B column-major (stored 256 x K). Returns 0, or -1 if K is not
// one of the instantiated depths.
int ref_tile_f16(float* out, const uint16_t* a, const uint16_t* b_dn, int k)
{
    switch (k) {
        case 256: run_f16_tile<256>(out, a, b_dn); return 0;
        case 1024: run_f16_tile<1024>(out, a, b_dn); return 0;
        case 6144: run_f16_tile<6144>(out, a, b_dn); return 0;
        default: return -1;
    }
}

int ref_tile_f32(float* out, const float* a, const float* b_dn, int k)
{
    switch (k) {
        case 256: run_f32_tile<256>(out, a, b_dn); return 0;
        case 1024: run_f32_tile<1024>(out, a, b_dn); return 0;
        case 4096: run_f32_tile<4096>(out, a, b_dn); return 0;
        case 8192: run_f32_tile<8192>(out, a, b_dn); return 0;
        case 65536: run_f32_tile<65536>(out, a, b_dn); return 0;
        default: return -1;
    }
}

int ref_tile_s8(int32_t* out, const int8_t* a, const int8_t* b_dn, int k)
{
    switch (k) {
        case 256: run_s8_tile<256>(out, a, b_dn); return 0;
        case 1024: run_s8_tile<1024>(out, a, b_dn); return 0;
        case 8192: run_s8_tile<8192>(out, a, b_dn); return 0;
        default: return -1;
    }
}

// fmt: 5 = e4m3, 6 = e5m2, 7 = e2m1 packed two per byte (the pto_b200_dtype values). k must be a multiple of 128.
int ref_tile_mx(float* out, const uint8_t* a, const uint8_t* b_dn, const uint8_t* sfa, const uint8_t* sfb, int k,
                int a_fmt, int b_fmt)
{
    if (k <= 0 || k % 128 != 0) {
        return -1;
    }
    if (a_fmt == 5 && b_fmt == 5) {
        run_mx_tile<float8_e4m3_t, float8_e4m3_t>(out, a, b_dn, sfa, sfb, k);
    } else if (a_fmt == 6 && b_fmt == 6) {
        run_mx_tile<float8_e5m2_t, float8_e5m2_t>(out, a, b_dn, sfa, sfb, k);
    } else if (a_fmt == 5 && b_fmt == 6) {
        run_mx_tile<float8_e4m3_t, float8_e5m2_t>(out, a, b_dn, sfa, sfb, k);
    } else if (a_fmt == 6 && b_fmt == 5) {
        run_mx_tile<float8_e5m2_t, float8_e4m3_t>(out, a, b_dn, sfa, sfb, k);
    } else if (a_fmt == 7 && b_fmt == 7) { // MXFP4: float4_e2m1x2_t operands, two per byte
        run_mx_tile<float4_e2m1x2_t, float4_e2m1x2_t>(out, a, b_dn, sfa, sfb, k);
    } else {
        return -1;
    }
    return 0;
}

// Fixpipe per-column dequant of one int32 accumulator (vector form: the 64-bit scale word carries the fp32
// bits of s_col in [31:0], of which the simulator reads [31:13]); returns the fp32 value before the output cast.
float ref_dequant_col(int32_t acc, float s_col)
{
    uint32_t bits;
    std::memcpy(&bits, &s_col, 4);
    return quantize_element<float, int32_t, QuantMode_t::VQS322BF16_PRE, false>(acc, static_cast<uint64_t>(bits));
}

// TSTORE with a pre-quant scale word, one accumulator value through the simulator's own ConvertStoreValue /
// quantize_element (include/pto/cpu/TStore.hpp:154-181, include/pto/cpu/common.hpp:139-198), with the mode the
// TSTORE overloads pick (GetScalarPreQuantMode / GetVectorPreQuantMode, common.hpp:58-108):
//   acc_is_int  1: int32 accumulator (acc_i), 0: float accumulator (acc_f)
//   out_f16     1: half destination, 0: bfloat16_t destination
//   vector      1: TSTORE(dst, acc, fpTile) / TSTORE_FP, scale in bits [31:13]; 0: TSTORE(dst, acc, preQuantScalar)
//   relu        ReluPreMode::NormalRelu
// Returns the 16 destination bits.
uint16_t ref_quant_store(int acc_is_int, int out_f16, int vector, int relu, int32_t acc_i, float acc_f, uint64_t word)
{
    uint16_t bits = 0;
    auto run = [&](auto dst_tag, auto src_tag, auto vec_tag, auto relu_tag) {
        using D = decltype(dst_tag);
        using S = decltype(src_tag);
        constexpr bool kVec = decltype(vec_tag)::value;
        constexpr bool kRelu = decltype(relu_tag)::value;
        constexpr QuantMode_t mode = kVec ? GetVectorPreQuantMode<S, D>() : GetScalarPreQuantMode<S, D>();
        const S v = std::is_same_v<S, int32_t> ? static_cast<S>(acc_i) : static_cast<S>(acc_f);
        const D d = ConvertStoreValue<D, S, mode, kRelu>(v, word);
        std::memcpy(&bits, &d, sizeof(D));
    };
    auto with_relu = [&](auto d, auto s, auto v) {
        if (relu) {
            run(d, s, v, std::true_type{});
        } else {
            run(d, s, v, std::false_type{});
        }
    };
    auto with_vec = [&](auto d, auto s) {
        if (vector) {
            with_relu(d, s, std::true_type{});
        } else {
            with_relu(d, s, std::false_type{});
        }
    };
    auto with_src = [&](auto d) {
        if (acc_is_int) {
            with_vec(d, int32_t{});
        } else {
            with_vec(d, float{});
        }
    };
    switch (out_f16) { // destination: 0 bfloat16, 1 half, 2 int8, 3 uint8 (results in the low byte), 4 int16
        case 1:
            with_src(half{});
            break;
        case 2:
            with_src(int8_t{});
            break;
        case 3:
            with_src(uint8_t{});
            break;
        case 4: // SHIFTS322S16 / VSHIFTS322S16: int32 accumulators only
            if (vector) {
                if (relu) run(int16_t{}, int32_t{}, std::true_type{}, std::true_type{});
                else run(int16_t{}, int32_t{}, std::true_type{}, std::false_type{});
            } else {
                if (relu) run(int16_t{}, int32_t{}, std::false_type{}, std::true_type{});
                else run(int16_t{}, int32_t{}, std::false_type{}, std::false_type{});
            }
            break;
        default:
            with_src(bfloat16_t{});
            break;
    }
    return bits;
}

// TSTORE's no-quant cast, static_cast<Dst>(float) (include/pto/cpu/common.hpp:187-198).
uint16_t ref_cast_bf16(float v)
{
    const bfloat16_t h = ConvertStoreValue<bfloat16_t, float, QuantMode_t::NoQuant, false>(v, 0);
    uint16_t u;
    std::memcpy(&u, &h, 2);
    return u;
}

uint16_t ref_cast_f16(float v)
{
    const half h = ConvertStoreValue<half, float, QuantMode_t::NoQuant, false>(v, 0);
    uint16_t u;
    std::memcpy(&u, &h, 2);
    return u;
}

// OCP MX quantiser pieces (include/pto/cpu/TQuant.hpp:178-190, 226-237, 118-153) applied per row and 32-wide block.
void ref_mx_quantize_e4m3(const float* src, uint8_t* data, uint8_t* scales, int rows, int k)
{
    using namespace pto::cpu_quant;
    const int groups = k / 32;
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < groups; ++g) {
            const float* x = src + static_cast<size_t>(r) * k + g * 32;
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) {
                amax = std::max(amax, std::fabs(x[i]));
            }
            const uint8_t e = ComputeSharedExponent(amax);
            const float scaling = ComputeMxScalingFromExponent(e);
            scales[static_cast<size_t>(r) * groups + g] = e;
            for (int i = 0; i < 32; ++i) {
                data[static_cast<size_t>(r) * k + g * 32 + i] = EncodeE4M3Fn<QuantScaleAlg::OCP>(x[i] * scaling);
            }
        }
    }
}

// The same with the NV scale rule (include/pto/cpu/TQuant.hpp:194-211 ComputeNvSharedExponent with the e4m3 spec
// :33-37, :239-248 ComputeNvScalingFromExponent, :118-131 EncodeE4M3Fn<NV>).
void ref_mx_quantize_e4m3_nv(const float* src, uint8_t* data, uint8_t* scales, int rows, int k)
{
    using namespace pto::cpu_quant;
    const int groups = k / 32;
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < groups; ++g) {
            const float* x = src + static_cast<size_t>(r) * k + g * 32;
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) {
                amax = std::max(amax, std::fabs(x[i]));
            }
            const uint8_t e = ComputeMxSharedExponent<QuantType::MXFP8, QuantScaleAlg::NV>(amax);
            const float scaling = ComputeMxGroupScaling<QuantType::MXFP8, QuantScaleAlg::NV>(amax, e);
            scales[static_cast<size_t>(r) * groups + g] = e;
            for (int i = 0; i < 32; ++i) {
                data[static_cast<size_t>(r) * k + g * 32 + i] = EncodeE4M3Fn<QuantScaleAlg::NV>(x[i] * scaling);
            }
        }
    }
}

// TQUANT<QuantType::MXFP4_E2M1> per row and 32-wide block with either scale rule (include/pto/cpu/TQuant.hpp:
// ComputeMxGroupMax :280-305, ComputeMxSharedExponent :316-334, ComputeMxGroupScaling :336-347, StoreMxEncodedValue
// :349-372 with EncodeE2M1Magic :155-176), float source; data: rows x k/2 bytes, element 2i in the low nibble.
void ref_mx_quantize_e2m1(const float* src, uint8_t* data, uint8_t* scales, int rows, int k, int nv)
{
    using namespace pto::cpu_quant;
    const int groups = k / 32;
    std::memset(data, 0, static_cast<size_t>(rows) * (k / 2));
    for (int r = 0; r < rows; ++r) {
        for (int g = 0; g < groups; ++g) {
            const float* x = src + static_cast<size_t>(r) * k + g * 32;
            float amax = 0.0f;
            uint16_t amax_bits = 0;
            for (int i = 0; i < 32; ++i) {
                if (nv) {
                    amax = std::max(amax, std::fabs(x[i]));
                } else {
                    amax_bits = std::max(amax_bits, AbsBf16BitsFromFloat(x[i]));
                }
            }
            if (!nv) {
                amax = Bf16BitsToFloat(amax_bits);
            }
            uint8_t e;
            float scaling;
            if (nv) {
                e = ComputeMxSharedExponent<QuantType::MXFP4_E2M1, QuantScaleAlg::NV>(amax);
                scaling = ComputeMxGroupScaling<QuantType::MXFP4_E2M1, QuantScaleAlg::NV>(amax, e);
            } else {
                e = ComputeMxSharedExponent<QuantType::MXFP4_E2M1, QuantScaleAlg::OCP>(amax);
                scaling = ComputeMxGroupScaling<QuantType::MXFP4_E2M1, QuantScaleAlg::OCP>(amax, e);
            }
            scales[static_cast<size_t>(r) * groups + g] = e;
            for (int i = 0; i < 32; ++i) {
                uint8_t code = NvMxFp4E2M1Spec::PS_MAX;
                if (std::isinf(scaling)) {
                    code = (scaling > 0) ? NvMxFp4E2M1Spec::PS_MAX : NvMxFp4E2M1Spec::NG_MIN;
                } else if (!std::isnan(scaling)) {
                    code = EncodeE2M1Magic(ApplyE2M1ScaleForSource<float>(x[i], scaling));
                }
                const int col = g * 32 + i;
                uint8_t& byte = data[static_cast<size_t>(r) * (k / 2) + col / 2];
                byte = (col & 1) ? static_cast<uint8_t>((byte & 0x0F) | (code << 4)) : static_cast<uint8_t>((byte & 0xF0) | (code & 0x0F));
            }
        }
    }
}

double ref_fp8_to_double(uint8_t raw, int fmt)
{
    return fmt == 6 ? static_cast<double>(float8_e5m2_t::FromRaw(raw)) : static_cast<double>(float8_e4m3_t::FromRaw(raw));
}

double ref_e8m0_to_double(uint8_t raw) { return static_cast<double>(float8_e8m0_t::FromRaw(raw)); }

} // extern "C"
