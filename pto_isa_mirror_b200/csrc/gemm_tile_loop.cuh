// Persistent, warp-specialised GEMM tile loop for sm_100a.
//
// This is the B200 form of the PTO tile program TLOAD -> TEXTRACT -> TMATMUL / TMATMUL_ACC -> TSTORE
// (reference: kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:69-235 and its MX twin
// kernels/manual/a5/matmul_mxfp8_performance/mxmatmul_performance_kernel.cpp:153-344):
//
//   reference pipe / buffer                      this kernel
//   ---------------------------------------     -----------------------------------------------------
//   MTE2 TLOAD GM->L1 (ND->Nz / DN->Zn)          warp 0, one thread: TMA 2-D tiled loads into a ring of
//                                                128-byte-swizzled shared-memory stages
//   MTE1 TEXTRACT L1->L0A/L0B (baseK slices)     none: UMMA descriptors address the stage directly and a
//                                                K-slice is a start-address advance of 32 bytes
//   Cube TMATMUL (k==0) / TMATMUL_ACC (k>0)      warp 1, one thread: tcgen05.mma, enable_input_d = (k>0),
//                                                accumulator in tensor memory (the L0C analogue)
//   FIX  TSTORE L0C->GM (+cast / dequant)        warps 2..5: tcgen05.ld -> registers -> cast / scale -> stores
//   set_flag / wait_flag ping-pong               mbarrier full/empty rings; tcgen05.commit releases stages
//   get_block_idx() -> fixed C sub-matrix        persistent CTAs walking a grouped tile raster
//
// Every wait is bounded: a barrier that does not flip within the limit records a code in *status,
// raises a CTA-wide abort flag, lets in-flight copies land and leaves without trapping.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace pto_b200 {

enum MmaKind : int { KIND_F16 = 0, KIND_I8 = 1, KIND_MXF8 = 2 };
enum EpilogueMode : int {
    EPI_F32 = 0,     // store the fp32 accumulator
    EPI_BF16 = 1,    // static_cast<bfloat16>(fp32), round to nearest even
    EPI_F16 = 2,     // static_cast<half>(fp32), round to nearest even
    EPI_S32 = 3,     // store the int32 accumulator
    EPI_DEQ_BF16 = 4, // bf16((float(acc) * s_col[j]) * s_row[i])
    EPI_QUANT16 = 5,  // TSTORE with a pre-quant scale word: cast16(relu?(clamp(float(acc) * scale_j))), see QuantFlags
    EPI_QUANT8 = 6    // the same to int8 / uint8: relu?(clamp(rint(float(acc) * scale_j + offset)))
};

// EPI_QUANT16 variants (GemmParams::quant_flags): the accumulator type, the 16-bit destination, ReLU, and whether the
// scale is one word for the tile (TSTORE(dst, acc, preQuantScalar): fp32 in bits [31:0]) or one word per column
// (TSTORE(dst, acc, fpTile) / TSTORE_FP: the 19-bit (1,8,10) float in bits [31:13]); include/pto/cpu/common.hpp:116-185.
// EPI_QUANT8 (REQ8 / VREQ8 for int32 accumulators, QF322B8_PRE / VQF322B8_PRE for float ones, :151-156): the word also
// carries a 9-bit offset in bits [45:37], added before rounding to nearest even, and the sign flag in bit 46 (clamp to
// -128..127 when set, else to 0..255); the 8-bit result is stored as is.
// QUANT_OUT_S16 (SHIFTS322S16 / VSHIFTS322S16, :172-178): int16(acc >> (1 + bits [35:32] of the word)), no scale.
enum QuantFlags : int { QUANT_ACC_S32 = 1, QUANT_OUT_F16 = 2, QUANT_RELU = 4, QUANT_VECTOR = 8, QUANT_OUT_S16 = 16 };

struct GemmParams {
    void* c;
    long long ldc; // elements
    int m, n, k;
    int m_tiles, n_tiles, k_blocks, group_m;
    uint32_t idesc;
    const float* s_row;
    const float* s_col;
    const uint8_t* sfa; // scale factors re-tiled to 512-byte atoms, index (k_block, 128-row block of A)
    const uint8_t* sfb; // same, index (k_block, 128-column block of B)
    int sf_a_blocks;    // 128-row blocks per k_block in sfa (the same for every kernel: 2 * ceil(m / 256))
    int sf_b_blocks;    // 128-column blocks per k_block in sfb (2 * ceil(n / 256))
    const void* bias;   // TMATMUL_BIAS: one value per output column in the accumulator's type (fp32 / int32), or null
    int* status;
    // CTA-pair kernels, last partly filled wave: each leftover tile is cut in two K halves that run on two pairs at
    // once; each pair parks the accumulators of the columns the other pair finishes and adds the other's to its own.
    int tail_first_unit; // first work unit of the split tail (= number of tiles when nothing is split)
    int tail_tiles;      // leftover tiles that are split (0 = none)
    uint32_t* ws_partial; // [tail_tiles][2 K halves][2 CTAs][128 x 128] parked 32-bit accumulators
    int* ws_flags;        // [tail_tiles][2 K halves][8 store warps]: "my half is parked" = this launch's token
    int tail_token;       // never 0, different for every launch that splits tiles
    int mi_rotate;        // CTA-pair kernels: the tile raster starts at this row of tiles and wraps (0 = from the top)
    const unsigned long long* quant_words; // EPI_QUANT16, vector form: n scale words in device memory
    unsigned long long quant_word;         // EPI_QUANT16, scalar form: the scale word
    int quant_flags;                       // EPI_QUANT16: QuantFlags
    long long wait_limit; // cycles one bounded wait may take before the kernel gives up (kWaitLimitCycles by default)
    int tma_store;        // CTA-pair kernels: C is 16-byte aligned with a 16-byte row pitch, so finished tiles leave
                          // through shared memory and TMA stores; 0 = per-thread global stores
    int packed4;          // 1 when the operand tensor maps unpack 4-bit values (two per byte in memory, one per byte
                          // in shared memory): a load then completes half the bytes it writes on its barrier
};

constexpr int kBlockM = 128;
constexpr int kBlockKBytes = 128; // one 128-byte swizzle row per matrix row
constexpr int kUmmaKBytes = 32;
constexpr int kNumThreads = 192;
constexpr int kTmemCols = 512;
constexpr long long kWaitLimitCycles = 4000000000ll; // default limit of one wait: about two seconds

enum StatusCode : int {
    ST_OK = 0,
    ST_PRODUCER_TIMEOUT = 1,
    ST_MMA_FULL_TIMEOUT = 2,
    ST_MMA_ACC_TIMEOUT = 3,
    ST_EPILOGUE_TIMEOUT = 4
};

template <int KIND, int BLOCK_N, int STAGES>
struct SmemLayout {
    static constexpr int kABytes = kBlockM * kBlockKBytes;
    static constexpr int kBBytes = BLOCK_N * kBlockKBytes;
    static constexpr int kSfaBytes = (KIND == KIND_MXF8) ? 512 : 0;
    static constexpr int kSfbBytes = (KIND == KIND_MXF8) ? ((BLOCK_N + 127) / 128) * 512 : 0;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kAOff = 0;
    static constexpr int kBOff = STAGES * kABytes;
    static constexpr int kSfaOff = kBOff + STAGES * kBBytes;
    static constexpr int kSfbOff = kSfaOff + STAGES * kSfaBytes;
    static constexpr int kBarOff = kSfbOff + STAGES * kSfbBytes;
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;
    static constexpr int kTotal = kMiscOff + 16 + 1024; // + slack to align the base to 1024
};

// Bounded mbarrier wait. Returns false after the limit or once another role raised the abort flag.
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                             int* status, int code, long long limit)
{
    if (ptx::mbar_try_wait(bar, parity)) {
        return true;
    }
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
        if (((++spins) & 0x3Fu) == 0) {
            if (*abort_flag != 0) {
                return false;
            }
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

// Grouped raster: walk group_m row-tiles down, then step one column-tile right, so a wave of
// concurrent CTAs shares a small set of A and B panels in L2.
__device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& mi, int& ni)
{
    const int group_size = p.group_m * p.n_tiles;
    const int g = t / group_size;
    const int first_m = g * p.group_m;
    const int gm = min(p.m_tiles - first_m, p.group_m);
    const int r = t - g * group_size;
    mi = first_m + r % gm;
    ni = r / gm;
}

// Words one 32-column chunk of an accumulator row becomes on its way out: 32 for 32-bit outputs, 16 (two values each)
// for 16-bit outputs, 8 (four values each) for 8-bit outputs.
template <int EPI>
struct OutWords {
    static constexpr int kCount = (EPI == EPI_F32 || EPI == EPI_S32) ? 32 : (EPI == EPI_QUANT8 ? 8 : 16);
};

// The scale of a pre-quant word: fp32 in bits [31:0] (scalar form) or the 19-bit (1, 8, 10) float in bits [31:13]
// (vector form), extract_m1_from_quant, include/pto/cpu/common.hpp:116-137.
__device__ __forceinline__ float quant_word_scale(uint32_t lo, bool vector)
{
    if (!vector) {
        return __uint_as_float(lo);
    }
    // sign, 8 exponent and 10 mantissa bits from [31:13]: fp32 with the low 13 mantissa bits dropped; a zero exponent
    // field with a non-zero mantissa reads as (1 + m / 1024) * 2^-127 in the reference
    const uint32_t e = (lo >> 23) & 0xFFu;
    const uint32_t mnt = (lo >> 13) & 0x3FFu;
    if (e != 0u || mnt == 0u) {
        return __uint_as_float(e != 0u ? (lo & 0xFFFFE000u) : 0u);
    }
    const float mag = __fmul_rn(1.0f + static_cast<float>(mnt) * (1.0f / 1024.0f), __uint_as_float(0x00400000u)); // 2^-127
    return (lo >> 31) ? -mag : mag;
}

// One 32-column chunk of one accumulator row -> output words: optional bias, then cast / dequantise. The bias is
// added to the finished accumulator in the accumulator's own type, once per output element (TMATMUL_BIAS adds it
// after the first matmul of the K loop, include/pto/cpu/TMatmul.hpp:219-230: exact for int32, one fp32 rounding apart
// otherwise). Columns at or past N read neither bias nor scale; their words are never stored.
template <int EPI>
__device__ __forceinline__ void convert_chunk(const uint32_t (&v)[32], const GemmParams& p, int col0, float s_row,
                                              uint32_t (&o)[OutWords<EPI>::kCount])
{
    const int n_left = p.n - col0;
    uint32_t w[32];
    if (p.bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if constexpr (EPI == EPI_S32 || EPI == EPI_DEQ_BF16) {
                const uint32_t b = (i < n_left) ? __ldg(static_cast<const uint32_t*>(p.bias) + col0 + i) : 0u;
                w[i] = v[i] + b; // two's complement: the int32 sum
            } else {
                const float b = (i < n_left) ? __ldg(static_cast<const float*>(p.bias) + col0 + i) : 0.0f;
                w[i] = __float_as_uint(__fadd_rn(__uint_as_float(v[i]), b));
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            w[i] = v[i];
        }
    }
    if constexpr (EPI == EPI_F32 || EPI == EPI_S32) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            o[i] = w[i];
        }
    } else if constexpr (EPI == EPI_QUANT8) {
        const bool acc_int = (p.quant_flags & QUANT_ACC_S32) != 0;
        const bool relu = (p.quant_flags & QUANT_RELU) != 0;
        const bool vector = (p.quant_flags & QUANT_VECTOR) != 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const unsigned long long word = vector ? ((i < n_left) ? __ldg(p.quant_words + col0 + i) : 0ull) : p.quant_word;
            const float scale = quant_word_scale(static_cast<uint32_t>(word), vector);
            const float offset = static_cast<float>(static_cast<uint32_t>(word >> 37) & 0x1FFu);
            const bool is_signed = ((word >> 46) & 1ull) != 0;
            const float src = acc_int ? __int2float_rn(static_cast<int>(w[i])) : __uint_as_float(w[i]);
            float q = rintf(__fadd_rn(__fmul_rn(src, scale), offset));
            q = fminf(fmaxf(q, is_signed ? -128.0f : 0.0f), is_signed ? 127.0f : 255.0f);
            if (relu) {
                q = (q > 0.0f) ? q : 0.0f;
            }
            o[i >> 2] |= (static_cast<uint32_t>(__float2int_rn(q)) & 0xFFu) << ((i & 3) * 8);
        }
    } else {
        float f[32];
        if constexpr (EPI == EPI_QUANT16) {
            if ((p.quant_flags & QUANT_OUT_S16) != 0) {
                // the arithmetic shift, the wrapping cast to int16, ReLU
                const bool relu16 = (p.quant_flags & QUANT_RELU) != 0;
                const bool vector16 = (p.quant_flags & QUANT_VECTOR) != 0;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const unsigned long long word =
                        vector16 ? ((i < n_left) ? __ldg(p.quant_words + col0 + i) : 0ull) : p.quant_word;
                    const int shift = static_cast<int>((word >> 32) & 0xFull) + 1;
                    int v16 = static_cast<short>(static_cast<int>(w[i]) >> shift);
                    if (relu16 && v16 < 0) {
                        v16 = 0;
                    }
                    const uint32_t bits = static_cast<uint32_t>(v16) & 0xFFFFu;
                    if ((i & 1) == 0) {
                        o[i >> 1] = bits;
                    } else {
                        o[i >> 1] |= bits << 16;
                    }
                }
                return;
            }
        }
        if constexpr (EPI == EPI_QUANT16) {
            // quantize_element (include/pto/cpu/common.hpp:139-185): float(acc) * scale, the half forms clamp to
            // +-65504 (always for int32 accumulators, finite values only for float ones), ReLU after the scaling.
            const bool acc_int = (p.quant_flags & QUANT_ACC_S32) != 0;
            const bool out_f16 = (p.quant_flags & QUANT_OUT_F16) != 0;
            const bool relu = (p.quant_flags & QUANT_RELU) != 0;
            const bool vector = (p.quant_flags & QUANT_VECTOR) != 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const uint32_t lo = vector ? ((i < n_left) ? static_cast<uint32_t>(__ldg(p.quant_words + col0 + i)) : 0u)
                                           : static_cast<uint32_t>(p.quant_word);
                const float scale = quant_word_scale(lo, vector);
                const float src = acc_int ? __int2float_rn(static_cast<int>(w[i])) : __uint_as_float(w[i]);
                float r = __fmul_rn(src, scale);
                if (out_f16 && (acc_int || isfinite(r))) {
                    r = fminf(fmaxf(r, -65504.0f), 65504.0f);
                }
                if (relu) {
                    r = (r > 0.0f) ? r : 0.0f;
                }
                f[i] = r;
            }
        } else if constexpr (EPI == EPI_DEQ_BF16) {
            // Fixpipe per-column dequant, then the per-row (per-token) scale, two separately rounded
            // fp32 multiplies: quantize_element (include/pto/cpu/common.hpp:139-185) followed by
            // the row-scale multiply of the vector stage.
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float sc = (i < n_left) ? __ldg(p.s_col + col0 + i) : 0.0f;
                const float t = __fmul_rn(__int2float_rn(static_cast<int>(w[i])), sc);
                f[i] = __fmul_rn(t, s_row);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                f[i] = __uint_as_float(w[i]);
            }
        }
        bool to_half = (EPI == EPI_F16);
        if constexpr (EPI == EPI_QUANT16) {
            to_half = (p.quant_flags & QUANT_OUT_F16) != 0;
        }
        if (to_half) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
                o[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                o[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
    }
}

// The words of one chunk stored straight to C by the thread that owns the row: 16-byte stores when C allows them,
// element by element on unaligned or ragged edges.
template <int EPI>
__device__ __forceinline__ void store_words(const uint32_t (&o)[OutWords<EPI>::kCount], const GemmParams& p, int row,
                                            int col0, bool vec_ok)
{
    const int n_left = p.n - col0;
    if constexpr (EPI == EPI_F32 || EPI == EPI_S32) {
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
        if (vec_ok && n_left >= 32) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                d4[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (i < n_left) {
                    dst[i] = o[i];
                }
            }
        }
    } else if constexpr (EPI == EPI_QUANT8) {
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
        if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0 && n_left >= 32) {
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (i < n_left) {
                    dst[i] = static_cast<uint8_t>((o[i >> 2] >> ((i & 3) * 8)) & 0xFFu);
                }
            }
        }
    } else {
        uint16_t* dst = reinterpret_cast<uint16_t*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
        if (vec_ok && n_left >= 32) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                d4[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            }
        } else {
            // Rows that start off a 16-byte boundary (an odd pitch such as 8100 bf16) or the ragged last chunk: the
            // widest pieces the address allows - 8 bytes, 4 bytes, else single values - and single values at the end.
            const uintptr_t addr = reinterpret_cast<uintptr_t>(dst);
            const int piece = (addr & 7u) == 0 ? 4 : ((addr & 3u) == 0 ? 2 : 1); // 16-bit values per store
            if (piece == 4) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (4 * i + 4 <= n_left) {
                        reinterpret_cast<uint2*>(dst)[i] = make_uint2(o[2 * i], o[2 * i + 1]);
                    }
                }
            } else if (piece == 2) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (2 * i + 2 <= n_left) {
                        reinterpret_cast<uint32_t*>(dst)[i] = o[i];
                    }
                }
            }
            const int done = piece == 1 ? 0 : (n_left >= 32 ? 32 : n_left / piece * piece);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                if (i >= done && i < n_left) {
                    dst[i] = static_cast<uint16_t>((o[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu);
                }
            }
        }
    }
}

// One 32-column chunk of one accumulator row: bias, cast / dequantise, store.
template <int EPI>
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[32], const GemmParams& p, int row, int col0,
                                            bool vec_ok, float s_row)
{
    if (row >= p.m) {
        return;
    }
    uint32_t o[OutWords<EPI>::kCount];
    convert_chunk<EPI>(v, p, col0, s_row, o);
    store_words<EPI>(o, p, row, col0, vec_ok);
}

template <int KIND, int BLOCK_N, int STAGES, int EPI, bool B_MN_MAJOR>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_tile_loop(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const GemmParams p)
{
    using L = SmemLayout<KIND, BLOCK_N, STAGES>;
    static_assert((BLOCK_N == 32 || BLOCK_N % 64 == 0) && BLOCK_N <= 256, "BLOCK_N");
    static_assert(!B_MN_MAJOR || (KIND == KIND_F16 && BLOCK_N % 64 == 0), "N-major B is for 16-bit inputs");
    // Block-scaled tiles keep their scale factors in TMEM beside one accumulator; the others double-buffer.
    constexpr int kNumAcc = (KIND == KIND_MXF8) ? 1 : 2;
    constexpr int kAccCols = 256;
    constexpr uint32_t kSfaCol = 256;
    constexpr uint32_t kSfbCol = 260;
    constexpr int kBlockKElems = (KIND == KIND_F16) ? 64 : 128;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full_bar = empty_bar + STAGES;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOff + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&acc_full_bar[a], 1);
            ptx::mbar_init(&acc_empty_bar[a], 4);
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_base_slot, kTmemCols);
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TLOAD role
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                int mi, ni;
                tile_coords(tile, p, mi, ni);
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    ok = bounded_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, ST_PRODUCER_TIMEOUT, p.wait_limit);
                    if (!ok) {
                        break;
                    }
                    ptx::mbar_arrive_expect_tx(&full_bar[stage], ((L::kABytes + L::kBBytes) >> p.packed4) + L::kSfaBytes + L::kSfbBytes);
                    uint8_t* a_dst = smem + L::kAOff + stage * L::kABytes;
                    uint8_t* b_dst = smem + L::kBOff + stage * L::kBBytes;
                    ptx::tma_load_2d(a_dst, &tmap_a, &full_bar[stage], kb * kBlockKElems, mi * kBlockM);
                    if constexpr (B_MN_MAJOR) {
                        // B stored [K, N] row-major (the ND form of the CPU demo): boxes of 64 k-rows x 64 columns.
#pragma unroll
                        for (int j = 0; j < BLOCK_N / 64; ++j) {
                            ptx::tma_load_2d(b_dst + j * 8192, &tmap_b, &full_bar[stage], ni * BLOCK_N + j * 64,
                                             kb * kBlockKElems);
                        }
                    } else {
                        // B stored [N, K] row-major (= column-major K x N, the DN form of gemm_performance).
                        ptx::tma_load_2d(b_dst, &tmap_b, &full_bar[stage], kb * kBlockKElems, ni * BLOCK_N);
                    }
                    if constexpr (KIND == KIND_MXF8) {
                        constexpr int kNB = L::kSfbBytes / 512;
                        const uint8_t* sfa_src = p.sfa + (static_cast<size_t>(kb) * p.sf_a_blocks + mi) * 512;
                        const uint8_t* sfb_src =
                            p.sfb + (static_cast<size_t>(kb) * p.sf_b_blocks + static_cast<size_t>(ni) * kNB) * 512;
                        ptx::bulk_load_1d(smem + L::kSfaOff + stage * L::kSfaBytes, sfa_src, L::kSfaBytes,
                                          &full_bar[stage]);
                        ptx::bulk_load_1d(smem + L::kSfbOff + stage * L::kSfbBytes, sfb_src, L::kSfbBytes,
                                          &full_bar[stage]);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- TMATMUL / TMATMUL_ACC role
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                ok = bounded_wait(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag, p.status, ST_MMA_ACC_TIMEOUT, p.wait_limit);
                if (!ok) {
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kAccCols);
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    ok = bounded_wait(&full_bar[stage], phase, abort_flag, p.status, ST_MMA_FULL_TIMEOUT, p.wait_limit);
                    if (!ok) {
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_base = ptx::smem_u32(smem + L::kAOff + stage * L::kABytes);
                    const uint32_t b_base = ptx::smem_u32(smem + L::kBOff + stage * L::kBBytes);
                    if constexpr (KIND == KIND_MXF8) {
                        const uint32_t sfa_base = ptx::smem_u32(smem + L::kSfaOff + stage * L::kSfaBytes);
                        const uint32_t sfb_base = ptx::smem_u32(smem + L::kSfbOff + stage * L::kSfbBytes);
                        ptx::tmem_cp_32x128b_warpx4(tmem_base + kSfaCol,
                                                    ptx::make_smem_desc(sfa_base, 0, 128, ptx::kSwizzleNone));
#pragma unroll
                        for (int j = 0; j < L::kSfbBytes / 512; ++j) {
                            ptx::tmem_cp_32x128b_warpx4(
                                tmem_base + kSfbCol + 4u * j,
                                ptx::make_smem_desc(sfb_base + 512u * j, 0, 128, ptx::kSwizzleNone));
                        }
                    }
#pragma unroll
                    for (int kk = 0; kk < kBlockKBytes / kUmmaKBytes; ++kk) {
                        const uint64_t a_desc =
                            ptx::make_smem_desc(a_base + kk * kUmmaKBytes, 16, 1024, ptx::kSwizzle128B);
                        uint64_t b_desc;
                        if constexpr (B_MN_MAJOR) {
                            // 16 k-rows of 128 bytes per instruction; 64-column blocks 8 KiB apart.
                            b_desc = ptx::make_smem_desc(b_base + kk * 2048, 8192, 1024, ptx::kSwizzle128B);
                        } else {
                            b_desc = ptx::make_smem_desc(b_base + kk * kUmmaKBytes, 16, 1024, ptx::kSwizzle128B);
                        }
                        const uint32_t accumulate = (kb > 0 || kk > 0) ? 1u : 0u;
                        if constexpr (KIND == KIND_F16) {
                            ptx::umma_f16(d_tmem, a_desc, b_desc, p.idesc, accumulate);
                        } else if constexpr (KIND == KIND_I8) {
                            ptx::umma_i8(d_tmem, a_desc, b_desc, p.idesc, accumulate);
                        } else {
                            // scale-factor ids pick byte kk of each 32-bit scale column (one byte per 32 K-elements)
                            const uint32_t idesc =
                                p.idesc | (static_cast<uint32_t>(kk) << 4) | (static_cast<uint32_t>(kk) << 29);
                            ptx::umma_mxf8(d_tmem, a_desc, b_desc, idesc, tmem_base + kSfaCol, tmem_base + kSfbCol,
                                           accumulate);
                        }
                    }
                    ptx::umma_commit(&empty_bar[stage]);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) {
                    break;
                }
                ptx::umma_commit(&acc_full_bar[acc]);
                if (++acc == kNumAcc) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- TSTORE role
        const int quarter = warp & 3; // TMEM lanes this warp may read
        const int esize = (EPI == EPI_F32 || EPI == EPI_S32) ? 4 : (EPI == EPI_QUANT8 ? 1 : 2);
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0) && (((p.ldc * esize) & 15) == 0);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
            int mi, ni;
            tile_coords(tile, p, mi, ni);
            ok = bounded_wait(&acc_full_bar[acc], acc_phase, abort_flag, p.status, ST_EPILOGUE_TIMEOUT, p.wait_limit);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) {
                break;
            }
            ptx::tc_fence_after_sync();
            const int row = mi * kBlockM + quarter * 32 + lane;
            float s_row = 1.0f;
            if constexpr (EPI == EPI_DEQ_BF16) {
                s_row = (row < p.m) ? __ldg(p.s_row + row) : 0.0f;
            }
            const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * kAccCols) +
                                   (static_cast<uint32_t>(quarter * 32) << 16);
            // Read-back software-pipelined over 32-column chunks: the TMEM load of the next chunk is in flight while
            // the current one is converted and stored (columns past N are loaded but never stored), and the
            // accumulator goes back to the MMA role as soon as its last chunk is in registers.
            const int col_tile = ni * BLOCK_N;
            auto release_accumulator = [&]() {
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&acc_empty_bar[acc]);
                }
            };
            uint32_t va[32];
            ptx::tmem_ld_32x32b_x32(t_row, va);
            if constexpr (BLOCK_N == 32) {
                ptx::tmem_ld_wait();
                release_accumulator();
                store_chunk<EPI>(va, p, row, col_tile, vec_ok, s_row);
            } else {
                uint32_t vb[32];
#pragma unroll
                for (int g = 0; g < BLOCK_N / 64; ++g) {
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(g * 64 + 32), vb);
                    if (col_tile + g * 64 < p.n) {
                        store_chunk<EPI>(va, p, row, col_tile + g * 64, vec_ok, s_row);
                    }
                    ptx::tmem_ld_wait();
                    if (g + 1 < BLOCK_N / 64) {
                        ptx::tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(g * 64 + 64), va);
                    } else {
                        release_accumulator();
                    }
                    if (col_tile + g * 64 + 32 < p.n) {
                        store_chunk<EPI>(vb, p, row, col_tile + g * 64 + 32, vec_ok, s_row);
                    }
                }
            }
            if (++acc == kNumAcc) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // Let bulk copies and MMAs that were already issued finish before smem and TMEM go away.
        for (int i = 0; i < 2000; ++i) {
            __nanosleep(1000);
        }
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------- small helper kernels

// Re-tile e8m0 scale factors from the reference's row-major [rows, K/32] GM form (Layout::MX_A_ND for A,
// Layout::MX_B_DN for B; include/pto/common/pto_tile.hpp:883-910,1073-1102) into 512-byte atoms the
// tcgen05.cp 32x128b.warpx4 copy expects: atom (k_block, row_block) holds 128 rows x 4 scales with
// byte offset (r % 32) * 16 + (r / 32) * 4 + j. Rows / K-blocks past the end get 127 (= 2^0).
// One launch re-tiles both operands' scales: items [0, a_blocks * k_blocks * 128) belong to A, the rest to B.
__global__ void retile_scales_kernel(const uint8_t* __restrict__ src_a, uint8_t* __restrict__ dst_a, int rows_a,
                                     long long ld_a, int a_blocks, const uint8_t* __restrict__ src_b,
                                     uint8_t* __restrict__ dst_b, int rows_b, long long ld_b, int b_blocks, int k_groups,
                                     int k_blocks)
{
    const long long total_a = static_cast<long long>(a_blocks) * k_blocks * 128;
    const long long total = total_a + static_cast<long long>(b_blocks) * k_blocks * 128;
    for (long long it = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; it < total;
         it += static_cast<long long>(gridDim.x) * blockDim.x) {
        const bool is_a = it < total_a;
        const long long i = is_a ? it : it - total_a;
        const uint8_t* src = is_a ? src_a : src_b;
        uint8_t* dst = is_a ? dst_a : dst_b;
        const int rows = is_a ? rows_a : rows_b;
        const long long ld = is_a ? ld_a : ld_b;
        const int row_blocks = is_a ? a_blocks : b_blocks;
        const int r_in = static_cast<int>(i % 128);
        const long long atom = i / 128;
        const int rb = static_cast<int>(atom % row_blocks);
        const int kb = static_cast<int>(atom / row_blocks);
        const int row = rb * 128 + r_in;
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kg = kb * 4 + j;
            uint32_t b = 127u;
            if (row < rows && kg < k_groups) {
                b = src[static_cast<long long>(row) * ld + kg];
            }
            word |= b << (8 * j);
        }
        uint32_t* out = reinterpret_cast<uint32_t*>(dst + atom * 512 + (r_in % 32) * 16 + (r_in / 32) * 4);
        *out = word;
    }
}

// fp32 -> bf16 (round to nearest even) over a contiguous buffer; used after the K-split reduction.
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long count)
{
    const long long n4 = count / 4;
    const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = tid; i < n4; i += stride) {
        const float4 f = reinterpret_cast<const float4*>(src)[i];
        const __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(f.z, f.w);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        reinterpret_cast<uint2*>(dst)[i] = o;
    }
    for (long long i = n4 * 4 + tid; i < count; i += stride) {
        dst[i] = __float2bfloat16_rn(src[i]);
    }
}

} // namespace pto_b200
