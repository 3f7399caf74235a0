// pto-inst.hpp - the PTO tile-program surface for the GEMM hot path, hosted on a B200.
//
// The reference's tile instructions run inside an AI core on tiles that live in L1 / L0A / L0B / L0C
// (include/pto/common/pto_tile.hpp, pto_instr.hpp). On a B200 the whole tile loop is one kernel, so here a
// tile program is written on the HOST with the same types and instruction names and is executed lazily:
//
//   TLOAD    binds a Mat/Left/Right/Scale tile to the GlobalTensor region it was loaded from (no copy);
//   TMOV / TEXTRACT derive a tile bound to (a sub-window of) the source tile's region;
//   TMATMUL  starts, TMATMUL_ACC / the accumulating TMATMUL_MX extend, the product chain held by the Acc tile;
//   TSTORE   launches ONE tcgen05 GEMM over the whole chain through the C ABI (include/pto_b200.h) when the
//            chain's K slices are contiguous in memory - which is what the reference's K loops produce
//            (kernels/manual/a2a3/gemm_performance/gemm_performance_kernel.cpp:220-231) - and reports an error
//            otherwise.
//
// Template parameter order and names follow the reference (Tile: pto_tile.hpp:1422-1428; TileLeft/Right/Acc/
// LeftScale/RightScale: :1785-1830; GlobalTensor: :276-277; Shape/Stride: :34-261; TileShape2D/BaseShape2D:
// :745-847; enums: include/pto/common/type.hpp:121-187,232-252,301-322,356-361). Only what the GEMM path uses is
// provided. There is no CPU execution path: without the CUDA library nothing here computes.
#ifndef PTO_B200_PTO_INST_HPP
#define PTO_B200_PTO_INST_HPP

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <type_traits>
#include <vector>

#include "../pto_b200.h"

#define PTO_INST inline
#define PTO_INTERNAL inline
#ifndef __gm__
#define __gm__
#endif
#ifndef AICORE
#define AICORE
#endif

namespace pto {

constexpr int DYNAMIC = -1;
constexpr int MX_BLOCK_SIZE = 32; // include/pto/common/constants.hpp:42

enum class TileType { Vec, Mat, Left, Right, Acc, Bias, Scaling, ScaleLeft, ScaleRight, Ctrl };
enum class BLayout { RowMajor = 0, ColMajor = 1 };
enum class SLayout { NoneBox = 0, RowMajor = 1, ColMajor = 2 };
enum class Layout { ND, DN, NZ, SCALE, MX_A_ND, MX_A_DN, MX_A_ZZ, MX_B_ND, MX_B_DN, MX_B_NN, MAX };
enum class STPhase : uint8_t { Unspecified = 0x0, Partial = 0x2, Final = 0x3 };
enum class AccPhase : uint8_t { Unspecified = 0x0, Unknown = Unspecified, Partial = 0x2, Final = 0x3 };
enum class ReluPreMode : uint8_t { NoRelu = 0, NormalRelu = 1 };
enum class AtomicType : uint8_t { AtomicNone = 0, AtomicAdd = 1 };
enum class PadValue : uint64_t { Null = 0, Zero = 1, Max = 2, Min = 3 };
enum class CompactMode { Null, Normal, RowPlusOne, RowAlignedPadding };

struct TileConfig {
    static constexpr int fractalABSize = 512;
    static constexpr int fractalCSize = 1024;
    static constexpr int fractalMxSize = 32;
};

// ---------------------------------------------------------------- element types (storage only on the host)
struct half { uint16_t bits; };
struct bfloat16_t { uint16_t bits; };
struct float8_e4m3_t { uint8_t data; };
struct float8_e5m2_t { uint8_t data; };
struct float8_e8m0_t { uint8_t data; };

namespace b200 {

template <typename T> struct dtype_of { static constexpr int value = -1; };
template <> struct dtype_of<half> { static constexpr int value = PTO_B200_F16; };
template <> struct dtype_of<uint16_t> { static constexpr int value = PTO_B200_F16; }; // LaunchGEMME2E<uint16_t>
template <> struct dtype_of<bfloat16_t> { static constexpr int value = PTO_B200_BF16; };
template <> struct dtype_of<float> { static constexpr int value = PTO_B200_F32; };
template <> struct dtype_of<int8_t> { static constexpr int value = PTO_B200_S8; };
template <> struct dtype_of<uint8_t> { static constexpr int value = PTO_B200_U8; };
template <> struct dtype_of<int16_t> { static constexpr int value = PTO_B200_S16; };
template <> struct dtype_of<int32_t> { static constexpr int value = PTO_B200_S32; };
template <> struct dtype_of<float8_e4m3_t> { static constexpr int value = PTO_B200_E4M3; };
template <> struct dtype_of<float8_e5m2_t> { static constexpr int value = PTO_B200_E5M2; };

// Errors follow the CPU simulator's PTO_CPU_ASSERT behaviour (message, then abort; include/pto/common/type.hpp:70-92)
// unless a handler is installed.
using ErrorHandler = void (*)(const char* what, int code);
inline ErrorHandler& error_handler()
{
    static ErrorHandler h = nullptr;
    return h;
}
inline void fail(const char* what, int code)
{
    if (error_handler() != nullptr) {
        error_handler()(what, code);
        return;
    }
    std::fprintf(stderr, "[PTO][B200] %s (%s)\n", what, code ? pto_b200_error_string(code) : "tile program");
    std::abort();
}

// The CUDA stream tile programs launch on (thread-local; the reference passes `void* stream` to its launchers).
inline void*& current_stream()
{
    thread_local void* s = nullptr;
    return s;
}
inline void set_stream(void* stream) { current_stream() = stream; }

// Optional device scratch for tile programs whose TSTORE needs one (block-scaled chains: the re-tiled scale factors).
// Without it a block-scaled chain uses the library's built-in array (pto_b200_gemm_mx_static); the bias form of a
// block-scaled chain has no such variant and needs this workspace.
struct Workspace {
    uint8_t* ptr = nullptr;
    size_t bytes = 0;
};
inline Workspace& current_workspace()
{
    thread_local Workspace w;
    return w;
}
inline void set_workspace(void* ptr, size_t bytes)
{
    current_workspace().ptr = static_cast<uint8_t*>(ptr);
    current_workspace().bytes = bytes;
}

// A bound tile: a rows x cols window of device memory with element strides.
struct View {
    const uint8_t* ptr = nullptr;
    long long rows = 0, cols = 0;
    long long row_stride = 0, col_stride = 0; // elements
    int elem_size = 0;
    bool bound() const { return ptr != nullptr; }
};

struct Product {
    View a, b, sa, sb;
    bool mx = false;
    int a_dtype = -1, b_dtype = -1; // pto_b200_dtype of the operand tiles
};

} // namespace b200

// ---------------------------------------------------------------- Shape / Stride / GlobalTensor
template <int64_t N1 = DYNAMIC, int64_t N2 = DYNAMIC, int64_t N3 = DYNAMIC, int64_t N4 = DYNAMIC, int64_t N5 = DYNAMIC>
struct Shape {
    static constexpr int64_t staticShape[5] = {N1, N2, N3, N4, N5};
    int64_t shape[5] = {N1, N2, N3, N4, N5};
    Shape() = default;
    Shape(int64_t a, int64_t b, int64_t c, int64_t d, int64_t e) : shape{a, b, c, d, e} {}
};

template <int64_t S1 = DYNAMIC, int64_t S2 = DYNAMIC, int64_t S3 = DYNAMIC, int64_t S4 = DYNAMIC, int64_t S5 = DYNAMIC>
struct Stride {
    static constexpr int64_t staticStride[5] = {S1, S2, S3, S4, S5};
    int64_t stride[5] = {S1, S2, S3, S4, S5};
    Stride() = default;
    Stride(int64_t a, int64_t b, int64_t c, int64_t d, int64_t e) : stride{a, b, c, d, e} {}
};

// A 2-D window [rows, cols] of a tensor (the last two of five dimensions).
template <typename T, int64_t rows, int64_t cols, Layout L = Layout::ND>
struct TileShape2D : public Shape<1, 1, 1, rows, cols> {
    using Parent = Shape<1, 1, 1, rows, cols>;
    TileShape2D() = default;
    TileShape2D(int64_t dynamicRows, int64_t dynamicCols) : Parent(1, 1, 1, dynamicRows, dynamicCols) {}
};

// Strides of the whole [rows, cols] tensor a window is cut from. ND / MX_A_ND: row-major (cols, 1);
// DN / MX_B_DN: column-major (1, rows).
template <typename T, int64_t rows, int64_t cols, Layout L = Layout::ND>
struct BaseShape2D : public Stride<rows * cols, rows * cols, rows * cols, cols, 1> {
    using Parent = Stride<rows * cols, rows * cols, rows * cols, cols, 1>;
    BaseShape2D() = default;
    BaseShape2D(int64_t dynamicRows, int64_t dynamicCols)
        : Parent(dynamicRows * dynamicCols, dynamicRows * dynamicCols, dynamicRows * dynamicCols, dynamicCols, 1)
    {}
};
template <typename T, int64_t rows, int64_t cols>
struct BaseShape2D<T, rows, cols, Layout::DN> : public Stride<rows * cols, rows * cols, rows * cols, 1, rows> {
    using Parent = Stride<rows * cols, rows * cols, rows * cols, 1, rows>;
    BaseShape2D() = default;
    BaseShape2D(int64_t dynamicRows, int64_t dynamicCols)
        : Parent(dynamicRows * dynamicCols, dynamicRows * dynamicCols, dynamicRows * dynamicCols, 1, dynamicRows)
    {}
};
template <typename T, int64_t rows, int64_t cols>
struct BaseShape2D<T, rows, cols, Layout::MX_A_ND> : public BaseShape2D<T, rows, cols, Layout::ND> {
    using BaseShape2D<T, rows, cols, Layout::ND>::BaseShape2D;
};
template <typename T, int64_t rows, int64_t cols>
struct BaseShape2D<T, rows, cols, Layout::MX_B_DN> : public BaseShape2D<T, rows, cols, Layout::DN> {
    using BaseShape2D<T, rows, cols, Layout::DN>::BaseShape2D;
};

template <typename Element_, typename Shape_, typename Stride_, Layout Layout_ = Layout::ND>
struct GlobalTensor {
    using Shape = Shape_;
    using Stride = Stride_;
    using RawDType = Element_;
    using DType = Element_;
    static constexpr Layout layout = Layout_;

    GlobalTensor(DType* data, const Shape& shape = Shape(), const Stride& stride = Stride())
        : data_(data), shape_(shape), stride_(stride)
    {}
    DType* data() const { return data_; }
    int64_t GetShape(int dim) const { return shape_.shape[dim]; }
    int64_t GetStride(int dim) const { return stride_.stride[dim]; }

private:
    DType* data_;
    Shape shape_;
    Stride stride_;
};

// ---------------------------------------------------------------- Tile
template <TileType Loc_, typename Element_, const int Rows_, const int Cols_, const BLayout BFractal_ = BLayout::RowMajor,
          const int RowValid_ = Rows_, const int ColValid_ = Cols_, const SLayout SFractal_ = SLayout::NoneBox,
          const int SFractalSize_ = TileConfig::fractalABSize, auto PadVal_ = PadValue::Null,
          const CompactMode Compact_ = CompactMode::Null>
struct Tile {
    using DType = Element_;
    static constexpr TileType Loc = Loc_;
    static constexpr int Rows = Rows_;
    static constexpr int Cols = Cols_;
    static constexpr int ValidRow = RowValid_;
    static constexpr int ValidCol = ColValid_;
    static constexpr BLayout BFractal = BFractal_;
    static constexpr SLayout SFractal = SFractal_;
    static constexpr bool isRowMajor = (BFractal_ == BLayout::RowMajor);

    int GetValidRow() const { return ValidRow; }
    int GetValidCol() const { return ValidCol; }

    // host-side state of the lazily executed tile program
    b200::View view;                      // Mat / Left / Right / Scale tiles: where the data lives
    std::vector<b200::Product> products;  // Acc tiles: the pending TMATMUL(+_ACC) chain
    b200::View bias;                      // Acc tiles: the bias row of a TMATMUL_BIAS / TGEMV_BIAS chain, if any
    bool one_row = false;                 // Acc tiles: the chain was started by TGEMV (one left row)
    uint64_t assigned_addr = 0;           // TASSIGN bookkeeping only
};

template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileLeft = Tile<TileType::Left, Element_, Rows_, Cols_, BLayout::ColMajor, RowValid_, ColValid_, SLayout::RowMajor,
                      TileConfig::fractalABSize>;
template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileRight = Tile<TileType::Right, Element_, Rows_, Cols_, BLayout::RowMajor, RowValid_, ColValid_, SLayout::ColMajor,
                       TileConfig::fractalABSize>;
template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileLeftScale = Tile<TileType::ScaleLeft, Element_, Rows_, Cols_, BLayout::RowMajor, RowValid_, ColValid_,
                           SLayout::RowMajor, TileConfig::fractalMxSize>;
template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileRightScale = Tile<TileType::ScaleRight, Element_, Rows_, Cols_, BLayout::ColMajor, RowValid_, ColValid_,
                            SLayout::ColMajor, TileConfig::fractalMxSize>;
template <typename Element_, const int Rows_, const int Cols_, const int RowValid_ = Rows_, const int ColValid_ = Cols_>
using TileAcc = Tile<TileType::Acc, Element_, Rows_, Cols_, BLayout::ColMajor, RowValid_, ColValid_, SLayout::RowMajor,
                     TileConfig::fractalCSize>;

struct RecordEvent {}; // instructions return an event in the reference (pto_instr.hpp:70-79); ordering here is the stream's

// ---------------------------------------------------------------- legality (CheckMadValid, cpu/TMatmul.hpp:31-75,121-142)
namespace b200 {
template <typename TileAcc_, typename TileLeft_, typename TileRight_>
constexpr void check_mad_valid()
{
    using A = typename TileLeft_::DType;
    using B = typename TileRight_::DType;
    using C = typename TileAcc_::DType;
    static_assert((std::is_same_v<A, int8_t> && std::is_same_v<B, int8_t> && std::is_same_v<C, int32_t>) ||
                      (std::is_same_v<A, half> && std::is_same_v<B, half> && std::is_same_v<C, float>) ||
                      (std::is_same_v<A, bfloat16_t> && std::is_same_v<B, bfloat16_t> && std::is_same_v<C, float>),
                  "[PTO][SA] Not supported data type");
    static_assert((TileLeft_::Rows == TileAcc_::Rows) && (TileLeft_::Cols == TileRight_::Rows) &&
                      (TileRight_::Cols == TileAcc_::Cols),
                  "[PTO][SA] Inconsistent number of m, k, n");
    static_assert(TileLeft_::Loc == TileType::Left && TileRight_::Loc == TileType::Right && TileAcc_::Loc == TileType::Acc,
                  "[PTO][SA] Non-conforming matrix fractal");
}

template <typename TileAcc_, typename TileLeft_, typename TileRight_>
constexpr void check_mad_mx_valid()
{
    using A = typename TileLeft_::DType;
    using B = typename TileRight_::DType;
    constexpr bool a8 = std::is_same_v<A, float8_e4m3_t> || std::is_same_v<A, float8_e5m2_t>;
    constexpr bool b8 = std::is_same_v<B, float8_e4m3_t> || std::is_same_v<B, float8_e5m2_t>;
    static_assert(a8 && b8 && std::is_same_v<typename TileAcc_::DType, float>,
                  "[PTO][SA] TMatmulMX:No supported data type combination.");
    static_assert(TileLeft_::Cols % 64 == 0, "[PTO][SA] TMatmulMX: aMatrixCol must be a multiple of 64.");
}
} // namespace b200

// ---------------------------------------------------------------- instructions
template <typename TileData>
PTO_INST RecordEvent TASSIGN(TileData& tile, uint64_t addr)
{
    tile.assigned_addr = addr; // on-chip placement is the kernel's business on a B200 (stage ring / TMEM columns)
    return {};
}

template <typename TileData, typename GlobalData>
PTO_INST RecordEvent TLOAD(TileData& dst, GlobalData& src)
{
    static_assert(sizeof(typename TileData::DType) == sizeof(typename GlobalData::DType), "[PTO][SA] TLOAD dtype mismatch");
    b200::View v;
    v.ptr = reinterpret_cast<const uint8_t*>(src.data());
    v.rows = src.GetShape(3);
    v.cols = src.GetShape(4);
    v.row_stride = src.GetStride(3);
    v.col_stride = src.GetStride(4);
    v.elem_size = static_cast<int>(sizeof(typename TileData::DType));
    if (v.rows == DYNAMIC || v.cols == DYNAMIC) {
        b200::fail("TLOAD: dynamic shape without run-time values", 0);
    }
    dst.view = v;
    return {};
}

template <typename DstTile, typename SrcTile>
PTO_INST RecordEvent TMOV(DstTile& dst, SrcTile& src)
{
    dst.view = src.view;
    return {};
}

// dst = the DstTile::Rows x DstTile::Cols window of src starting at (indexRow, indexCol).
template <typename DstTile, typename SrcTile>
PTO_INST RecordEvent TEXTRACT(DstTile& dst, SrcTile& src, uint16_t indexRow = 0, uint16_t indexCol = 0)
{
    if (!src.view.bound()) {
        b200::fail("TEXTRACT: source tile was never loaded", 0);
    }
    b200::View v = src.view;
    v.ptr += (static_cast<long long>(indexRow) * v.row_stride + static_cast<long long>(indexCol) * v.col_stride) * v.elem_size;
    v.rows = DstTile::ValidRow < v.rows - indexRow ? DstTile::ValidRow : v.rows - indexRow;
    v.cols = DstTile::ValidCol < v.cols - indexCol ? DstTile::ValidCol : v.cols - indexCol;
    dst.view = v;
    return {};
}

template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileRight_>
PTO_INST RecordEvent TMATMUL(TileRes& cMatrix, TileLeft_& aMatrix, TileRight_& bMatrix)
{
    b200::check_mad_valid<TileRes, TileLeft_, TileRight_>();
    cMatrix.products.clear();
    cMatrix.bias = b200::View{};
    cMatrix.one_row = false;
    cMatrix.products.push_back(b200::Product{aMatrix.view, bMatrix.view, {}, {}, false,
                                             b200::dtype_of<typename TileLeft_::DType>::value,
                                             b200::dtype_of<typename TileRight_::DType>::value});
    return {};
}

// Bias legality (CheckBiasValid, cpu/TMatmul.hpp:159-167): bias type == accumulator type, one row-major row.
template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileRight_,
          typename TileBias_>
PTO_INST RecordEvent TMATMUL_BIAS(TileRes& cMatrix, TileLeft_& aMatrix, TileRight_& bMatrix, TileBias_& biasData)
{
    static_assert(std::is_same_v<typename TileRes::DType, typename TileBias_::DType>, "[PTO][SA] No supported bias data type");
    static_assert(TileBias_::Loc == TileType::Bias && TileBias_::Rows == 1 && TileBias_::isRowMajor,
                  "[PTO][SA] Non-conforming bias fractal");
    TMATMUL<Phase>(cMatrix, aMatrix, bMatrix);
    if (!biasData.view.bound()) {
        b200::fail("TMATMUL_BIAS: bias tile was never loaded", 0);
    }
    cMatrix.bias = biasData.view;
    return {};
}

// One left row (cpu/TMatmul.hpp:232-252: the TMATMUL arithmetic): TSTORE then streams B once instead of running
// 128-row tensor-core tiles.
template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileRight_>
PTO_INST RecordEvent TGEMV(TileRes& cMatrix, TileLeft_& aMatrix, TileRight_& bMatrix)
{
    TMATMUL<Phase>(cMatrix, aMatrix, bMatrix);
    cMatrix.one_row = true;
    return {};
}

// The accumulating forms are declared after TMATMUL_ACC below.
template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileRight_,
          typename TileBias_>
PTO_INST RecordEvent TGEMV_BIAS(TileRes& cMatrix, TileLeft_& aMatrix, TileRight_& bMatrix, TileBias_& biasData)
{
    TMATMUL_BIAS<Phase>(cMatrix, aMatrix, bMatrix, biasData);
    cMatrix.one_row = true;
    return {};
}

template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileRight_>
PTO_INST RecordEvent TMATMUL_ACC(TileRes& cOutMatrix, TileRes& cInMatrix, TileLeft_& aMatrix, TileRight_& bMatrix)
{
    b200::check_mad_valid<TileRes, TileLeft_, TileRight_>();
    if (&cOutMatrix != &cInMatrix) {
        cOutMatrix.products = cInMatrix.products;
        cOutMatrix.bias = cInMatrix.bias;
        cOutMatrix.one_row = cInMatrix.one_row;
    }
    cOutMatrix.products.push_back(b200::Product{aMatrix.view, bMatrix.view, {}, {}, false,
                                                b200::dtype_of<typename TileLeft_::DType>::value,
                                                b200::dtype_of<typename TileRight_::DType>::value});
    return {};
}

// TGEMV_ACC (cpu/TMatmul.hpp:239-244): the next K slice of a one-row chain.
template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileRight_>
PTO_INST RecordEvent TGEMV_ACC(TileRes& cOutMatrix, TileRes& cInMatrix, TileLeft_& aMatrix, TileRight_& bMatrix)
{
    return TMATMUL_ACC<Phase>(cOutMatrix, cInMatrix, aMatrix, bMatrix);
}

template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileLeftScale_,
          typename TileRight_, typename TileRightScale_>
PTO_INST RecordEvent TMATMUL_MX(TileRes& cMatrix, TileLeft_& aMatrix, TileLeftScale_& aScaleMatrix, TileRight_& bMatrix,
                                TileRightScale_& bScaleMatrix)
{
    b200::check_mad_mx_valid<TileRes, TileLeft_, TileRight_>();
    cMatrix.products.clear();
    cMatrix.bias = b200::View{};
    cMatrix.one_row = false;
    cMatrix.products.push_back(b200::Product{aMatrix.view, bMatrix.view, aScaleMatrix.view, bScaleMatrix.view, true,
                                             b200::dtype_of<typename TileLeft_::DType>::value,
                                             b200::dtype_of<typename TileRight_::DType>::value});
    return {};
}

// The bias form (include/pto/common/pto_instr.hpp:918-942): one fp32 value per column joins the accumulator.
template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileLeftScale_,
          typename TileRight_, typename TileRightScale_, typename TileBias_,
          std::enable_if_t<TileBias_::Loc == TileType::Bias, int> = 0>
PTO_INST RecordEvent TMATMUL_MX(TileRes& cMatrix, TileLeft_& aMatrix, TileLeftScale_& aScaleMatrix, TileRight_& bMatrix,
                                TileRightScale_& bScaleMatrix, TileBias_& biasData)
{
    static_assert(std::is_same_v<typename TileBias_::DType, float> && TileBias_::Rows == 1,
                  "[PTO][SA] TMatmulMX: the bias is one row of float");
    TMATMUL_MX<Phase>(cMatrix, aMatrix, aScaleMatrix, bMatrix, bScaleMatrix);
    if (!biasData.view.bound()) {
        b200::fail("TMATMUL_MX: bias tile was never loaded", 0);
    }
    cMatrix.bias = biasData.view;
    return {};
}

template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileLeftScale_,
          typename TileRight_, typename TileRightScale_,
          std::enable_if_t<TileRight_::Loc == TileType::Right, int> = 0>
PTO_INST RecordEvent TMATMUL_MX(TileRes& cOutMatrix, TileRes& cInMatrix, TileLeft_& aMatrix, TileLeftScale_& aScaleMatrix,
                                TileRight_& bMatrix, TileRightScale_& bScaleMatrix)
{
    b200::check_mad_mx_valid<TileRes, TileLeft_, TileRight_>();
    if (&cOutMatrix != &cInMatrix) {
        cOutMatrix.products = cInMatrix.products;
        cOutMatrix.bias = cInMatrix.bias;
    }
    cOutMatrix.products.push_back(b200::Product{aMatrix.view, bMatrix.view, aScaleMatrix.view, bScaleMatrix.view, true,
                                                b200::dtype_of<typename TileLeft_::DType>::value,
                                                b200::dtype_of<typename TileRight_::DType>::value});
    return {};
}

// TGEMV_MX (include/pto/common/pto_instr.hpp:797-862): the block-scaled forms with a one-row left tile; TSTORE then
// streams B and its scales once (pto_b200_gemv_mx) instead of running 128-row tensor-core tiles.
template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileLeftScale_,
          typename TileRight_, typename TileRightScale_>
PTO_INST RecordEvent TGEMV_MX(TileRes& cMatrix, TileLeft_& aMatrix, TileLeftScale_& aScaleMatrix, TileRight_& bMatrix,
                              TileRightScale_& bScaleMatrix)
{
    TMATMUL_MX<Phase>(cMatrix, aMatrix, aScaleMatrix, bMatrix, bScaleMatrix);
    cMatrix.one_row = true;
    return {};
}

template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileLeftScale_,
          typename TileRight_, typename TileRightScale_, std::enable_if_t<TileRight_::Loc == TileType::Right, int> = 0>
PTO_INST RecordEvent TGEMV_MX(TileRes& cOutMatrix, TileRes& cInMatrix, TileLeft_& aMatrix, TileLeftScale_& aScaleMatrix,
                              TileRight_& bMatrix, TileRightScale_& bScaleMatrix)
{
    TMATMUL_MX<Phase>(cOutMatrix, cInMatrix, aMatrix, aScaleMatrix, bMatrix, bScaleMatrix);
    cOutMatrix.one_row = (&cOutMatrix == &cInMatrix) ? cOutMatrix.one_row : cInMatrix.one_row;
    return {};
}

template <AccPhase Phase = AccPhase::Unspecified, typename TileRes, typename TileLeft_, typename TileLeftScale_,
          typename TileRight_, typename TileRightScale_, typename TileBias_,
          std::enable_if_t<TileBias_::Loc == TileType::Bias, int> = 0>
PTO_INST RecordEvent TGEMV_MX(TileRes& cMatrix, TileLeft_& aMatrix, TileLeftScale_& aScaleMatrix, TileRight_& bMatrix,
                              TileRightScale_& bScaleMatrix, TileBias_& biasData)
{
    TMATMUL_MX<Phase>(cMatrix, aMatrix, aScaleMatrix, bMatrix, bScaleMatrix, biasData);
    cMatrix.one_row = true;
    return {};
}

namespace b200 {
// true if `next` continues `prev` along K: A windows side by side in a row-major matrix.
inline bool a_continues(const View& prev, const View& next)
{
    return next.ptr == prev.ptr + prev.cols * prev.col_stride * prev.elem_size && next.rows == prev.rows &&
           next.row_stride == prev.row_stride && next.col_stride == prev.col_stride;
}
// B windows stacked along their rows (the K axis of the logical K x N matrix).
inline bool b_continues(const View& prev, const View& next)
{
    return next.ptr == prev.ptr + prev.rows * prev.row_stride * prev.elem_size && next.cols == prev.cols &&
           next.row_stride == prev.row_stride && next.col_stride == prev.col_stride;
}

// The pre-quant part of a TSTORE: none, one scale word for the tile, or one word per column.
struct StoreQuant {
    bool on = false;
    uint64_t scalar = 0;
    const uint8_t* words = nullptr; // device memory, n 64-bit words
    long long word_count = 0;
    bool relu = false;
};

// Launch the GEMM of an accumulator tile's pending product chain and store into dst.
template <typename TileAcc_, typename GlobalData>
inline void store_chain(GlobalData& dst, TileAcc_& src, const StoreQuant& quant)
{
    static_assert(TileAcc_::Loc == TileType::Acc, "[PTO][SA] this TSTORE form takes an accumulator tile");
    if (src.products.empty()) {
        fail("TSTORE: accumulator tile holds no TMATMUL result", 0);
        return;
    }
    const Product& first = src.products.front();
    View a = first.a, b = first.b, sa = first.sa, sb = first.sb;
    long long k_total = a.cols;
    for (size_t i = 1; i < src.products.size(); ++i) {
        const Product& prev = src.products[i - 1];
        const Product& cur = src.products[i];
        if (cur.mx != first.mx || !a_continues(prev.a, cur.a) || !b_continues(prev.b, cur.b)) {
            fail("TSTORE: the TMATMUL_ACC chain is not a run of adjacent K slices; only such chains map to one GEMM", 0);
            return;
        }
        // block-scaled chains: the scale windows must continue the same way, one scale per 32 K elements, or the one
        // GEMM over the whole K would read scales the program never named
        if (first.mx && (!a_continues(prev.sa, cur.sa) || !b_continues(prev.sb, cur.sb) ||
                         prev.sa.cols * MX_BLOCK_SIZE != prev.a.cols || prev.sb.rows * MX_BLOCK_SIZE != prev.b.rows)) {
            fail("TSTORE: the scale tiles of the TMATMUL_MX chain are not adjacent K/32 slices of one scale tensor", 0);
            return;
        }
        k_total += cur.a.cols;
    }
    if (!a.bound() || !b.bound() || a.col_stride != 1 || b.rows != a.cols) {
        fail("TSTORE: operand tiles are not bound to row-major A / K x N B regions", 0);
        return;
    }
    const int m = static_cast<int>(a.rows);
    const int n = static_cast<int>(b.cols);
    if (dst.GetShape(3) < m || dst.GetShape(4) < n) {
        fail("TSTORE: the destination tensor is smaller than the accumulator tile's m x n", 0);
        return;
    }
    // B: DN (element (k, n) at k + n * ld) -> col_stride = ld, row_stride = 1; ND -> row_stride = ld, col_stride = 1
    const bool b_dn = (b.row_stride == 1);
    const long long ldb = b_dn ? b.col_stride : b.row_stride;
    const long long ldc = dst.GetStride(3);
    if (dst.GetStride(4) != 1) {
        fail("TSTORE: destination must be row-major (ND)", 0);
        return;
    }
    using OutT = typename GlobalData::DType;
    uint8_t* out = reinterpret_cast<uint8_t*>(dst.data());
    void* stream = current_stream();
    const int k = static_cast<int>(k_total);
    int rc;
    if (quant.on) {
        if (first.mx || src.bias.bound() || !b_dn) {
            fail("TSTORE: the pre-quant forms apply to TMATMUL / TMATMUL_ACC chains with a column-major B and no bias", 0);
            return;
        }
        if (quant.words != nullptr && quant.word_count < n) {
            fail("TSTORE: the scaling tile has fewer words than the accumulator has columns", 0);
            return;
        }
        rc = pto_b200_gemm_quant(stream, out, a.ptr, b.ptr, m, n, k, a.row_stride, ldb, ldc, first.a_dtype,
                                 dtype_of<OutT>::value, quant.scalar,
                                 reinterpret_cast<const unsigned long long*>(quant.words), quant.relu ? 1 : 0);
    } else if (first.mx) {
        // scale tensors: A's is row-major [m, K/32] (MX_A_ND), B's holds the K/32 scales of a column contiguously
        // (MX_B_DN: element (kg, n) at kg + n * ld), the layouts TLOAD binds for the reference's MX kernels
        if (sa.col_stride != 1 || sb.row_stride != 1 || !b_dn) {
            fail("TSTORE: TMATMUL_MX chains take MX_A_ND / MX_B_DN scale tensors and a column-major B", 0);
            return;
        }
        const long long ld_sfa = sa.row_stride, ld_sfb = sb.col_stride;
        const Workspace& ws = current_workspace();
        rc = PTO_B200_EALIGN;
        if (src.one_row && m == 1) { // TGEMV_MX: no workspace, no tensor-core tile
            rc = pto_b200_gemv_mx(stream, out, a.ptr, b.ptr, sa.ptr, sb.ptr, src.bias.ptr, n, k, ldb, ld_sfb, first.a_dtype,
                                  first.b_dtype, dtype_of<OutT>::value);
        }
        if (rc != PTO_B200_EALIGN) {
            // launched (or rejected for a reason other than the row's alignment)
        } else if (src.bias.bound()) {
            if (ws.ptr == nullptr) {
                fail("TSTORE: the bias form of TMATMUL_MX needs scratch: call pto::b200::set_workspace first", 0);
                return;
            }
            rc = pto_b200_gemm_mx_bias(stream, out, a.ptr, b.ptr, sa.ptr, sb.ptr, src.bias.ptr, ws.ptr, ws.bytes, m, n, k,
                                       a.row_stride, ldb, ldc, ld_sfa, ld_sfb, first.a_dtype, first.b_dtype,
                                       dtype_of<OutT>::value);
        } else if (ws.ptr != nullptr) {
            rc = pto_b200_gemm_mx(stream, out, a.ptr, b.ptr, sa.ptr, sb.ptr, ws.ptr, ws.bytes, m, n, k, a.row_stride, ldb,
                                  ldc, ld_sfa, ld_sfb, first.a_dtype, first.b_dtype, dtype_of<OutT>::value);
        } else {
            rc = pto_b200_gemm_mx_static(stream, out, a.ptr, b.ptr, sa.ptr, sb.ptr, m, n, k, a.row_stride, ldb, ldc,
                                         ld_sfa, ld_sfb, first.a_dtype, first.b_dtype, dtype_of<OutT>::value);
        }
    } else {
        rc = PTO_B200_EALIGN;
        if (src.one_row && m == 1 && b_dn) {
            rc = pto_b200_gemv(stream, out, a.ptr, b.ptr, src.bias.ptr, n, k, ldb, first.a_dtype, dtype_of<OutT>::value);
        }
        if (rc == PTO_B200_EALIGN && src.bias.bound()) { // not a one-row chain, or its row is not 16-byte aligned
            rc = pto_b200_gemm_bias(stream, out, a.ptr, b.ptr, src.bias.ptr, m, n, k, a.row_stride, ldb, ldc, first.a_dtype,
                                    dtype_of<OutT>::value, b_dn ? PTO_B200_B_DN : PTO_B200_B_ND);
        } else if (rc == PTO_B200_EALIGN) {
            rc = pto_b200_gemm(stream, out, a.ptr, b.ptr, m, n, k, a.row_stride, ldb, ldc, first.a_dtype,
                               dtype_of<OutT>::value, b_dn ? PTO_B200_B_DN : PTO_B200_B_ND);
        }
    }
    if (rc != PTO_B200_OK) {
        fail("TSTORE: launch rejected", rc);
    }
}

// CheckStoreQuantValid: the pre-quant forms implemented here take int32 or float accumulators to half / bfloat16
// (QS322BF16_PRE, VQS322BF16_PRE, DEQF16, VDEQF16, QF322BF16_PRE, VQF322BF16_PRE, QF322F16_PRE, VQF322F16_PRE of
// include/pto/cpu/common.hpp:19-37), to int8_t / uint8_t (REQ8, VREQ8, QF322B8_PRE, VQF322B8_PRE) and, from int32
// accumulators, to int16_t (SHIFTS322S16, VSHIFTS322S16).
template <typename TileData, typename GlobalData>
constexpr void check_store_quant_valid()
{
    using S = typename TileData::DType;
    using D = typename GlobalData::DType;
    static_assert((std::is_same_v<S, int32_t> || std::is_same_v<S, float>) &&
                      (std::is_same_v<D, half> || std::is_same_v<D, bfloat16_t> || std::is_same_v<D, int8_t> ||
                       std::is_same_v<D, uint8_t> || (std::is_same_v<D, int16_t> && std::is_same_v<S, int32_t>)),
                  "[PTO][SA] TSTORE pre-quant: int32 / float accumulators to half / bfloat16_t / int8_t / uint8_t, int32 "
                  "accumulators to int16_t");
}
} // namespace b200

// TSTORE of an accumulator tile: launches the GEMM for the pending product chain and stores cast(acc) to dst
// (include/pto/common/pto_instr.hpp:378-439). Template parameter order as in the reference: tile, tensor, atomic, relu.
template <typename TileData, typename GlobalData, AtomicType atomicType = AtomicType::AtomicNone,
          ReluPreMode reluPreMode = ReluPreMode::NoRelu>
PTO_INST RecordEvent TSTORE(GlobalData& dst, TileData& src)
{
    static_assert(atomicType == AtomicType::AtomicNone && reluPreMode == ReluPreMode::NoRelu,
                  "[PTO][SA] plain TSTORE: atomic add and ReLU are not built on this path");
    b200::store_chain(dst, src, b200::StoreQuant{});
    return {};
}

// TSTORE(dst, acc, preQuantScalar) (pto_instr.hpp:441-462): one scale for the whole tile, the fp32 value in bits [31:0].
template <typename TileData, typename GlobalData, AtomicType atomicType = AtomicType::AtomicNone,
          ReluPreMode reluPreMode = ReluPreMode::NoRelu>
PTO_INST RecordEvent TSTORE(GlobalData& dst, TileData& src, uint64_t preQuantScalar)
{
    static_assert(atomicType == AtomicType::AtomicNone, "[PTO][SA] TSTORE pre-quant: atomic add is not built");
    b200::check_store_quant_valid<TileData, GlobalData>();
    b200::StoreQuant q;
    q.on = true;
    q.scalar = preQuantScalar;
    q.relu = (reluPreMode == ReluPreMode::NormalRelu);
    b200::store_chain(dst, src, q);
    return {};
}

// TSTORE(dst, acc, fpTile) (pto_instr.hpp:464-489): one 64-bit scale word per column in a TileType::Scaling tile that
// was loaded (TLOAD, or TMOV from a Mat tile) from device memory; the scale is read from bits [31:13] of each word.
template <typename TileData, typename GlobalData, typename FpTileData, AtomicType atomicType = AtomicType::AtomicNone,
          ReluPreMode reluPreMode = ReluPreMode::NoRelu, std::enable_if_t<FpTileData::Loc == TileType::Scaling, int> = 0>
PTO_INST RecordEvent TSTORE(GlobalData& dst, TileData& src, FpTileData& fp)
{
    static_assert(atomicType == AtomicType::AtomicNone, "[PTO][SA] TSTORE pre-quant: atomic add is not built");
    static_assert(sizeof(typename FpTileData::DType) == 8, "[PTO][SA] the scaling tile holds 64-bit words");
    b200::check_store_quant_valid<TileData, GlobalData>();
    if (!fp.view.bound() || fp.view.col_stride != 1) {
        b200::fail("TSTORE: the scaling tile was never loaded from a contiguous row of words", 0);
        return {};
    }
    b200::StoreQuant q;
    q.on = true;
    q.words = fp.view.ptr;
    q.word_count = fp.view.cols;
    q.relu = (reluPreMode == ReluPreMode::NormalRelu);
    b200::store_chain(dst, src, q);
    return {};
}

// TSTORE_FP (pto_instr.hpp:491-518): the same store under its own name.
template <typename TileData, typename GlobalData, typename FpTileData, AtomicType atomicType = AtomicType::AtomicNone,
          ReluPreMode reluPreMode = ReluPreMode::NoRelu>
PTO_INST RecordEvent TSTORE_FP(GlobalData& dst, TileData& src, FpTileData& fp)
{
    return TSTORE<TileData, GlobalData, FpTileData, atomicType, reluPreMode>(dst, src, fp);
}

} // namespace pto
#endif // PTO_B200_PTO_INST_HPP
