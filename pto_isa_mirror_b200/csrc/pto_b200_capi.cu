// C ABI over the sm_100a GEMM tile loop: argument validation, TMA descriptor construction, variant
// selection and launch. No device memory is allocated here and no call synchronises unless it says so.
#include "../../include/pto_b200.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_tile_loop.cuh"
#include "gemm_tile_loop_2cta.cuh"
#include "gemv.cuh"
#include "gemv_mx.cuh"
#include "ksplit_reduce.cuh"
#include "mx_quantize.cuh"

#if !defined(__CUDACC__)
#error "pto_b200 is CUDA source: build it with nvcc -gencode arch=compute_100a,code=sm_100a"
#endif
// Device passes: only the architecture-specific sm_100a target has tcgen05, tensor memory and the TMA forms used
// here. There is no other back end and no fallback, so any other target is a build error, not a slower path.
#if defined(__CUDA_ARCH__) && !(__CUDA_ARCH__ == 1000 && defined(__CUDA_ARCH_FEAT_SM100_ALL))
#error "pto_b200 kernels are written for sm_100a only (nvcc -gencode arch=compute_100a,code=sm_100a)"
#endif

namespace pto_b200 {
namespace {

__device__ int g_status_word = 0;

thread_local char t_cuda_error[256] = "";
std::atomic<unsigned long long> g_launches{0};
std::atomic<long long> g_wait_limit{kWaitLimitCycles}; // cycles one bounded wait may take (pto_b200_set_wait_limit)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceInfo {
    bool ready = false;
    int err = PTO_B200_OK;
    int sm_count = 0;
    int* status_ptr = nullptr;
    bool force_1cta = false;   // PTO_B200_FORCE_1CTA=1 in the environment: never pick the two-CTA kernels
    bool no_tma_store = false; // PTO_B200_NO_TMA_STORE=1: the two-CTA kernels store C from registers (A/B measurements)
};

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
DeviceInfo g_devices[kMaxDevices];
EncodeTiledFn g_encode = nullptr;

int note_cuda(cudaError_t e, const char* what)
{
    if (e == cudaSuccess) {
        return PTO_B200_OK;
    }
    std::snprintf(t_cuda_error, sizeof(t_cuda_error), "%s: %s", what, cudaGetErrorString(e));
    return PTO_B200_ECUDA;
}

// One-time set-up per device (capability check, SM count, status word address, driver entry point).
int device_info(DeviceInfo** out)
{
    int dev = 0;
    if (int rc = note_cuda(cudaGetDevice(&dev), "cudaGetDevice")) {
        return rc;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        return PTO_B200_EDEVICE;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo& d = g_devices[dev];
    if (!d.ready) {
        int major = 0, minor = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
        if (major != 10 || minor != 0) {
            d.err = PTO_B200_EDEVICE;
        } else {
            cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
            const char* force = std::getenv("PTO_B200_FORCE_1CTA");
            d.force_1cta = (force != nullptr && force[0] == '1');
            const char* no_tma = std::getenv("PTO_B200_NO_TMA_STORE");
            d.no_tma_store = (no_tma != nullptr && no_tma[0] == '1');
            d.err = note_cuda(cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status_ptr), g_status_word),
                              "cudaGetSymbolAddress(status)");
            if (d.err == PTO_B200_OK && g_encode == nullptr) {
                void* fn = nullptr;
                cudaDriverEntryPointQueryResult qres;
                cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
                if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
                    std::snprintf(t_cuda_error, sizeof(t_cuda_error), "cuTensorMapEncodeTiled entry point not found");
                    d.err = PTO_B200_ECUDA;
                } else {
                    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
                }
            }
        }
        d.ready = true;
    }
    *out = &d;
    return d.err;
}

int elem_size(int dtype)
{
    switch (dtype) {
        case PTO_B200_F16:
        case PTO_B200_BF16:
        case PTO_B200_S16:
            return 2;
        case PTO_B200_F32:
        case PTO_B200_S32:
            return 4;
        case PTO_B200_S8:
        case PTO_B200_U8:
        case PTO_B200_E4M3:
        case PTO_B200_E5M2:
            return 1;
        default:
            return 0;
    }
}

// 2-D row-major view [rows, cols] with leading dimension ld (elements), 128-byte swizzled boxes.
int make_tensor_map(CUtensorMap* map, int dtype, const void* base, long long rows, long long cols, long long ld,
                    int box_cols, int box_rows, bool swizzle128 = true)
{
    CUtensorMapDataType dt;
    switch (dtype) {
        case PTO_B200_F16:
            dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
            break;
        case PTO_B200_BF16:
            dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
            break;
        case PTO_B200_S16:
            dt = CU_TENSOR_MAP_DATA_TYPE_UINT16; // store maps only: the bytes move unchanged
            break;
        case PTO_B200_F32:
        case PTO_B200_S32:
            dt = CU_TENSOR_MAP_DATA_TYPE_UINT32; // store maps only: the bytes move unchanged
            break;
        default:
            dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
            break;
    }
    const int es = elem_size(dtype);
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * es};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        std::snprintf(t_cuda_error, sizeof(t_cuda_error), "cuTensorMapEncodeTiled failed with CUresult %d",
                      static_cast<int>(r));
        return PTO_B200_ECUDA;
    }
    return PTO_B200_OK;
}

// Packed 4-bit operand (PTO_B200_E2M1, two elements per byte) as the block-scaled MMA of kind::mxf8f6f4 wants it in
// shared memory: the TMA type 16U4_ALIGN16B expands every 8 bytes of 16 packed values to a 16-byte piece, so a row of
// 128 elements (64 bytes in memory) fills one 128-byte swizzle row, exactly like 128 fp8 elements. rows x k_elems
// elements, leading dimension ld_elems elements (the driver wants a 32-byte aligned base, a 32-byte pitch and k a
// multiple of 128).
int make_tensor_map_fp4(CUtensorMap* map, const void* base, long long rows, long long k_elems, long long ld_elems,
                        int box_rows)
{
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(k_elems), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems / 2)};
    cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        std::snprintf(t_cuda_error, sizeof(t_cuda_error), "cuTensorMapEncodeTiled (4-bit) failed with CUresult %d",
                      static_cast<int>(r));
        return PTO_B200_ECUDA;
    }
    return PTO_B200_OK;
}

// tcgen05 instruction descriptor (dense kinds): D format [4,6), A format [7,10), B format [10,13),
// A/B major bits 15/16 (0 = K-major), N >> 3 at [17,23), M >> 4 at [24,29).
uint32_t make_idesc(int c_fmt, int a_fmt, int b_fmt, bool b_mn_major, int n, bool block_scaled_e8m0,
                    int m_inst = kBlockM)
{
    uint32_t d = 0;
    if (!block_scaled_e8m0) {
        d |= static_cast<uint32_t>(c_fmt) << 4;
    }
    d |= static_cast<uint32_t>(a_fmt) << 7;
    d |= static_cast<uint32_t>(b_fmt) << 10;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= static_cast<uint32_t>(n >> 3) << 17;
    if (block_scaled_e8m0) {
        d |= 1u << 23; // scale format e8m0
    }
    d |= static_cast<uint32_t>(m_inst >> 4) << 24;
    return d;
}

// Workspace of the split last wave: counters first, then up to kGemmWorkspaceTiles parked 256 x 256 accumulators.
constexpr int kGemmWorkspaceTiles = 40;
constexpr size_t kGemmWorkspaceFlagBytes = 4096;
constexpr size_t kGemmWorkspaceBytes = kGemmWorkspaceFlagBytes + static_cast<size_t>(kGemmWorkspaceTiles) * 256 * 256 * 4;

struct Problem {
    int m, n, k;
    long long lda, ldb, ldc;
};

template <int KIND, int BLOCK_N, int EPI, bool B_MN>
int launch_variant(cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                   int sm_count, int block_limit = 0)
{
    constexpr int STAGES = 4;
    using L = SmemLayout<KIND, BLOCK_N, STAGES>;
    auto kernel = gemm_tile_loop<KIND, BLOCK_N, STAGES, EPI, B_MN>;
    static std::atomic<int> attr_done[kMaxDevices];
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_done[dev].load(std::memory_order_acquire) == 0) {
        if (int rc = note_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal),
                               "cudaFuncSetAttribute")) {
            return rc;
        }
        attr_done[dev].store(1, std::memory_order_release);
    }
    const int tiles = p.m_tiles * p.n_tiles;
    int grid = tiles < sm_count ? tiles : sm_count;
    if (block_limit > 0 && block_limit < grid) {
        grid = block_limit;
    }
    kernel<<<grid, kNumThreads, L::kTotal, stream>>>(ta, tb, p);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "gemm_tile_loop launch");
}

template <int KIND, int EPI, bool B_MN>
int launch_block_n(int block_n, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb,
                   const GemmParams& p, int sm_count, int block_limit = 0)
{
    if (block_n == 128) {
        return launch_variant<KIND, 128, EPI, B_MN>(stream, ta, tb, p, sm_count, block_limit);
    }
    return launch_variant<KIND, 256, EPI, B_MN>(stream, ta, tb, p, sm_count, block_limit);
}

// Two-CTA kernels: 256 x 256 tiles on clusters of two CTAs. Returns -1 when the problem should stay on the
// one-CTA kernel (fewer tiles than CTA pairs the device can hold at once), otherwise a PTO_B200 code.
struct PairLaunch {
    const CUtensorMap* sfa_map = nullptr; // block-scaled kinds only
    const CUtensorMap* sfb_map = nullptr;
    int block_limit = 0;                  // cap on thread blocks (launch_block_count), 0 = every SM
    uint8_t* workspace = nullptr;         // split last wave, or null
    size_t workspace_bytes = 0;
    int out_dtype = PTO_B200_F32;         // element type of C (for the store map)
    const KsplitFusedArgs* fused = nullptr; // K-split form: exchange arguments (group height = its panel height)
    const GatherArgs* gather = nullptr;     // all-gather form: push arguments
    bool no_tma_store = false;
};

template <int KIND, int EPI, int COMM = COMM_NONE>
int launch_pair(cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, const Problem& q,
                const PairLaunch& o)
{
#ifndef PTO_B200_PAIR_STAGES
#define PTO_B200_PAIR_STAGES 6
#endif
    constexpr int STAGES = (KIND == KIND_MXF8) ? PTO_B200_MX_PAIR_STAGES : PTO_B200_PAIR_STAGES;
    constexpr int kEpiBufs = kPairEpiBufs<KIND>;
    constexpr bool FUSED_AR = (COMM == COMM_KSPLIT);
    constexpr int kThreads = kNumThreads + (COMM != COMM_NONE ? kExchangeThreads : 0);
    using L = PairSmemLayout<KIND, STAGES, kEpiBufs>;
    auto kernel = gemm_tile_loop_2cta<KIND, STAGES, EPI, COMM>;
    static std::atomic<int> max_clusters[kMaxDevices];
    int dev = 0;
    cudaGetDevice(&dev);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kTotal;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = max_clusters[dev].load(std::memory_order_acquire);
    if (clusters == 0) {
        if (int rc = note_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal),
                               "cudaFuncSetAttribute(pair)")) {
            return rc;
        }
        cfg.gridDim = dim3(2, 1, 1);
        int n = 0;
        if (int rc = note_cuda(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg), "cudaOccupancyMaxActiveClusters")) {
            return rc;
        }
        clusters = n > 0 ? n : -1;
        max_clusters[dev].store(clusters, std::memory_order_release);
    }
    if (clusters < 0) {
        return -1;
    }
    p.m_tiles = (q.m + kPairBlockM - 1) / kPairBlockM;
    p.n_tiles = (q.n + kPairBlockN - 1) / kPairBlockN;
    p.group_m = FUSED_AR ? o.fused->panel_tile_rows : 8;
    const int tiles = p.m_tiles * p.n_tiles;
    if (tiles < clusters && COMM == COMM_NONE) {
        return -1;
    }
    if (COMM == COMM_GATHER) {
        p.mi_rotate = (o.gather->rank * o.gather->blocks_per_rank) % p.m_tiles;
    }
    int pairs = tiles < clusters ? tiles : clusters;
    if (o.block_limit > 0 && o.block_limit / 2 < pairs) {
        pairs = o.block_limit / 2 > 0 ? o.block_limit / 2 : 1;
    }
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    // Last wave: when the leftover tiles would occupy at most half of the pairs, cut each of them into two K halves
    // that run on two pairs at once and swap halves of their accumulators through the caller's workspace. The two
    // pairs wait for each other in the kernel, so the split is only used when this launch may take every SM (no
    // block cap) and is never combined with the K-split form.
    const int leftover = tiles % pairs;
    p.tail_first_unit = tiles;
    p.tail_tiles = 0;
    if (COMM == COMM_NONE && o.workspace != nullptr && o.workspace_bytes >= kGemmWorkspaceBytes && o.block_limit == 0 &&
        leftover > 0 && 2 * leftover <= pairs && leftover <= kGemmWorkspaceTiles && p.k_blocks >= 2) {
        p.tail_first_unit = tiles - leftover;
        p.tail_tiles = leftover;
        p.ws_flags = reinterpret_cast<int*>(o.workspace);
        p.ws_partial = reinterpret_cast<uint32_t*>(o.workspace + kGemmWorkspaceFlagBytes);
        // the pairs' "parked" flags carry a token no earlier launch used, so the flag area never needs clearing
        static std::atomic<unsigned> token{0};
        unsigned t = token.fetch_add(1, std::memory_order_relaxed) + 1;
        p.tail_token = static_cast<int>((t % 0x7FFFFFFEu) + 1);
    }
    // C leaves through TMA stores when it is 16-byte aligned with a 16-byte row pitch (the rule for any TMA copy)
    constexpr int esize = (EPI == EPI_F32 || EPI == EPI_S32) ? 4 : (EPI == EPI_QUANT8 ? 1 : 2);
    CUtensorMap tc = ta;
    p.tma_store = 0;
    // ... and its rows end on a 16-byte boundary: at a ragged end the store unit is a whole 16-byte piece, which
    // would run past column N (measured: bf16, N = 2500 wrote columns 2500..2503)
    if (!o.no_tma_store && (reinterpret_cast<uintptr_t>(p.c) & 15u) == 0 && ((p.ldc * esize) & 15) == 0 &&
        ((static_cast<long long>(q.n) * esize) & 15) == 0) {
        if (int rc = make_tensor_map(&tc, o.out_dtype, p.c, q.m, q.n, p.ldc, 128 / esize, 32)) {
            return rc;
        }
        p.tma_store = 1;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    // the scale maps are only read by the block-scaled instantiations; the others get copies of the A map
    const CUtensorMap& ma = o.sfa_map ? *o.sfa_map : ta;
    const CUtensorMap& mb = o.sfb_map ? *o.sfb_map : ta;
    KsplitFusedArgs none;
    std::memset(&none, 0, sizeof(none));
    const KsplitFusedArgs& fa = o.fused ? *o.fused : none;
    GatherArgs no_gather;
    std::memset(&no_gather, 0, sizeof(no_gather));
    const GatherArgs& gargs = o.gather ? *o.gather : no_gather;
    return note_cuda(cudaLaunchKernelEx(&cfg, kernel, ta, tb, ma, mb, tc, p, fa, gargs), "gemm_tile_loop_2cta launch");
}

// 128-wide tiles when 256-wide ones would leave SMs without work and the narrower split fills more of them.
int pick_block_n(int m, int n, int sm_count)
{
    const int m_tiles = (m + kBlockM - 1) / kBlockM;
    const int t256 = m_tiles * ((n + 255) / 256);
    if (n <= 128) {
        return 128;
    }
    return (t256 < sm_count) ? 128 : 256;
}


int check_common(const void* out, const void* a, const void* b, const Problem& q, int a_es, int b_es, bool b_nd)
{
    if (out == nullptr || a == nullptr || b == nullptr || q.m <= 0 || q.n <= 0 || q.k <= 0) {
        return PTO_B200_EINVAL;
    }
    if (q.lda < q.k || q.ldc < q.n || q.ldb < (b_nd ? q.n : q.k)) {
        return PTO_B200_EINVAL;
    }
    if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(b) & 15u) || ((q.lda * a_es) & 15) ||
        ((q.ldb * b_es) & 15)) {
        return PTO_B200_EALIGN;
    }
    return PTO_B200_OK;
}

void fill_params(GemmParams& p, void* out, const Problem& q, int block_n, int k_elems_per_block, int* status)
{
    std::memset(&p, 0, sizeof(p));
    p.c = out;
    p.ldc = q.ldc;
    p.m = q.m;
    p.n = q.n;
    p.k = q.k;
    p.m_tiles = (q.m + kBlockM - 1) / kBlockM;
    p.n_tiles = (q.n + block_n - 1) / block_n;
    p.k_blocks = (q.k + k_elems_per_block - 1) / k_elems_per_block;
    p.group_m = 16;
    p.status = status;
    p.wait_limit = g_wait_limit.load(std::memory_order_relaxed);
}

} // namespace
} // namespace pto_b200

using namespace pto_b200;

extern "C" int pto_b200_gemm(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n, int k,
                             long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype, int b_layout)
{
    return pto_b200_gemm_ex(stream, out, src0, src1, m, n, k, lda, ldb, ldc, in_dtype, out_dtype, b_layout, 0);
}

extern "C" int pto_b200_gemm_ex(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n,
                                int k, long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype,
                                int b_layout, int launch_block_count)
{
    return pto_b200_gemm_ws(stream, out, src0, src1, m, n, k, lda, ldb, ldc, in_dtype, out_dtype, b_layout,
                            launch_block_count, nullptr, 0);
}

extern "C" size_t pto_b200_gemm_workspace_bytes(void) { return kGemmWorkspaceBytes; }

static int gemm_dense_impl(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n, int k,
                           long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype, int b_layout,
                           int launch_block_count, uint8_t* workspace, size_t workspace_bytes, const void* bias)
{
    if (launch_block_count < 0) {
        return PTO_B200_EINVAL;
    }
    if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 3u)) {
        return PTO_B200_EALIGN;
    }
    if (workspace != nullptr && ((reinterpret_cast<uintptr_t>(workspace) & 15u) || workspace_bytes < kGemmWorkspaceBytes)) {
        return PTO_B200_EWORKSPACE;
    }
    const bool is16 = (in_dtype == PTO_B200_F16 || in_dtype == PTO_B200_BF16);
    const bool is8 = (in_dtype == PTO_B200_S8);
    if (!is16 && !is8) {
        return PTO_B200_EDTYPE;
    }
    if (b_layout != PTO_B200_B_DN && b_layout != PTO_B200_B_ND) {
        return PTO_B200_EDTYPE;
    }
    const bool b_nd = (b_layout == PTO_B200_B_ND);
    if (is16 && !(out_dtype == PTO_B200_F32 || out_dtype == PTO_B200_BF16 || out_dtype == PTO_B200_F16)) {
        return PTO_B200_EDTYPE;
    }
    if (is8 && (out_dtype != PTO_B200_S32 || b_nd)) {
        return PTO_B200_EDTYPE;
    }
    const Problem q{m, n, k, lda, ldb, ldc};
    const int es = elem_size(in_dtype);
    if (int rc = check_common(out, src0, src1, q, es, es, b_nd)) {
        return rc;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    const int block_n = pick_block_n(m, n, dev->sm_count);
    const int kelems = kBlockKBytes / es;
    GemmParams p;
    fill_params(p, out, q, block_n, kelems, dev->status_ptr);
    p.bias = bias;
    CUtensorMap ta, tb;
    if (int rc = make_tensor_map(&ta, in_dtype, src0, m, k, lda, kelems, kBlockM)) {
        return rc;
    }
    if (b_nd) {
        if (int rc = make_tensor_map(&tb, in_dtype, src1, k, n, ldb, 64, 64)) {
            return rc;
        }
    } else {
        if (int rc = make_tensor_map(&tb, in_dtype, src1, n, k, ldb, kelems, block_n)) {
            return rc;
        }
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int fmt = (in_dtype == PTO_B200_BF16) ? 1 : 0;
    if (!b_nd && !dev->force_1cta && m > kBlockM) {
        // CTA pairs on 256 x 256 tiles when there are enough tiles to occupy every pair
        CUtensorMap tb_half;
        if (int rc = make_tensor_map(&tb_half, in_dtype, src1, n, k, ldb, kelems, kPairBlockN / 2)) {
            return rc;
        }
        GemmParams pp = p;
        int rc = -1;
        PairLaunch o;
        o.block_limit = launch_block_count;
        o.workspace = workspace;
        o.workspace_bytes = workspace_bytes;
        o.out_dtype = out_dtype;
        o.no_tma_store = dev->no_tma_store;
        if (is8) {
            pp.idesc = make_idesc(2, 1, 1, false, kPairBlockN, false, kPairBlockM);
            rc = launch_pair<KIND_I8, EPI_S32>(s, ta, tb_half, pp, q, o);
        } else {
            pp.idesc = make_idesc(1, fmt, fmt, false, kPairBlockN, false, kPairBlockM);
            switch (out_dtype) {
                case PTO_B200_F32:
                    rc = launch_pair<KIND_F16, EPI_F32>(s, ta, tb_half, pp, q, o);
                    break;
                case PTO_B200_BF16:
                    rc = launch_pair<KIND_F16, EPI_BF16>(s, ta, tb_half, pp, q, o);
                    break;
                default:
                    rc = launch_pair<KIND_F16, EPI_F16>(s, ta, tb_half, pp, q, o);
                    break;
            }
        }
        if (rc != -1) {
            return rc;
        }
    }
    if (is8) {
        p.idesc = make_idesc(2 /*S32*/, 1 /*S8*/, 1 /*S8*/, false, block_n, false);
        return launch_block_n<KIND_I8, EPI_S32, false>(block_n, s, ta, tb, p, dev->sm_count, launch_block_count);
    }
    p.idesc = make_idesc(1 /*F32*/, fmt, fmt, b_nd, block_n, false);
    if (b_nd) {
        switch (out_dtype) {
            case PTO_B200_F32:
                return launch_block_n<KIND_F16, EPI_F32, true>(block_n, s, ta, tb, p, dev->sm_count, launch_block_count);
            case PTO_B200_BF16:
                return launch_block_n<KIND_F16, EPI_BF16, true>(block_n, s, ta, tb, p, dev->sm_count, launch_block_count);
            default:
                return launch_block_n<KIND_F16, EPI_F16, true>(block_n, s, ta, tb, p, dev->sm_count, launch_block_count);
        }
    }
    switch (out_dtype) {
        case PTO_B200_F32:
            return launch_block_n<KIND_F16, EPI_F32, false>(block_n, s, ta, tb, p, dev->sm_count, launch_block_count);
        case PTO_B200_BF16:
            return launch_block_n<KIND_F16, EPI_BF16, false>(block_n, s, ta, tb, p, dev->sm_count, launch_block_count);
        default:
            return launch_block_n<KIND_F16, EPI_F16, false>(block_n, s, ta, tb, p, dev->sm_count, launch_block_count);
    }
}

extern "C" int pto_b200_gemm_ws(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n,
                                int k, long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype,
                                int b_layout, int launch_block_count, uint8_t* workspace, size_t workspace_bytes)
{
    return gemm_dense_impl(stream, out, src0, src1, m, n, k, lda, ldb, ldc, in_dtype, out_dtype, b_layout,
                           launch_block_count, workspace, workspace_bytes, nullptr);
}

extern "C" int pto_b200_gemm_bias(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                                  const uint8_t* bias, int m, int n, int k, long long lda, long long ldb,
                                  long long ldc, int in_dtype, int out_dtype, int b_layout)
{
    if (bias == nullptr) {
        return PTO_B200_EINVAL;
    }
    return gemm_dense_impl(stream, out, src0, src1, m, n, k, lda, ldb, ldc, in_dtype, out_dtype, b_layout, 0, nullptr,
                           0, bias);
}

extern "C" int pto_b200_gemm_quant(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, int m, int n,
                                   int k, long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype,
                                   unsigned long long pre_quant_scalar, const unsigned long long* fp_words, int relu)
{
    const bool is16 = (in_dtype == PTO_B200_F16 || in_dtype == PTO_B200_BF16);
    const bool is8 = (in_dtype == PTO_B200_S8);
    const bool out8 = (out_dtype == PTO_B200_S8 || out_dtype == PTO_B200_U8);
    const bool out_s16 = (out_dtype == PTO_B200_S16);
    if ((!is16 && !is8) || !(out_dtype == PTO_B200_BF16 || out_dtype == PTO_B200_F16 || out8 || out_s16) ||
        (out_s16 && !is8)) { // the shift form exists for int32 accumulators only
        return PTO_B200_EDTYPE;
    }
    if (fp_words != nullptr && (reinterpret_cast<uintptr_t>(fp_words) & 7u)) {
        return PTO_B200_EALIGN;
    }
    const Problem q{m, n, k, lda, ldb, ldc};
    const int es = elem_size(in_dtype);
    if (int rc = check_common(out, src0, src1, q, es, es, false)) {
        return rc;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    const int block_n = pick_block_n(m, n, dev->sm_count);
    const int kelems = kBlockKBytes / es;
    GemmParams p;
    fill_params(p, out, q, block_n, kelems, dev->status_ptr);
    p.quant_word = pre_quant_scalar;
    p.quant_words = fp_words;
    p.quant_flags = (is8 ? QUANT_ACC_S32 : 0) | (out_dtype == PTO_B200_F16 ? QUANT_OUT_F16 : 0) |
                    (out_s16 ? QUANT_OUT_S16 : 0) |
                    (relu ? QUANT_RELU : 0) | (fp_words != nullptr ? QUANT_VECTOR : 0);
    CUtensorMap ta, tb;
    if (int rc = make_tensor_map(&ta, in_dtype, src0, m, k, lda, kelems, kBlockM)) {
        return rc;
    }
    if (int rc = make_tensor_map(&tb, in_dtype, src1, n, k, ldb, kelems, block_n)) {
        return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int fmt = (in_dtype == PTO_B200_BF16) ? 1 : 0;
    if (!dev->force_1cta && m > kBlockM) {
        CUtensorMap tb_half;
        if (int rc = make_tensor_map(&tb_half, in_dtype, src1, n, k, ldb, kelems, kPairBlockN / 2)) {
            return rc;
        }
        GemmParams pp = p;
        PairLaunch o;
        o.out_dtype = out_dtype;
        o.no_tma_store = dev->no_tma_store || out8; // 8-bit results leave from registers
        int rc;
        if (is8) {
            pp.idesc = make_idesc(2, 1, 1, false, kPairBlockN, false, kPairBlockM);
            rc = out8 ? launch_pair<KIND_I8, EPI_QUANT8>(s, ta, tb_half, pp, q, o)
                      : launch_pair<KIND_I8, EPI_QUANT16>(s, ta, tb_half, pp, q, o);
        } else {
            pp.idesc = make_idesc(1, fmt, fmt, false, kPairBlockN, false, kPairBlockM);
            rc = out8 ? launch_pair<KIND_F16, EPI_QUANT8>(s, ta, tb_half, pp, q, o)
                      : launch_pair<KIND_F16, EPI_QUANT16>(s, ta, tb_half, pp, q, o);
        }
        if (rc != -1) {
            return rc;
        }
    }
    if (is8) {
        p.idesc = make_idesc(2, 1, 1, false, block_n, false);
        return out8 ? launch_block_n<KIND_I8, EPI_QUANT8, false>(block_n, s, ta, tb, p, dev->sm_count)
                    : launch_block_n<KIND_I8, EPI_QUANT16, false>(block_n, s, ta, tb, p, dev->sm_count);
    }
    p.idesc = make_idesc(1, fmt, fmt, false, block_n, false);
    return out8 ? launch_block_n<KIND_F16, EPI_QUANT8, false>(block_n, s, ta, tb, p, dev->sm_count)
                : launch_block_n<KIND_F16, EPI_QUANT16, false>(block_n, s, ta, tb, p, dev->sm_count);
}

extern "C" int pto_b200_gemm_s8_dequant(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                                        const float* s_row, const float* s_col, int m, int n, int k, long long lda,
                                        long long ldb, long long ldc)
{
    if (s_row == nullptr || s_col == nullptr) {
        return PTO_B200_EINVAL;
    }
    const Problem q{m, n, k, lda, ldb, ldc};
    if (int rc = check_common(out, src0, src1, q, 1, 1, false)) {
        return rc;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    const int block_n = pick_block_n(m, n, dev->sm_count);
    GemmParams p;
    fill_params(p, out, q, block_n, kBlockKBytes, dev->status_ptr);
    p.s_row = s_row;
    p.s_col = s_col;
    p.idesc = make_idesc(2, 1, 1, false, block_n, false);
    CUtensorMap ta, tb;
    if (int rc = make_tensor_map(&ta, PTO_B200_S8, src0, m, k, lda, kBlockKBytes, kBlockM)) {
        return rc;
    }
    if (int rc = make_tensor_map(&tb, PTO_B200_S8, src1, n, k, ldb, kBlockKBytes, block_n)) {
        return rc;
    }
    if (!dev->force_1cta && m > kBlockM) {
        CUtensorMap tb_half;
        if (int rc = make_tensor_map(&tb_half, PTO_B200_S8, src1, n, k, ldb, kBlockKBytes, kPairBlockN / 2)) {
            return rc;
        }
        GemmParams pp = p;
        pp.idesc = make_idesc(2, 1, 1, false, kPairBlockN, false, kPairBlockM);
        PairLaunch o;
        o.out_dtype = PTO_B200_BF16;
        o.no_tma_store = dev->no_tma_store;
        const int rc = launch_pair<KIND_I8, EPI_DEQ_BF16>(static_cast<cudaStream_t>(stream), ta, tb_half, pp, q, o);
        if (rc != -1) {
            return rc;
        }
    }
    return launch_block_n<KIND_I8, EPI_DEQ_BF16, false>(block_n, static_cast<cudaStream_t>(stream), ta, tb, p,
                                                        dev->sm_count);
}

extern "C" size_t pto_b200_gemm_mx_workspace_bytes(int m, int n, int k)
{
    if (m <= 0 || n <= 0 || k <= 0) {
        return 0;
    }
    // 128-row scale blocks, counted in pairs so that either tile shape (128- or 256-row tiles) fits
    const size_t m_blocks = 2 * ((static_cast<size_t>(m) + 255) / 256);
    const size_t n_blocks = 2 * ((static_cast<size_t>(n) + 255) / 256);
    const size_t k_blocks = (static_cast<size_t>(k) + kBlockKBytes - 1) / kBlockKBytes;
    return k_blocks * (m_blocks + n_blocks) * 512;
}

// Argument checks of the block-scaled GEMM that need no device: dtype table, pointers, sizes, TMA alignment.
static int mx_check_args(const uint8_t* out, const uint8_t* src0, const uint8_t* src1, const uint8_t* src2,
                         const uint8_t* src3, int m, int n, int k, long long lda, long long ldb, long long ldc,
                         long long ld_sfa, long long ld_sfb, int a_dtype, int b_dtype, int out_dtype, const void* bias)
{
    if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 3u)) {
        return PTO_B200_EALIGN;
    }
    const bool a_ok = (a_dtype == PTO_B200_E4M3 || a_dtype == PTO_B200_E5M2);
    const bool b_ok = (b_dtype == PTO_B200_E4M3 || b_dtype == PTO_B200_E5M2);
    // CheckMadMxValid (include/pto/cpu/TMatmul.hpp:113-131): any mix of the fp8 types, or both operands fp4
    const bool fp4 = (a_dtype == PTO_B200_E2M1 && b_dtype == PTO_B200_E2M1);
    if (!((a_ok && b_ok) || fp4) || !(out_dtype == PTO_B200_BF16 || out_dtype == PTO_B200_F32)) {
        return PTO_B200_EDTYPE;
    }
    if (src2 == nullptr || src3 == nullptr) {
        return PTO_B200_EINVAL;
    }
    const Problem q{m, n, k, lda, ldb, ldc};
    if (int rc = check_common(out, src0, src1, q, 1, 1, false)) {
        return rc;
    }
    if (k % 32 != 0 || ld_sfa < k / 32 || ld_sfb < k / 32) {
        return PTO_B200_EINVAL;
    }
    if (fp4) {
        // two elements per byte: the 4-bit TMA type wants k a multiple of 128, 32-byte aligned bases and pitches
        if (k % 128 != 0) {
            return PTO_B200_EINVAL;
        }
        if ((reinterpret_cast<uintptr_t>(src0) & 31u) || (reinterpret_cast<uintptr_t>(src1) & 31u) || (lda & 63) ||
            (ldb & 63)) {
            return PTO_B200_EALIGN;
        }
    }
    return PTO_B200_OK;
}

// What a call of the block-scaled path does: re-tile the scales into the workspace, multiply, or both.
enum MxSteps : int { MX_RETILE = 1, MX_MULTIPLY = 2 };

static int gemm_mx_impl(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, const uint8_t* src2,
                        const uint8_t* src3, uint8_t* workspace, size_t workspace_bytes, int m, int n, int k,
                        long long lda, long long ldb, long long ldc, long long ld_sfa, long long ld_sfb, int a_dtype,
                        int b_dtype, int out_dtype, const void* bias, int steps = MX_RETILE | MX_MULTIPLY)
{
    if (int rc = mx_check_args(out, src0, src1, src2, src3, m, n, k, lda, ldb, ldc, ld_sfa, ld_sfb, a_dtype, b_dtype,
                               out_dtype, bias)) {
        return rc;
    }
    const Problem q{m, n, k, lda, ldb, ldc};
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15u) ||
        workspace_bytes < pto_b200_gemm_mx_workspace_bytes(m, n, k)) {
        return PTO_B200_EWORKSPACE;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // operand format codes of kind::mxf8f6f4: e4m3 0, e5m2 1, e2m1 5
    const bool fp4 = (a_dtype == PTO_B200_E2M1);
    const int a_fmt = fp4 ? 5 : (a_dtype == PTO_B200_E5M2 ? 1 : 0);
    const int b_fmt = fp4 ? 5 : (b_dtype == PTO_B200_E5M2 ? 1 : 0);
    // Re-tile the scales, then the GEMM. `pairs` picks the two-CTA kernel (256 x 256 tiles, scale row blocks in
    // units of 128 rows: 2 per row-tile of A, 2 per column-tile of B) when the problem has enough tiles for it.
    auto run = [&](bool pairs, int block_n) -> int {
        GemmParams p;
        fill_params(p, out, q, block_n, kBlockKBytes, dev->status_ptr);
        // one layout of the re-tiled scales whatever kernel reads them: 128-row blocks counted in pairs
        const int a_blocks = 2 * ((m + kPairBlockM - 1) / kPairBlockM);
        const int b_blocks = 2 * ((n + kPairBlockN - 1) / kPairBlockN);
        if (pairs) {
            p.m_tiles = (m + kPairBlockM - 1) / kPairBlockM;
            p.n_tiles = (n + kPairBlockN - 1) / kPairBlockN;
        }
        uint8_t* sfa_ws = workspace;
        uint8_t* sfb_ws = workspace + static_cast<size_t>(p.k_blocks) * a_blocks * 512;
        p.bias = bias;
        p.sfa = sfa_ws;
        p.sfb = sfb_ws;
        p.sf_a_blocks = a_blocks;
        p.sf_b_blocks = b_blocks;
        p.packed4 = fp4 ? 1 : 0;
        CUtensorMap ta, tb, tsa, tsb;
        const int b_box_rows = pairs ? kPairBlockN / 2 : block_n;
        if (fp4) {
            if (int rc = make_tensor_map_fp4(&ta, src0, m, k, lda, kBlockM)) {
                return rc;
            }
            if (int rc = make_tensor_map_fp4(&tb, src1, n, k, ldb, b_box_rows)) {
                return rc;
            }
        } else {
            if (int rc = make_tensor_map(&ta, a_dtype, src0, m, k, lda, kBlockKBytes, kBlockM)) {
                return rc;
            }
            if (int rc = make_tensor_map(&tb, b_dtype, src1, n, k, ldb, kBlockKBytes, b_box_rows)) {
                return rc;
            }
        }
        if (pairs) {
            const long long rows_a = static_cast<long long>(p.k_blocks) * a_blocks * 2;
            const long long rows_b = static_cast<long long>(p.k_blocks) * b_blocks * 2;
            if (int rc = make_tensor_map(&tsa, PTO_B200_S8, sfa_ws, rows_a, 256, 256, 256, 2, false)) {
                return rc;
            }
            if (int rc = make_tensor_map(&tsb, PTO_B200_S8, sfb_ws, rows_b, 256, 256, 256, 4, false)) {
                return rc;
            }
            // refuse early (before the re-tile kernels) if the pair kernel would decline this shape
            p.idesc = make_idesc(0, a_fmt, b_fmt, false, kPairBlockN, true, kPairBlockM);
        } else {
            p.idesc = make_idesc(0, a_fmt, b_fmt, false, block_n, true);
        }
        const long long items = (static_cast<long long>(a_blocks) + b_blocks) * p.k_blocks * 128;
        const int grid = static_cast<int>((items + 255) / 256 < 8192 ? (items + 255) / 256 : 8192);
        if (steps & MX_RETILE) {
            retile_scales_kernel<<<grid, 256, 0, s>>>(src2, sfa_ws, m, ld_sfa, a_blocks, src3, sfb_ws, n, ld_sfb, b_blocks,
                                                      k / 32, p.k_blocks);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            if (int rc = note_cuda(cudaGetLastError(), "retile_scales launch")) {
                return rc;
            }
        }
        if (!(steps & MX_MULTIPLY)) {
            return PTO_B200_OK;
        }
        if (pairs) {
            PairLaunch o;
            o.sfa_map = &tsa;
            o.sfb_map = &tsb;
            o.out_dtype = out_dtype;
            o.no_tma_store = dev->no_tma_store;
            // a workspace with room beyond the re-tiled scales (pto_b200_gemm_workspace_bytes() more) also lets the
            // last, partly filled wave of tiles be cut into K halves, as for the dense kernels
            const size_t scale_bytes = pto_b200_gemm_mx_workspace_bytes(m, n, k);
            if (workspace_bytes >= scale_bytes + kGemmWorkspaceBytes) {
                o.workspace = workspace + scale_bytes;
                o.workspace_bytes = workspace_bytes - scale_bytes;
            }
            if (out_dtype == PTO_B200_F32) {
                return launch_pair<KIND_MXF8, EPI_F32>(s, ta, tb, p, q, o);
            }
            return launch_pair<KIND_MXF8, EPI_BF16>(s, ta, tb, p, q, o);
        }
        if (out_dtype == PTO_B200_F32) {
            return launch_block_n<KIND_MXF8, EPI_F32, false>(block_n, s, ta, tb, p, dev->sm_count);
        }
        return launch_block_n<KIND_MXF8, EPI_BF16, false>(block_n, s, ta, tb, p, dev->sm_count);
    };
    // the pair kernel wants at least one 256 x 256 tile per CTA pair (74 pairs on a full B200)
    const long long tiles256 = static_cast<long long>((m + kPairBlockM - 1) / kPairBlockM) * ((n + kPairBlockN - 1) / kPairBlockN);
    if (!dev->force_1cta && m > kBlockM && tiles256 >= dev->sm_count / 2) {
        const int rc = run(true, kPairBlockN);
        if (rc != -1) {
            return rc;
        }
    }
    return run(false, pick_block_n(m, n, dev->sm_count));
}

extern "C" int pto_b200_gemm_mx(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                                const uint8_t* src2, const uint8_t* src3, uint8_t* workspace, size_t workspace_bytes,
                                int m, int n, int k, long long lda, long long ldb, long long ldc, long long ld_sfa,
                                long long ld_sfb, int a_dtype, int b_dtype, int out_dtype)
{
    return gemm_mx_impl(stream, out, src0, src1, src2, src3, workspace, workspace_bytes, m, n, k, lda, ldb, ldc, ld_sfa,
                        ld_sfb, a_dtype, b_dtype, out_dtype, nullptr);
}

extern "C" int pto_b200_mx_retile_scales(void* stream, uint8_t* workspace, size_t workspace_bytes, const uint8_t* src2,
                                         const uint8_t* src3, int m, int n, int k, long long ld_sfa, long long ld_sfb)
{
    // the operand pointers are not touched by this step: any aligned non-null value passes the shared checks
    const uint8_t* aligned = reinterpret_cast<const uint8_t*>(static_cast<uintptr_t>(16));
    return gemm_mx_impl(stream, const_cast<uint8_t*>(aligned), aligned, aligned, src2, src3, workspace, workspace_bytes, m,
                        n, k, k, k, n, ld_sfa, ld_sfb, PTO_B200_E4M3, PTO_B200_E4M3, PTO_B200_BF16, nullptr, MX_RETILE);
}

extern "C" int pto_b200_gemm_mx_pretiled(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                                         const uint8_t* tiled_scales, size_t tiled_bytes, int m, int n, int k,
                                         long long lda, long long ldb, long long ldc, int a_dtype, int b_dtype,
                                         int out_dtype)
{
    // the scale tensors themselves are not read: the workspace already holds them re-tiled
    const uint8_t* unused = reinterpret_cast<const uint8_t*>(static_cast<uintptr_t>(16));
    return gemm_mx_impl(stream, out, src0, src1, unused, unused, const_cast<uint8_t*>(tiled_scales), tiled_bytes, m, n, k,
                        lda, ldb, ldc, k / 32, k / 32, a_dtype, b_dtype, out_dtype, nullptr, MX_MULTIPLY);
}

extern "C" int pto_b200_gemm_mx_bias(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                                     const uint8_t* src2, const uint8_t* src3, const uint8_t* bias, uint8_t* workspace,
                                     size_t workspace_bytes, int m, int n, int k, long long lda, long long ldb,
                                     long long ldc, long long ld_sfa, long long ld_sfb, int a_dtype, int b_dtype,
                                     int out_dtype)
{
    if (bias == nullptr) {
        return PTO_B200_EINVAL;
    }
    return gemm_mx_impl(stream, out, src0, src1, src2, src3, workspace, workspace_bytes, m, n, k, lda, ldb, ldc, ld_sfa,
                        ld_sfb, a_dtype, b_dtype, out_dtype, bias);
}

extern "C" int pto_b200_cast_f32_to_bf16(void* stream, uint8_t* out, const uint8_t* in, long long count)
{
    if (out == nullptr || in == nullptr || count < 0) {
        return PTO_B200_EINVAL;
    }
    if ((reinterpret_cast<uintptr_t>(in) & 15u) || (reinterpret_cast<uintptr_t>(out) & 7u)) {
        return PTO_B200_EALIGN;
    }
    if (count == 0) {
        return PTO_B200_OK;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    const long long want = (count / 4 + 255) / 256 + 1;
    const long long cap = static_cast<long long>(dev->sm_count) * 16;
    const int grid = static_cast<int>(want < cap ? want : cap);
    cast_f32_bf16_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float*>(in), reinterpret_cast<__nv_bfloat16*>(out), count);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "cast_f32_bf16 launch");
}

// ---------------------------------------------------------------- TGEMV (one left row) and the MX quantiser

template <int IN>
static int launch_gemv(cudaStream_t s, int grid, int out_dtype, const void* a, const void* b, const void* bias,
                       void* out, int n, int k, long long ldb)
{
    if constexpr (IN == GEMV_S8) {
        gemv_kernel<GEMV_S8, GEMV_OUT_S32><<<grid, kGemvThreads, 0, s>>>(a, b, bias, out, n, k, ldb);
    } else {
        switch (out_dtype) {
            case PTO_B200_F32:
                gemv_kernel<IN, GEMV_OUT_F32><<<grid, kGemvThreads, 0, s>>>(a, b, bias, out, n, k, ldb);
                break;
            case PTO_B200_BF16:
                gemv_kernel<IN, GEMV_OUT_BF16><<<grid, kGemvThreads, 0, s>>>(a, b, bias, out, n, k, ldb);
                break;
            default:
                gemv_kernel<IN, GEMV_OUT_F16><<<grid, kGemvThreads, 0, s>>>(a, b, bias, out, n, k, ldb);
                break;
        }
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "gemv launch");
}

extern "C" int pto_b200_gemv(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                             const uint8_t* bias, int n, int k, long long ldb, int in_dtype, int out_dtype)
{
    const bool is16 = (in_dtype == PTO_B200_F16 || in_dtype == PTO_B200_BF16);
    const bool is8 = (in_dtype == PTO_B200_S8);
    if (!is16 && !is8) {
        return PTO_B200_EDTYPE;
    }
    if (is16 && !(out_dtype == PTO_B200_F32 || out_dtype == PTO_B200_BF16 || out_dtype == PTO_B200_F16)) {
        return PTO_B200_EDTYPE;
    }
    if (is8 && out_dtype != PTO_B200_S32) {
        return PTO_B200_EDTYPE;
    }
    if (out == nullptr || src0 == nullptr || src1 == nullptr || n <= 0 || k <= 0 || ldb < k) {
        return PTO_B200_EINVAL;
    }
    const int es = is8 ? 1 : 2;
    const int out_es = (out_dtype == PTO_B200_F32 || out_dtype == PTO_B200_S32) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(src0) & 15u) || (reinterpret_cast<uintptr_t>(src1) & 15u) ||
        ((ldb * es) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & static_cast<uintptr_t>(out_es - 1)) ||
        (reinterpret_cast<uintptr_t>(bias) & 3u)) {
        return PTO_B200_EALIGN;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    const int warps_per_block = kGemvThreads / 32;
    const long long want = (static_cast<long long>(n) + warps_per_block - 1) / warps_per_block;
    const long long cap = static_cast<long long>(dev->sm_count) * 8; // 8 x 256 threads fill an SM
    const int grid = static_cast<int>(want < cap ? want : cap);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (is8) {
        return launch_gemv<GEMV_S8>(s, grid, out_dtype, src0, src1, bias, out, n, k, ldb);
    }
    if (in_dtype == PTO_B200_BF16) {
        return launch_gemv<GEMV_BF16>(s, grid, out_dtype, src0, src1, bias, out, n, k, ldb);
    }
    return launch_gemv<GEMV_F16>(s, grid, out_dtype, src0, src1, bias, out, n, k, ldb);
}

template <bool A52, bool B52, int OUT>
static int launch_gemv_mx_out(cudaStream_t s, int grid, const uint8_t* a, const uint8_t* sa, const uint8_t* b,
                              const uint8_t* sb, const float* bias, void* out, int n, int k, long long ldb,
                              long long ld_sfb)
{
    if (k <= kGemvMxSmemK) {
        // the left row as floats in slot order (whole 512-value pieces) + one float per scale block
        const size_t smem = static_cast<size_t>((k + 511) / 512) * 512 * sizeof(float) + static_cast<size_t>(k / 32) * sizeof(float);
        auto kernel = gemv_mx_kernel<A52, B52, OUT>;
        if (smem > 48 * 1024) {
            if (int rc = note_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                                   "cudaFuncSetAttribute(gemv_mx)")) {
                return rc;
            }
        }
        kernel<<<grid, kGemvThreads, smem, s>>>(a, sa, b, sb, bias, out, n, k, ldb, ld_sfb);
    } else {
        constexpr int cols_per_block = (kGemvThreads / 32) * kGemvMxColsPerWarp; // a warp owns two columns
        const long long want = (static_cast<long long>(n) + cols_per_block - 1) / cols_per_block;
        gemv_mx_mma_kernel<A52, B52, OUT><<<static_cast<int>(want < grid ? want : grid), kGemvThreads, 0, s>>>(
            a, sa, b, sb, bias, out, n, k, ldb, ld_sfb);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "gemv_mx launch");
}

template <bool A52, bool B52>
static int launch_gemv_mx(cudaStream_t s, int grid, int out_dtype, const uint8_t* a, const uint8_t* sa, const uint8_t* b,
                          const uint8_t* sb, const float* bias, void* out, int n, int k, long long ldb, long long ld_sfb)
{
    if (out_dtype == PTO_B200_F32) {
        return launch_gemv_mx_out<A52, B52, GEMV_OUT_F32>(s, grid, a, sa, b, sb, bias, out, n, k, ldb, ld_sfb);
    }
    return launch_gemv_mx_out<A52, B52, GEMV_OUT_BF16>(s, grid, a, sa, b, sb, bias, out, n, k, ldb, ld_sfb);
}

extern "C" int pto_b200_gemv_mx(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1, const uint8_t* src2,
                                const uint8_t* src3, const uint8_t* bias, int n, int k, long long ldb, long long ld_sfb,
                                int a_dtype, int b_dtype, int out_dtype)
{
    const bool a_ok = (a_dtype == PTO_B200_E4M3 || a_dtype == PTO_B200_E5M2);
    const bool b_ok = (b_dtype == PTO_B200_E4M3 || b_dtype == PTO_B200_E5M2);
    if (!a_ok || !b_ok || !(out_dtype == PTO_B200_F32 || out_dtype == PTO_B200_BF16)) {
        return PTO_B200_EDTYPE;
    }
    if (out == nullptr || src0 == nullptr || src1 == nullptr || src2 == nullptr || src3 == nullptr || n <= 0 || k <= 0 ||
        k % 32 != 0 || ldb < k || ld_sfb < k / 32) {
        return PTO_B200_EINVAL;
    }
    const int out_es = (out_dtype == PTO_B200_F32) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(src0) & 15u) || (reinterpret_cast<uintptr_t>(src1) & 15u) || (ldb & 15) != 0 ||
        (reinterpret_cast<uintptr_t>(out) & static_cast<uintptr_t>(out_es - 1)) ||
        (reinterpret_cast<uintptr_t>(bias) & 3u)) {
        return PTO_B200_EALIGN;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    const int warps_per_block = kGemvThreads / 32;                           // one column per warp and pass
    const long long want = (static_cast<long long>(n) + warps_per_block - 1) / warps_per_block;
    const long long cap = static_cast<long long>(dev->sm_count) * 8;
    const int grid = static_cast<int>(want < cap ? want : cap);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float* fb = reinterpret_cast<const float*>(bias);
    const bool a52 = (a_dtype == PTO_B200_E5M2), b52 = (b_dtype == PTO_B200_E5M2);
    if (a52 && b52) {
        return launch_gemv_mx<true, true>(s, grid, out_dtype, src0, src2, src1, src3, fb, out, n, k, ldb, ld_sfb);
    }
    if (a52) {
        return launch_gemv_mx<true, false>(s, grid, out_dtype, src0, src2, src1, src3, fb, out, n, k, ldb, ld_sfb);
    }
    if (b52) {
        return launch_gemv_mx<false, true>(s, grid, out_dtype, src0, src2, src1, src3, fb, out, n, k, ldb, ld_sfb);
    }
    return launch_gemv_mx<false, false>(s, grid, out_dtype, src0, src2, src1, src3, fb, out, n, k, ldb, ld_sfb);
}

extern "C" int pto_b200_mx_quantize_e4m3_ex(void* stream, uint8_t* data, uint8_t* scales, const uint8_t* src, int rows,
                                            int k, long long ld_src, long long ld_data, long long ld_scales, int scale_alg)
{
    if (data == nullptr || scales == nullptr || src == nullptr || rows <= 0 || k <= 0 || k % 32 != 0 || ld_src < k ||
        ld_data < k || ld_scales < k / 32) {
        return PTO_B200_EINVAL;
    }
    if (scale_alg != PTO_B200_SCALE_OCP && scale_alg != PTO_B200_SCALE_NV) {
        return PTO_B200_EDTYPE;
    }
    if ((reinterpret_cast<uintptr_t>(src) & 15u) || (ld_src & 3) != 0 || (reinterpret_cast<uintptr_t>(data) & 3u) ||
        (ld_data & 3) != 0) {
        return PTO_B200_EALIGN;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    auto kernel = scale_alg == PTO_B200_SCALE_NV ? mx_quantize_e4m3_kernel<MX_SCALE_NV> : mx_quantize_e4m3_kernel<MX_SCALE_OCP>;
    // one resident wave of blocks walking the matrix with a grid stride: no partly filled second wave
    int blocks_per_sm = 0;
    if (int rc = note_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, kernel, kQuantThreads, 0),
                           "mx_quantize occupancy")) {
        return rc;
    }
    const long long items = static_cast<long long>(rows) * (k / 4);
    const long long want = (items + kQuantThreads - 1) / kQuantThreads;
    const long long cap = static_cast<long long>(dev->sm_count) * (blocks_per_sm > 0 ? blocks_per_sm : 1);
    const int grid = static_cast<int>(want < cap ? want : cap);
    kernel<<<grid, kQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const float*>(src), data, scales,
                                                                          rows, k, ld_src, ld_data, ld_scales);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "mx_quantize launch");
}

extern "C" int pto_b200_mx_quantize_e4m3(void* stream, uint8_t* data, uint8_t* scales, const uint8_t* src, int rows,
                                         int k, long long ld_src, long long ld_data, long long ld_scales)
{
    return pto_b200_mx_quantize_e4m3_ex(stream, data, scales, src, rows, k, ld_src, ld_data, ld_scales,
                                        PTO_B200_SCALE_OCP);
}

extern "C" int pto_b200_mx_quantize_e2m1(void* stream, uint8_t* data, uint8_t* scales, const uint8_t* src, int rows,
                                         int k, long long ld_src, long long ld_data, long long ld_scales, int scale_alg)
{
    if (data == nullptr || scales == nullptr || src == nullptr || rows <= 0 || k <= 0 || k % 32 != 0 || ld_src < k ||
        ld_data < k / 2 || ld_scales < k / 32) {
        return PTO_B200_EINVAL;
    }
    if (scale_alg != PTO_B200_SCALE_OCP && scale_alg != PTO_B200_SCALE_NV) {
        return PTO_B200_EDTYPE;
    }
    if ((reinterpret_cast<uintptr_t>(src) & 15u) || (ld_src & 3) != 0 || (reinterpret_cast<uintptr_t>(data) & 1u) ||
        (ld_data & 1) != 0) {
        return PTO_B200_EALIGN;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    auto kernel = scale_alg == PTO_B200_SCALE_NV ? mx_quantize_e2m1_kernel<MX_SCALE_NV> : mx_quantize_e2m1_kernel<MX_SCALE_OCP>;
    int blocks_per_sm = 0;
    if (int rc = note_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, kernel, kQuantThreads, 0),
                           "mx_quantize occupancy")) {
        return rc;
    }
    const long long items = static_cast<long long>(rows) * (k / 4);
    const long long want = (items + kQuantThreads - 1) / kQuantThreads;
    const long long cap = static_cast<long long>(dev->sm_count) * (blocks_per_sm > 0 ? blocks_per_sm : 1);
    const int grid = static_cast<int>(want < cap ? want : cap);
    kernel<<<grid, kQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const float*>(src), data, scales,
                                                                          rows, k, ld_src, ld_data, ld_scales);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "mx_quantize_e2m1 launch");
}

// ---------------------------------------------------------------- K-split reduction over peer memory

static int fill_peers(PeerPointers& pp, void* const* ptrs, int world)
{
    if (ptrs == nullptr) {
        return PTO_B200_EINVAL;
    }
    for (int r = 0; r < kMaxRanks; ++r) {
        pp.p[r] = (r < world) ? ptrs[r] : nullptr;
        if (r < world && ptrs[r] == nullptr) {
            return PTO_B200_EINVAL;
        }
    }
    return PTO_B200_OK;
}

extern "C" int pto_b200_ksplit_signal(void* stream, void* const* flag_arrays, int world, int rank, int slot, int epoch)
{
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || slot < 0 || epoch < 1) {
        return PTO_B200_EINVAL;
    }
    PeerPointers fp;
    if (int rc = fill_peers(fp, flag_arrays, world)) {
        return rc;
    }
    ksplit_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(fp, world, rank, slot, epoch);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "ksplit_signal launch");
}

extern "C" int pto_b200_ksplit_reduce(void* stream, void* const* partial_ptrs, void* const* out_ptrs,
                                      void* const* done_arrays, const int* ready_local, int* cta_counters_local,
                                      int world, int rank, int slot, int epoch, long long row0, int rows, int n,
                                      long long ld_partial, long long ld_out, int launch_block_count,
                                      const void* multicast_partial, void* multicast_out)
{
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || slot < 0 || epoch < 1 || rows <= 0 || n <= 0 ||
        ready_local == nullptr || cta_counters_local == nullptr || ld_partial < n || ld_out < n || row0 < 0) {
        return PTO_B200_EINVAL;
    }
    if ((n & 3) || (ld_partial & 3) || (ld_out & 3)) {
        return PTO_B200_EALIGN;
    }
    KsplitReduceArgs a;
    if (int rc = fill_peers(a.shard.partial, partial_ptrs, world)) {
        return rc;
    }
    if (int rc = fill_peers(a.shard.out, out_ptrs, world)) {
        return rc;
    }
    if (int rc = fill_peers(a.done, done_arrays, world)) {
        return rc;
    }
    for (int r = 0; r < world; ++r) {
        if ((reinterpret_cast<uintptr_t>(partial_ptrs[r]) & 15u) || (reinterpret_cast<uintptr_t>(out_ptrs[r]) & 7u)) {
            return PTO_B200_EALIGN;
        }
    }
    if ((reinterpret_cast<uintptr_t>(multicast_partial) & 15u) || (reinterpret_cast<uintptr_t>(multicast_out) & 7u)) {
        return PTO_B200_EALIGN;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    a.shard.mc_partial = static_cast<const float*>(multicast_partial);
    a.shard.mc_out = multicast_out;
    a.shard.world = world;
    a.shard.row0 = row0;
    a.shard.rows = rows;
    a.shard.n = n;
    a.shard.ld_partial = ld_partial;
    a.shard.ld_out = ld_out;
    a.ready = ready_local;
    a.cta_counter = cta_counters_local;
    a.status = dev->status_ptr;
    a.wait_limit = g_wait_limit.load(std::memory_order_relaxed);
    a.rank = rank;
    a.slot = slot;
    a.epoch = epoch;
    const long long work = (static_cast<long long>(rows) * (n / 4) + kReduceThreads - 1) / kReduceThreads;
    int grid = launch_block_count > 0 ? launch_block_count : 32;
    if (work < grid) {
        grid = static_cast<int>(work);
    }
    ksplit_reduce_kernel<<<grid, kReduceThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "ksplit_reduce launch");
}

extern "C" int pto_b200_ksplit_wait(void* stream, const int* done_local, int world, int slot0, int slots, int epoch)
{
    if (done_local == nullptr || world < 1 || world > kMaxRanks || slot0 < 0 || slots < 1 || epoch < 1) {
        return PTO_B200_EINVAL;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    ksplit_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        done_local, world, slot0, slots, epoch, dev->status_ptr, g_wait_limit.load(std::memory_order_relaxed));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return note_cuda(cudaGetLastError(), "ksplit_wait launch");
}

extern "C" int pto_b200_ksplit_gemm_allreduce(void* stream, const uint8_t* src0, const uint8_t* src1, int m, int n,
                                              int k_local, long long lda, long long ldb, int in_dtype,
                                              void* const* partial_ptrs, void* const* out_ptrs,
                                              void* const* ready_arrays, void* const* done_arrays,
                                              int* panel_counters_local, int* exchange_counters_local, int world,
                                              int rank, int slot0, int epoch, int panel_rows, long long ld_partial,
                                              long long ld_out, const void* multicast_partial, void* multicast_out,
                                              int launch_block_count)
{
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || slot0 < 0 || epoch < 1 ||
        panel_counters_local == nullptr || exchange_counters_local == nullptr || launch_block_count < 0 ||
        panel_rows <= 0 || panel_rows % kPairBlockM != 0 || ld_partial < n || ld_out < n) {
        return PTO_B200_EINVAL;
    }
    if (in_dtype != PTO_B200_F16 && in_dtype != PTO_B200_BF16) {
        return PTO_B200_EDTYPE;
    }
    KsplitFusedArgs fa;
    std::memset(&fa, 0, sizeof(fa));
    if (int rc = fill_peers(fa.partial, partial_ptrs, world)) {
        return rc;
    }
    if (int rc = fill_peers(fa.out, out_ptrs, world)) {
        return rc;
    }
    if (int rc = fill_peers(fa.ready, ready_arrays, world)) {
        return rc;
    }
    if (int rc = fill_peers(fa.done, done_arrays, world)) {
        return rc;
    }
    uint8_t* partial_local = static_cast<uint8_t*>(partial_ptrs[rank]);
    const Problem q{m, n, k_local, lda, ldb, ld_partial};
    if (int rc = check_common(partial_local, src0, src1, q, 2, 2, false)) {
        return rc;
    }
    if ((n & 3) || (ld_partial & 3) || (ld_out & 3)) {
        return PTO_B200_EALIGN;
    }
    for (int r = 0; r < world; ++r) {
        if ((reinterpret_cast<uintptr_t>(partial_ptrs[r]) & 15u) || (reinterpret_cast<uintptr_t>(out_ptrs[r]) & 7u)) {
            return PTO_B200_EALIGN;
        }
    }
    if ((reinterpret_cast<uintptr_t>(multicast_partial) & 15u) || (reinterpret_cast<uintptr_t>(multicast_out) & 7u)) {
        return PTO_B200_EALIGN;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    fa.mc_partial = static_cast<const float*>(multicast_partial);
    fa.mc_out = multicast_out;
    fa.panel_counter = panel_counters_local;
    fa.exchange_counter = exchange_counters_local;
    fa.ld_partial = ld_partial;
    fa.ld_out = ld_out;
    fa.world = world;
    fa.rank = rank;
    fa.epoch = epoch;
    fa.slot0 = slot0;
    fa.panel_tile_rows = panel_rows / kPairBlockM;
    fa.panels = (m + panel_rows - 1) / panel_rows;
    const int kelems = kBlockKBytes / 2;
    GemmParams p;
    fill_params(p, partial_local, q, kPairBlockN, kelems, dev->status_ptr);
    const int fmt = (in_dtype == PTO_B200_BF16) ? 1 : 0;
    p.idesc = make_idesc(1, fmt, fmt, false, kPairBlockN, false, kPairBlockM);
    CUtensorMap ta, tb_half;
    if (int rc = make_tensor_map(&ta, in_dtype, src0, m, k_local, lda, kelems, kBlockM)) {
        return rc;
    }
    if (int rc = make_tensor_map(&tb_half, in_dtype, src1, n, k_local, ldb, kelems, kPairBlockN / 2)) {
        return rc;
    }
    PairLaunch o;
    o.block_limit = launch_block_count;
    o.out_dtype = PTO_B200_F32;
    o.fused = &fa;
    o.no_tma_store = dev->no_tma_store;
    const int rc = launch_pair<KIND_F16, EPI_F32, COMM_KSPLIT>(static_cast<cudaStream_t>(stream), ta, tb_half, p, q, o);
    return rc == -1 ? PTO_B200_EDEVICE : rc;
}

extern "C" int pto_b200_allgather_gemm(void* stream, uint8_t* out, void* const* a_ptrs, const uint8_t* src1, int m, int n,
                                       int k, long long lda, long long ldb, long long ldc, int in_dtype, int out_dtype,
                                       void* const* flag_arrays, int* block_counters_local, int* done_counter_local,
                                       int world, int rank, int epoch, void* multicast_a, int launch_block_count)
{
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || epoch < 1 || block_counters_local == nullptr ||
        done_counter_local == nullptr || launch_block_count < 0 || m <= 0) {
        return PTO_B200_EINVAL;
    }
    if (in_dtype != PTO_B200_F16 && in_dtype != PTO_B200_BF16) {
        return PTO_B200_EDTYPE;
    }
    if (!(out_dtype == PTO_B200_F32 || out_dtype == PTO_B200_BF16 || out_dtype == PTO_B200_F16)) {
        return PTO_B200_EDTYPE;
    }
    // every rank's slice is a whole number of 256-row blocks: a block is the unit that is pushed, flagged and waited for
    if (m % (kPairBlockM * world) != 0) {
        return PTO_B200_EINVAL;
    }
    GatherArgs g;
    std::memset(&g, 0, sizeof(g));
    if (int rc = fill_peers(g.a_full, a_ptrs, world)) {
        return rc;
    }
    if (int rc = fill_peers(g.flags, flag_arrays, world)) {
        return rc;
    }
    const uint8_t* a_local = static_cast<const uint8_t*>(a_ptrs[rank]);
    const Problem q{m, n, k, lda, ldb, ldc};
    if (int rc = check_common(out, a_local, src1, q, 2, 2, false)) {
        return rc;
    }
    for (int r = 0; r < world; ++r) {
        if (reinterpret_cast<uintptr_t>(a_ptrs[r]) & 15u) {
            return PTO_B200_EALIGN;
        }
    }
    if ((k & 7) || (reinterpret_cast<uintptr_t>(multicast_a) & 15u)) { // rows are pushed in 16-byte pieces
        return PTO_B200_EALIGN;
    }
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    g.mc_a = multicast_a;
    g.block_counter = block_counters_local;
    g.done_counter = done_counter_local;
    g.lda_bytes = lda * 2;
    g.row_bytes = k * 2;
    g.world = world;
    g.rank = rank;
    g.epoch = epoch;
    g.blocks_per_rank = m / (kPairBlockM * world);
    const int kelems = kBlockKBytes / 2;
    GemmParams p;
    fill_params(p, out, q, kPairBlockN, kelems, dev->status_ptr);
    const int fmt = (in_dtype == PTO_B200_BF16) ? 1 : 0;
    p.idesc = make_idesc(1, fmt, fmt, false, kPairBlockN, false, kPairBlockM);
    CUtensorMap ta, tb_half;
    if (int rc = make_tensor_map(&ta, in_dtype, a_local, m, k, lda, kelems, kBlockM)) {
        return rc;
    }
    if (int rc = make_tensor_map(&tb_half, in_dtype, src1, n, k, ldb, kelems, kPairBlockN / 2)) {
        return rc;
    }
    PairLaunch o;
    o.block_limit = launch_block_count;
    o.out_dtype = out_dtype;
    o.gather = &g;
    o.no_tma_store = dev->no_tma_store;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc;
    switch (out_dtype) {
        case PTO_B200_F32:
            rc = launch_pair<KIND_F16, EPI_F32, COMM_GATHER>(s, ta, tb_half, p, q, o);
            break;
        case PTO_B200_BF16:
            rc = launch_pair<KIND_F16, EPI_BF16, COMM_GATHER>(s, ta, tb_half, p, q, o);
            break;
        default:
            rc = launch_pair<KIND_F16, EPI_F16, COMM_GATHER>(s, ta, tb_half, p, q, o);
            break;
    }
    return rc == -1 ? PTO_B200_EDEVICE : rc;
}

extern "C" long long pto_b200_set_wait_limit(long long cycles)
{
    return g_wait_limit.exchange(cycles > 0 ? cycles : kWaitLimitCycles, std::memory_order_relaxed);
}

extern "C" void call_kernel(uint32_t blockDim, void* stream, uint8_t* out, uint8_t* src0, uint8_t* src1)
{
    (void)blockDim;
    constexpr int kDim = 6144;
    (void)pto_b200_gemm(stream, out, src0, src1, kDim, kDim, kDim, kDim, kDim, kDim, PTO_B200_F16, PTO_B200_F32,
                        PTO_B200_B_DN);
}

extern "C" int pto_b200_device_status(int* status)
{
    DeviceInfo* dev = nullptr;
    if (int rc = device_info(&dev)) {
        return rc;
    }
    if (int rc = note_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) {
        return rc;
    }
    int host = 0;
    if (int rc = note_cuda(cudaMemcpy(&host, dev->status_ptr, sizeof(int), cudaMemcpyDeviceToHost), "status read")) {
        return rc;
    }
    if (host != 0) {
        const int zero = 0;
        cudaMemcpy(dev->status_ptr, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    if (status != nullptr) {
        *status = host;
    }
    return host == 0 ? PTO_B200_OK : PTO_B200_ETIMEOUT;
}

extern "C" const char* pto_b200_error_string(int code)
{
    switch (code) {
        case PTO_B200_OK:
            return "ok";
        case PTO_B200_EINVAL:
            return "invalid argument (null pointer, non-positive size or leading dimension too small)";
        case PTO_B200_EALIGN:
            return "A/B base address or leading dimension is not a multiple of 16 bytes";
        case PTO_B200_EDTYPE:
            return "unsupported dtype / layout combination";
        case PTO_B200_EWORKSPACE:
            return "workspace missing, misaligned or too small";
        case PTO_B200_ECUDA:
            return "CUDA call failed";
        case PTO_B200_EDEVICE:
            return "current device is not an sm_100 GPU";
        case PTO_B200_ETIMEOUT:
            return "a kernel gave up on a bounded wait";
        case PTO_B200_ESCRATCH:
            return "problem needs more scratch than the library's built-in static array (PTO_B200_MX_STATIC_SCRATCH_BYTES)";
        default:
            return "unknown error code";
    }
}

extern "C" const char* pto_b200_last_cuda_error(void) { return t_cuda_error; }

extern "C" unsigned long long pto_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }


// ---------------------------------------------------------------------------------------------------------------
// MX GEMM for callers that cannot allocate device memory.
//
// Some users of this library have no buffer to give as the scale-factor workspace and no way to get one when they
// call: a launcher that must keep the reference's six-argument LaunchMxMatmul shape, or a process that gave all of
// its device memory to its own pool at start-up so that a later cudaMalloc fails or stalls the GPU. For them the
// scratch is this array inside the library's device image. It costs PTO_B200_MX_STATIC_SCRATCH_BYTES on every GPU
// that loads the library, for the life of the process.
//
// g_mx_static_scratch, as written in host code, is only the host-side handle of the symbol, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
// Every call shares the array and finds the previous call's bytes in it. The re-tile kernels overwrite every atom
// the GEMM kernel reads (rows and K blocks past the end included), so nothing needs clearing; calls that can
// overlap on the GPU race on it and must be serialised by the caller.
namespace pto_b200 {
namespace {

static __device__ __align__(256) uint8_t g_mx_static_scratch[PTO_B200_MX_STATIC_SCRATCH_BYTES];

struct StaticScratch {
    bool ready = false;
    uint8_t* ptr = nullptr;
};
StaticScratch g_static_scratch[kMaxDevices];

// First use on the current device: resolve the device address of the array. Later uses return the cached pointer.
int static_scratch_for_current_device(uint8_t** out)
{
    int dev = 0;
    if (int rc = note_cuda(cudaGetDevice(&dev), "cudaGetDevice")) {
        return rc;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        return PTO_B200_EDEVICE;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    StaticScratch& s = g_static_scratch[dev];
    if (!s.ready) {
        // A failed lookup (for instance a first call made while the stream is being captured) is reported to this
        // caller and tried again by the next one; only a resolved address is cached.
        void* p = nullptr;
        int err = note_cuda(cudaGetSymbolAddress(&p, g_mx_static_scratch), "cudaGetSymbolAddress(mx static scratch)");
        if (err == PTO_B200_OK && p == nullptr) {
            err = PTO_B200_ECUDA;
        }
        if (err != PTO_B200_OK) {
            (void)cudaGetLastError(); // do not leave the failure sticky for the caller's next CUDA call
            return err;
        }
        s.ptr = static_cast<uint8_t*>(p);
        s.ready = true;
    }
    *out = s.ptr;
    return PTO_B200_OK;
}

} // namespace
} // namespace pto_b200

extern "C" int pto_b200_gemm_mx_static(void* stream, uint8_t* out, const uint8_t* src0, const uint8_t* src1,
                                       const uint8_t* src2, const uint8_t* src3, int m, int n, int k, long long lda,
                                       long long ldb, long long ldc, long long ld_sfa, long long ld_sfb, int a_dtype,
                                       int b_dtype, int out_dtype)
{
    // the same argument errors, in the same order, as pto_b200_gemm_mx, before any CUDA call is made
    if (int rc = mx_check_args(out, src0, src1, src2, src3, m, n, k, lda, ldb, ldc, ld_sfa, ld_sfb, a_dtype, b_dtype,
                               out_dtype, nullptr)) {
        return rc;
    }
    if (pto_b200_gemm_mx_workspace_bytes(m, n, k) > static_cast<size_t>(PTO_B200_MX_STATIC_SCRATCH_BYTES)) {
        return PTO_B200_ESCRATCH;
    }
    uint8_t* scratch = nullptr;
    if (int rc = static_scratch_for_current_device(&scratch)) {
        return rc;
    }
    return pto_b200_gemm_mx(stream, out, src0, src1, src2, src3, scratch, PTO_B200_MX_STATIC_SCRATCH_BYTES, m, n, k,
                            lda, ldb, ldc, ld_sfa, ld_sfb, a_dtype, b_dtype, out_dtype);
}
