// Two-CTA form of the GEMM tile loop: a cluster of two CTAs (one per SM) owns a 256 x 256 output tile and
// issues `tcgen05.mma.cta_group::2`. Each CTA stages its own 128 rows of A and its own 128 columns of B
// (B column-major), so every B byte is loaded and read from shared memory once per pair instead of once per
// CTA; each CTA's tensor memory holds its 128 rows of the accumulator, all 256 columns.
//
// Roles per CTA are those of gemm_tile_loop (TLOAD warp, MMA warp, four TSTORE warps); only the leader CTA
// (cluster rank 0) issues MMAs. Hand-offs across the pair:
//   full[stage]   lives in the leader; both CTAs' TMA loads complete their bytes on it (no multicast: each CTA
//                 loads different data, the `.cta_group::2` form only lets the completion land in the peer)
//   empty[stage]  one in each CTA, released by the leader's tcgen05.commit to both
//   acc_full[a]   one in each CTA, published by the leader's tcgen05.commit to both
//   acc_empty[a]  lives in the leader; the peer's TSTORE warps arrive on it across the cluster
//
// TSTORE: a finished accumulator leaves tensor memory through registers into a 128-byte-swizzled shared-memory
// buffer per warp and from there with TMA tensor stores (one 32-row x 128-byte box at a time), so the tensor
// memory is free again after the read-back instead of after the global stores, and every store is a full line.
// When C does not meet the TMA alignment rule the warps store from registers as gemm_tile_loop does.
//
// Block-scaled kind: the e8m0 scale atoms of a stage arrive in shared memory with the operands; the MMA warp of the
// second CTA, which issues no MMAs, copies them into tensor memory (tcgen05.cp, every stage of the ring has its own
// scale columns) and commits to the leader, so no scale copy sits in the leader's MMA instruction stream.
//
// K-split form (COMM_KSPLIT): the kernel of one rank of the reference's GEMM + AllReduce
// (kernels/manual/a2a3/gemm_ar: gemm_compute_kernel.cpp:150-240 fills a ready queue tile by tile, comm_kernel.cpp
// :165-210 reduce-scatters, :377-400 all-gathers, :528-590 waits). Here both halves are ONE kernel: the tile loop
// walks the output row panel by row panel and counts finished tiles per panel; the warp that completes a panel
// publishes ready[panel][rank] to every rank; four extra warps per CTA (the exchange role) wait for all ranks' flags
// of a panel, sum this rank's row shard of it over the ranks' fp32 partials through peer memory (NVSwitch multimem
// or plain peer loads), cast to bf16, store the result into every rank's output, publish done[panel][rank], and at
// the end wait until every rank has delivered every panel here. No TMA load and no multicast load touches peer memory.
//
// All-gather form (COMM_GATHER): the kernel of one rank of the reference's AllGather + GEMM
// (kernels/manual/a2a3/allgather_gemm: every rank holds an M slice of A, B is replicated, every rank computes the
// whole C; allgather_gemm_comm_kernel.cpp pushes chunks and counts them, allgather_gemm_compute_kernel.cpp:393 waits per
// chunk and multiplies, local rows first). Here the four extra warps per CTA push this rank's slice of A, 256-row
// block by block, into every rank's copy of A (one NVSwitch multicast store per 16 bytes, or one store per peer) and
// publish arrived[block] to every rank; the tile loop starts with this rank's own rows and its TLOAD role waits for a
// remote block's flag before the first TMA load of a tile in it. TMA reads this GPU's own copy of A only.
//
// Every wait is bounded as in gemm_tile_loop; the pair leaves through a cluster barrier so neither CTA's shared
// or tensor memory disappears while the other can still touch it.
#pragma once
#include "gemm_tile_loop.cuh"
#include "ksplit_reduce.cuh"

namespace pto_b200 {

constexpr int kPairBlockM = 256;
constexpr int kPairBlockN = 256;

constexpr int ST_TAIL_TIMEOUT = 5;

constexpr int kExchangeThreads = 128; // four exchange warps per CTA in the K-split form
constexpr int kExchangeBarrierId = 1;
constexpr int ST_SCALE_TIMEOUT = 6;
constexpr int ST_GATHER_TIMEOUT = 18; // a remote block of A never arrived, or a rank never finished the previous step

__device__ __forceinline__ int ld_acquire_gpu(const int* ptr)
{
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

// What the K-split form needs besides the GEMM's own arguments. Peer pointer arrays hold one entry per rank (the
// rank's buffer as mapped in this process, own rank included).
struct KsplitFusedArgs {
    PeerPointers ready;      // every rank's ready-flag array
    PeerPointers done;       // every rank's done-flag array
    PeerPointers partial;    // every rank's fp32 partial [m, ld_partial] of this step
    PeerPointers out;        // every rank's bf16 output [m, ld_out]
    const float* mc_partial; // NVSwitch multicast address of the partials, or null (plain peer loads)
    void* mc_out;            // NVSwitch multicast address of the outputs, or null (one store per rank)
    int* panel_counter;      // local, one int per slot, zero between steps: finished TSTORE warps of a panel
    int* exchange_counter;   // local, one int per slot, zero between steps: CTAs that reduced their part of a shard
    long long ld_partial, ld_out;
    int world, rank, epoch;
    int slot0;               // first flag slot of this step (slots alternate with the partial buffer)
    int panels;              // row panels of the output
    int panel_tile_rows;     // 256-row tiles per panel (= the raster's group height)
};

// What the extra warps of a CTA do: nothing (no extra warps), the K-split exchange, or the all-gather push.
enum CommMode : int { COMM_NONE = 0, COMM_KSPLIT = 1, COMM_GATHER = 2 };

// What the all-gather form needs besides the GEMM's own arguments.
struct GatherArgs {
    PeerPointers a_full;    // every rank's copy of A [m, lda] (own rank included); rank r owns rows [r m/world, (r+1) m/world)
    PeerPointers flags;     // every rank's flag array: arrived[m_tiles] then done[kMaxRanks], epochs
    void* mc_a;             // NVSwitch multicast address of the A copies, or null (one store per peer)
    int* block_counter;     // local, one int per block of a slice, zero between steps: CTAs that pushed their part
    int* done_counter;      // local, one int, zero between steps: CTAs that finished the step
    long long lda_bytes;    // row pitch of A
    int row_bytes;          // bytes of a row that carry data (k elements), a multiple of 16
    int world, rank, epoch;
    int blocks_per_rank;    // 256-row blocks in one rank's slice
};

__device__ __forceinline__ void multimem_st_b128(void* mc_ptr, const uint4& v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

__device__ __forceinline__ void st_relaxed_sys_b128(void* ptr, const uint4& v)
{
    asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(ptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Ring stages and store boxes per TSTORE warp of the block-scaled instantiations (one accumulator, so the read-back
// is not hidden behind the next tile's MMAs). Measured on 16384 x 8192 x 8192: 6 stages + 1 box, 5 + 2, 5 + 3 and
// 4 + 4 all take 0.886-0.895 ms, so neither the ring depth nor a wait for a store box limits this kernel.
#ifndef PTO_B200_MX_PAIR_STAGES
#define PTO_B200_MX_PAIR_STAGES 6
#endif
#ifndef PTO_B200_MX_EPI_BUFS
#define PTO_B200_MX_EPI_BUFS 1
#endif
template <int KIND>
inline constexpr int kPairEpiBufs = (KIND == KIND_MXF8) ? PTO_B200_MX_EPI_BUFS : 2;

template <int KIND, int STAGES, int EPI_BUFS>
struct PairSmemLayout {
    static constexpr int kABytes = kBlockM * kBlockKBytes;        // this CTA's 128 rows of A
    static constexpr int kBBytes = (kPairBlockN / 2) * kBlockKBytes; // this CTA's 128 columns of B
    static constexpr int kSfaBytes = (KIND == KIND_MXF8) ? 512 : 0;
    static constexpr int kSfbBytes = (KIND == KIND_MXF8) ? 1024 : 0; // scales of all 256 columns, in both CTAs
    static constexpr int kStageBytes = kABytes + kBBytes; // operand bytes per CTA that complete on the leader's barrier
    static constexpr int kEpiBufBytes = 32 * 128;                 // 32 rows x 128 bytes: one TMA store box
    static constexpr int kEpiBytes = 4 * EPI_BUFS * kEpiBufBytes; // per TSTORE warp EPI_BUFS buffers
    static constexpr int kAOff = 0;
    static constexpr int kBOff = STAGES * kABytes;
    static constexpr int kEpiOff = kBOff + STAGES * kBBytes;      // 1024-byte aligned (swizzle atom)
    static constexpr int kSfaOff = kEpiOff + kEpiBytes;
    static constexpr int kSfbOff = kSfaOff + STAGES * kSfaBytes;
    static constexpr int kBarOff = kSfbOff + STAGES * kSfbBytes;
    // per stage: full, empty, scale bytes landed (local), scales in tensor memory (leader); 2 x 2 accumulator barriers
    static constexpr int kNumBars = 4 * STAGES + 4;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;
    static constexpr int kTotal = kMiscOff + 16 + 1024;
};

// One unit of work of a CTA pair: a whole 256 x 256 tile, or one K half of a tile of the last, partly filled wave.
struct PairUnit {
    int mi, ni;
    int kb0, kb1; // k-block range
    int role;     // 0 whole tile; 1 first K half (parks its accumulators); 2 second K half (adds them, stores)
    int tail_idx; // index of the tile among the split ones
};

__device__ __forceinline__ bool pair_unit(int u, const GemmParams& p, PairUnit& w)
{
    if (u < p.tail_first_unit) {
        tile_coords(u, p, w.mi, w.ni);
        if (p.mi_rotate != 0) { // all-gather form: the raster starts at this rank's own rows
            w.mi = (w.mi + p.mi_rotate) % p.m_tiles;
        }
        w.kb0 = 0;
        w.kb1 = p.k_blocks;
        w.role = 0;
        w.tail_idx = 0;
        return true;
    }
    const int t = u - p.tail_first_unit;
    if (t >= 2 * p.tail_tiles) {
        return false;
    }
    w.tail_idx = t >> 1;
    tile_coords(p.tail_first_unit + w.tail_idx, p, w.mi, w.ni);
    const int mid = p.k_blocks / 2;
    w.role = 1 + (t & 1);
    w.kb0 = (w.role == 1) ? 0 : mid;
    w.kb1 = (w.role == 1) ? mid : p.k_blocks;
    return true;
}

constexpr int kTailWarps = 8; // store warps of a pair: four in each CTA

// Parked accumulators of a split tile: per CTA and K half 128 rows x 128 columns of 32-bit words, laid out so that a
// warp's 16-byte accesses are contiguous: 16-byte index (chunk * 8 + i) * 128 + row for the i-th 16 bytes of the
// 32-column chunk `chunk` (0..3) of row `row`.
__device__ __forceinline__ uint4* parked_quad(uint32_t* cta_base, int chunk, int i, int row_in_cta)
{
    return reinterpret_cast<uint4*>(cta_base) + (chunk * 8 + i) * kBlockM + row_in_cta;
}

__device__ __forceinline__ void st_release_gpu(int* ptr, int v)
{
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}

template <int KIND, int STAGES, int EPI, int COMM>
__global__ void __cluster_dims__(2, 1, 1)
    __launch_bounds__(kNumThreads + (COMM != COMM_NONE ? kExchangeThreads : 0), 1)
    gemm_tile_loop_2cta(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                        const __grid_constant__ CUtensorMap tmap_c, const GemmParams p, const KsplitFusedArgs ar,
                        const GatherArgs ga)
{
    constexpr bool FUSED_AR = (COMM == COMM_KSPLIT);
    static_assert(COMM != COMM_GATHER || KIND == KIND_F16, "the all-gather form multiplies 16-bit inputs");
    constexpr int kEpiBufs = kPairEpiBufs<KIND>;
    using L = PairSmemLayout<KIND, STAGES, kEpiBufs>;
    constexpr int kNumAcc = (KIND == KIND_MXF8) ? 1 : 2;
    constexpr int kAccCols = 256;
    constexpr uint32_t kSfCol0 = 256;   // scale columns of stage s: [kSfCol0 + 12 s, +4) for A, the next 8 for B
    constexpr uint32_t kSfColsPerStage = 12;
    static_assert(KIND != KIND_MXF8 || kAccCols + STAGES * 12 <= kTmemCols, "scale columns of every stage beside one accumulator");
    constexpr int kBlockKElems = (KIND == KIND_F16) ? 64 : 128;
    constexpr bool kOut32 = (EPI == EPI_F32 || EPI == EPI_S32);
    constexpr int kWords = OutWords<EPI>::kCount;
    static_assert(!FUSED_AR || (KIND == KIND_F16 && EPI == EPI_F32), "the K-split form multiplies 16-bit inputs into fp32 partials");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* sf_landed_bar = empty_bar + STAGES;   // second CTA: both CTAs' scale atoms of the stage are in shared memory
    uint64_t* sf_full_bar = sf_landed_bar + STAGES; // leader: the stage's scales are in both CTAs' tensor memory
    uint64_t* acc_full_bar = sf_full_bar + STAGES;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOff + 4);
    volatile uint32_t* exchange_ok = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOff + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = ptx::cluster_ctarank();
    const bool leader = (cta_rank == 0);
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
            ptx::mbar_init(&sf_landed_bar[s], 1);
            ptx::mbar_init(&sf_full_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&acc_full_bar[a], 1);
            ptx::mbar_init(&acc_empty_bar[a], 8); // four TSTORE warps in each CTA of the pair
        }
        *abort_flag = 0;
        *exchange_ok = 1;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        if (p.tma_store != 0) {
            ptx::prefetch_tensormap(&tmap_c);
        }
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(tmem_base_slot, kTmemCols);
        ptx::tmem_relinquish_alloc_permit_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive(); // the peer's barriers must exist before anything is signalled across the pair
    ptx::cluster_wait();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TLOAD role (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            PairUnit w;
            for (int u = pair; ok && pair_unit(u, p, w); u += num_pairs) {
                const int mi = w.mi, ni = w.ni;
                const int row_a = mi * kPairBlockM + static_cast<int>(cta_rank) * kBlockM;
                const int row_b = ni * kPairBlockN + static_cast<int>(cta_rank) * (kPairBlockN / 2);
                if constexpr (COMM == COMM_GATHER) {
                    // rows of another rank: wait until its push of this 256-row block has been published here, then
                    // order the peer's (generic-proxy) writes before this thread's TMA (async-proxy) reads
                    if (mi / ga.blocks_per_rank != ga.rank) {
                        const int* arrived = static_cast<const int*>(ga.flags.p[ga.rank]);
                        if (!wait_epoch(arrived + mi, ga.epoch, p.status, ST_GATHER_TIMEOUT, p.wait_limit)) {
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        asm volatile("fence.proxy.async;" ::: "memory");
                    }
                }
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    ok = bounded_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, ST_PRODUCER_TIMEOUT,
                                      p.wait_limit);
                    if (!ok) {
                        break;
                    }
                    if (leader) {
                        ptx::mbar_arrive_expect_tx(&full_bar[stage], (2u * L::kStageBytes) >> p.packed4);
                    }
                    const uint32_t full_addr = ptx::map_to_cta(ptx::smem_u32(&full_bar[stage]), 0);
                    ptx::tma_load_2d_pair(smem + L::kAOff + stage * L::kABytes, &tmap_a, full_addr, kb * kBlockKElems,
                                          row_a);
                    ptx::tma_load_2d_pair(smem + L::kBOff + stage * L::kBBytes, &tmap_b, full_addr, kb * kBlockKElems,
                                          row_b);
                    if constexpr (KIND == KIND_MXF8) {
                        // Scale atoms through tensor maps over the re-tiled workspace viewed as rows of 256 bytes
                        // (an atom is two rows): A rows of this CTA (row block 2*mi + rank), B columns of the whole
                        // tile (two atoms). Both CTAs' scale bytes complete on a barrier of the second CTA, whose
                        // otherwise idle MMA warp copies them into tensor memory.
                        const int sfa_row = (kb * (2 * p.m_tiles) + 2 * mi + static_cast<int>(cta_rank)) * 2;
                        const int sfb_row = (kb * p.n_tiles + ni) * 4;
                        if (!leader) {
                            ptx::mbar_arrive_expect_tx(&sf_landed_bar[stage], 2u * (L::kSfaBytes + L::kSfbBytes));
                        }
                        const uint32_t landed_addr = ptx::map_to_cta(ptx::smem_u32(&sf_landed_bar[stage]), 1);
                        ptx::tma_load_2d_pair(smem + L::kSfaOff + stage * L::kSfaBytes, &tmap_sfa, landed_addr, 0, sfa_row);
                        ptx::tma_load_2d_pair(smem + L::kSfbOff + stage * L::kSfbBytes, &tmap_sfb, landed_addr, 0, sfb_row);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if constexpr (KIND == KIND_MXF8) {
            // ------------------------------------------------------------ scale copies (second CTA's MMA warp)
            // tcgen05.cp.cta_group::2 copies the same shared-memory offsets of both CTAs into both CTAs' tensor
            // memory; every stage of the ring has its own 12 scale columns. Issued from the CTA that issues no MMAs,
            // the copies stay out of the leader's MMA instruction stream; the commit tells the leader.
            if (!leader && lane == 0) {
                int stage = 0;
                uint32_t phase = 0;
                bool ok = true;
                PairUnit w;
                for (int u = pair; ok && pair_unit(u, p, w); u += num_pairs) {
                    for (int kb = w.kb0; kb < w.kb1; ++kb) {
                        ok = bounded_wait(&sf_landed_bar[stage], phase, abort_flag, p.status, ST_SCALE_TIMEOUT,
                                          p.wait_limit);
                        if (!ok) {
                            break;
                        }
                        ptx::tc_fence_after_sync();
                        const uint32_t sfa_base = ptx::smem_u32(smem + L::kSfaOff + stage * L::kSfaBytes);
                        const uint32_t sfb_base = ptx::smem_u32(smem + L::kSfbOff + stage * L::kSfbBytes);
                        const uint32_t sf = tmem_base + kSfCol0 + kSfColsPerStage * static_cast<uint32_t>(stage);
                        ptx::tmem_cp_32x128b_warpx4_pair(sf, ptx::make_smem_desc(sfa_base, 0, 128, ptx::kSwizzleNone));
                        ptx::tmem_cp_32x128b_warpx4_pair(sf + 4u, ptx::make_smem_desc(sfb_base, 0, 128, ptx::kSwizzleNone));
                        ptx::tmem_cp_32x128b_warpx4_pair(sf + 8u,
                                                         ptx::make_smem_desc(sfb_base + 512u, 0, 128, ptx::kSwizzleNone));
                        ptx::umma_commit_pair(&sf_full_bar[stage], 0x1);
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
            }
        }
        // ---------------------------------------------------------------- TMATMUL / TMATMUL_ACC role (leader only)
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            PairUnit w;
            for (int u = pair; ok && pair_unit(u, p, w); u += num_pairs) {
                ok = bounded_wait(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag, p.status, ST_MMA_ACC_TIMEOUT,
                                  p.wait_limit);
                if (!ok) {
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kAccCols);
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    ok = bounded_wait(&full_bar[stage], phase, abort_flag, p.status, ST_MMA_FULL_TIMEOUT, p.wait_limit);
                    if (!ok) {
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_base = ptx::smem_u32(smem + L::kAOff + stage * L::kABytes);
                    const uint32_t b_base = ptx::smem_u32(smem + L::kBOff + stage * L::kBBytes);
                    if constexpr (KIND == KIND_MXF8) {
                        // the scale role of both CTAs has put this stage's scales into tensor memory
                        ok = bounded_wait(&sf_full_bar[stage], phase, abort_flag, p.status, ST_SCALE_TIMEOUT, p.wait_limit);
                        if (!ok) {
                            break;
                        }
                        ptx::tc_fence_after_sync();
                    }
#pragma unroll
                    for (int kk = 0; kk < kBlockKBytes / kUmmaKBytes; ++kk) {
                        const uint64_t a_desc =
                            ptx::make_smem_desc(a_base + kk * kUmmaKBytes, 16, 1024, ptx::kSwizzle128B);
                        const uint64_t b_desc =
                            ptx::make_smem_desc(b_base + kk * kUmmaKBytes, 16, 1024, ptx::kSwizzle128B);
                        const uint32_t accumulate = (kb > w.kb0 || kk > 0) ? 1u : 0u;
                        if constexpr (KIND == KIND_F16) {
                            ptx::umma_f16_pair(d_tmem, a_desc, b_desc, p.idesc, accumulate);
                        } else if constexpr (KIND == KIND_I8) {
                            ptx::umma_i8_pair(d_tmem, a_desc, b_desc, p.idesc, accumulate);
                        } else {
                            const uint32_t idesc =
                                p.idesc | (static_cast<uint32_t>(kk) << 4) | (static_cast<uint32_t>(kk) << 29);
                            const uint32_t sf = tmem_base + kSfCol0 + kSfColsPerStage * static_cast<uint32_t>(stage);
                            ptx::umma_mxf8_pair(d_tmem, a_desc, b_desc, idesc, sf, sf + 4u, accumulate);
                        }
                    }
                    ptx::umma_commit_pair(&empty_bar[stage], 0x3);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) {
                    break;
                }
                ptx::umma_commit_pair(&acc_full_bar[acc], 0x3);
                if (++acc == kNumAcc) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- TSTORE role (both CTAs)
        const int quarter = warp & 3;
        const int esize = kOut32 ? 4 : (EPI == EPI_QUANT8 ? 1 : 2);
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0) && (((p.ldc * esize) & 15) == 0);
        uint8_t* epi_buf = smem + L::kEpiOff + quarter * kEpiBufs * L::kEpiBufBytes;
        uint8_t* my_line = epi_buf + lane * 128; // this thread's row inside a store box
        int acc = 0;
        uint32_t acc_phase = 0;
        uint32_t boxes = 0; // TMA store boxes this warp has issued
        bool ok = true;
        PairUnit w;
        for (int u = pair; ok && pair_unit(u, p, w); u += num_pairs) {
            const int mi = w.mi, ni = w.ni;
            ok = bounded_wait(&acc_full_bar[acc], acc_phase, abort_flag, p.status, ST_EPILOGUE_TIMEOUT, p.wait_limit);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) {
                break;
            }
            ptx::tc_fence_after_sync();
            const int row_in_cta = quarter * 32 + lane;
            const int row0_warp = mi * kPairBlockM + static_cast<int>(cta_rank) * kBlockM + quarter * 32;
            const int row = row0_warp + lane;
            float s_row = 1.0f;
            if constexpr (EPI == EPI_DEQ_BF16) {
                s_row = (row < p.m) ? __ldg(p.s_row + row) : 0.0f;
            }
            const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * kAccCols) +
                                   (static_cast<uint32_t>(quarter * 32) << 16);
            const bool use_tma = (p.tma_store != 0);
            // One finished 32-column chunk of this thread's row: convert and either write the words into the warp's
            // swizzled store box (a box is one chunk of 32-bit outputs or two chunks of 16-bit outputs; the box leaves
            // with one TMA store when it is full) or store them from registers.
            auto finish_chunk = [&](uint32_t (&v)[32], int chunk) {
                constexpr int kChunksPerBox = kOut32 ? 1 : 2;
                const int col0 = ni * kPairBlockN + chunk * 32;
                // nothing to do past N; a store box that starts before N is still filled and sent whole (TMA clips it)
                if ((use_tma ? col0 - (chunk % kChunksPerBox) * 32 : col0) >= p.n) {
                    return;
                }
                if (!use_tma) {
                    store_chunk<EPI>(v, p, row, col0, vec_ok, s_row);
                    return;
                }
                uint32_t o[kWords];
                convert_chunk<EPI>(v, p, col0, s_row, o);
                const int part = chunk % kChunksPerBox; // which half of the 128-byte line (16-bit outputs)
                uint8_t* line = my_line + (boxes % kEpiBufs) * L::kEpiBufBytes;
                if (part == 0) {
                    // the box that used this buffer kEpiBufs boxes ago must have been read out of shared memory
                    if (lane == 0) {
                        ptx::bulk_wait_group_read<kEpiBufs - 1>();
                    }
                    __syncwarp();
                }
                constexpr int kQuads = kWords / 4; // 16-byte pieces this chunk fills: 8 (32-bit) or 4 (16-bit)
#pragma unroll
                for (int i = 0; i < kQuads; ++i) {
                    const int piece = part * kQuads + i;          // 0..7 within the 128-byte line
                    const int sw = piece ^ (lane & 7);            // 128-byte swizzle: piece index XOR (row mod 8)
                    *reinterpret_cast<uint4*>(line + sw * 16) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                }
                if (part == kChunksPerBox - 1) {
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const int box_col0 = col0 - part * 32;
                        ptx::tma_store_2d(&tmap_c, epi_buf + (boxes % kEpiBufs) * L::kEpiBufBytes, box_col0, row0_warp);
                        ptx::bulk_commit_group();
                    }
                    ++boxes;
                }
            };
            auto release_accumulator = [&]() {
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (leader) {
                        ptx::mbar_arrive(&acc_empty_bar[acc]);
                    } else {
                        ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&acc_empty_bar[acc]), 0));
                    }
                }
            };
            if (w.role == 0) {
                // Accumulator read-back, software-pipelined over 32-column chunks: the TMEM load of the next chunk is
                // in flight while the current one is converted and stored (columns past N are loaded but never
                // stored). The accumulator is handed back to the MMA role as soon as its last chunk is in registers.
                uint32_t va[32], vb[32];
                ptx::tmem_ld_32x32b_x32(t_row + 0u, va);
#pragma unroll
                for (int g = 0; g < kPairBlockN / 64; ++g) {
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(g * 64 + 32), vb);
                    finish_chunk(va, g * 2 + 0);
                    ptx::tmem_ld_wait();
                    if (g + 1 < kPairBlockN / 64) {
                        ptx::tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>(g * 64 + 64), va);
                    } else {
                        release_accumulator();
                    }
                    finish_chunk(vb, g * 2 + 1);
                }
            } else {
                // A tile of the last, partly filled wave, cut into two K halves on two pairs. The halves swap: each
                // pair parks the accumulators of the 128 columns the OTHER pair will finish (role 1 finishes columns
                // 0..127, role 2 columns 128..255), tells the other, waits for the other's half, adds it to its own
                // accumulators and stores. Both pairs do the same amount of work and neither waits for a whole
                // read-back of the other. Flags carry this launch's token, so nothing is counted and nothing needs
                // resetting, whatever an earlier launch left behind.
                const int keep0 = (w.role == 1) ? 0 : 4;   // first of the four chunks this pair finishes
                const int give0 = 4 - keep0;
                const size_t half_words = static_cast<size_t>(kBlockM) * (kPairBlockN / 2);
                uint32_t* mine_parked = p.ws_partial + ((static_cast<size_t>(w.tail_idx) * 2 + (w.role - 1)) * 2 + cta_rank) * half_words;
                uint32_t* theirs_parked = p.ws_partial + ((static_cast<size_t>(w.tail_idx) * 2 + (2 - w.role)) * 2 + cta_rank) * half_words;
                int* my_flags = p.ws_flags + (w.tail_idx * 2 + (w.role - 1)) * kTailWarps;
                const int* their_flags = p.ws_flags + (w.tail_idx * 2 + (2 - w.role)) * kTailWarps;
                uint32_t v[32];
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    ptx::tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>((give0 + c) * 32), v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        *parked_quad(mine_parked, c, i, row_in_cta) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    }
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    st_release_gpu(my_flags + static_cast<int>(cta_rank) * 4 + quarter, p.tail_token);
                }
                // wait (bounded) until all eight store warps of the other pair have parked their half
                bool parked = true;
                if (lane < kTailWarps) {
                    const long long t0 = clock64();
                    while (ld_acquire_gpu(their_flags + lane) != p.tail_token) {
                        __nanosleep(32);
                        if (*abort_flag != 0 || clock64() - t0 > p.wait_limit) {
                            *abort_flag = 1;
                            atomicCAS(p.status, 0, ST_TAIL_TIMEOUT);
                            parked = false;
                            break;
                        }
                    }
                }
                parked = __all_sync(0xFFFFFFFFu, parked);
                if (!parked) {
                    ok = false;
                    break;
                }
                // finish this pair's four chunks; the parked values of the next chunk are in flight meanwhile
                uint4 qa[8], qb[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    qa[i] = __ldcg(parked_quad(theirs_parked, 0, i, row_in_cta));
                }
                auto add_parked = [&](const uint4 (&q)[8]) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t qv[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if constexpr (EPI == EPI_S32 || EPI == EPI_DEQ_BF16 || EPI == EPI_QUANT16 || EPI == EPI_QUANT8) {
                                if ((EPI != EPI_QUANT16 && EPI != EPI_QUANT8) || (p.quant_flags & QUANT_ACC_S32) != 0) {
                                    v[4 * i + j] += qv[j]; // int32 accumulators: exact
                                } else {
                                    v[4 * i + j] = __float_as_uint(__uint_as_float(qv[j]) + __uint_as_float(v[4 * i + j]));
                                }
                            } else {
                                v[4 * i + j] = __float_as_uint(__uint_as_float(qv[j]) + __uint_as_float(v[4 * i + j]));
                            }
                        }
                    }
                };
#pragma unroll
                for (int c = 0; c < 4; c += 2) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        qb[i] = __ldcg(parked_quad(theirs_parked, c + 1, i, row_in_cta));
                    }
                    ptx::tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>((keep0 + c) * 32), v);
                    ptx::tmem_ld_wait();
                    add_parked(qa);
                    finish_chunk(v, keep0 + c);
                    if (c + 2 < 4) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            qa[i] = __ldcg(parked_quad(theirs_parked, c + 2, i, row_in_cta));
                        }
                    }
                    ptx::tmem_ld_32x32b_x32(t_row + static_cast<uint32_t>((keep0 + c + 1) * 32), v);
                    ptx::tmem_ld_wait();
                    if (c + 2 >= 4) {
                        release_accumulator();
                    }
                    add_parked(qb);
                    finish_chunk(v, keep0 + c + 1);
                }
            }
            if constexpr (FUSED_AR) {
                // This warp's rows of the tile are written: count it for the tile's row panel. The warp that completes
                // the panel tells every rank that this rank's partial of the panel can be read.
                if (use_tma) {
                    if (lane == 0) {
                        ptx::bulk_wait_group<0>(); // the box stores have been performed, not merely read out
                    }
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    const int panel = mi / ar.panel_tile_rows;
                    const int tile_rows = min(p.m_tiles - panel * ar.panel_tile_rows, ar.panel_tile_rows);
                    const int expected = tile_rows * p.n_tiles * kTailWarps;
                    const int slot = ar.slot0 + panel;
                    if (atomicAdd(ar.panel_counter + slot, 1) == expected - 1) {
                        ar.panel_counter[slot] = 0;
                        __threadfence_system();
                        for (int r = 0; r < ar.world; ++r) {
                            st_release_sys(static_cast<int*>(ar.ready.p[r]) + slot * kFlagStride + ar.rank, ar.epoch);
                        }
                    }
                }
            }
            if (++acc == kNumAcc) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        // shared memory must outlive the reads of the last store boxes
        if (lane == 0) {
            ptx::bulk_wait_group_read<0>();
        }
    } else if constexpr (COMM == COMM_GATHER) {
        // ---------------------------------------------------------------- gather role (both CTAs, all-gather form)
        const int tid = static_cast<int>(threadIdx.x) - kNumThreads;
        const int* my_flags = static_cast<const int*>(ga.flags.p[ga.rank]);
        // Nobody may still be reading the previous step's rows: every rank published done[r] = epoch - 1 when its
        // last tile was loaded (flags start at zero, so the first step passes at once).
        if (tid < ga.world) {
            if (!wait_epoch(my_flags + p.m_tiles + tid, ga.epoch - 1, p.status, ST_GATHER_TIMEOUT, p.wait_limit)) {
                *exchange_ok = 0;
            }
        }
        ptx::named_barrier_sync(kExchangeBarrierId, kExchangeThreads);
        const bool ok = (*exchange_ok != 0);
        const int items_per_row = ga.row_bytes / 16;
        const uint8_t* mine = static_cast<const uint8_t*>(ga.a_full.p[ga.rank]);
        // The CTAs of the launch form up to four groups; group g pushes blocks g, g + groups, ... of the slice, so
        // several blocks are in flight at once and the wait for one block's stores to be acknowledged by the peers
        // (the system-scope fence before its flag) overlaps the next blocks' stores. Blocks still complete roughly
        // in the order the peers consume them.
        const int groups = min(ga.blocks_per_rank, min(4, static_cast<int>(gridDim.x)));
        const int group = static_cast<int>(blockIdx.x) % groups;
        const int group_ctas = (static_cast<int>(gridDim.x) - group + groups - 1) / groups;
        const long long first = static_cast<long long>(blockIdx.x / groups) * kExchangeThreads + tid;
        const long long stride = static_cast<long long>(group_ctas) * kExchangeThreads;
        for (int b = group; ok && ga.world > 1 && b < ga.blocks_per_rank; b += groups) {
            const int block = ga.rank * ga.blocks_per_rank + b;
            const int row0 = block * kPairBlockM;
            const int rows = min(kPairBlockM, p.m - row0);
            const long long total = static_cast<long long>(rows) * items_per_row;
            constexpr int kUnroll = 4;
            for (long long i0 = first; i0 < total; i0 += stride * kUnroll) {
                uint4 v[kUnroll];
                long long off[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const long long i = i0 + u * stride;
                    off[u] = -1;
                    if (i < total) {
                        off[u] = (row0 + i / items_per_row) * ga.lda_bytes + (i % items_per_row) * 16;
                        v[u] = __ldg(reinterpret_cast<const uint4*>(mine + off[u]));
                    }
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    if (off[u] < 0) {
                        continue;
                    }
                    if (ga.mc_a != nullptr) {
                        multimem_st_b128(static_cast<uint8_t*>(ga.mc_a) + off[u], v[u]);
                    } else {
                        for (int r = 0; r < ga.world; ++r) {
                            if (r != ga.rank) {
                                st_relaxed_sys_b128(static_cast<uint8_t*>(ga.a_full.p[r]) + off[u], v[u]);
                            }
                        }
                    }
                }
            }
            // the last CTA of the group to finish its part of the block publishes it to every rank
            __threadfence_system();
            ptx::named_barrier_sync(kExchangeBarrierId, kExchangeThreads);
            if (tid == 0) {
                if (atomicAdd(ga.block_counter + b, 1) == group_ctas - 1) {
                    ga.block_counter[b] = 0;
                    __threadfence_system();
                    for (int r = 0; r < ga.world; ++r) {
                        st_release_sys(static_cast<int*>(ga.flags.p[r]) + block, ga.epoch);
                    }
                }
            }
        }
    } else if constexpr (FUSED_AR) {
        // ---------------------------------------------------------------- exchange role (both CTAs, K-split form)
        const int tid = static_cast<int>(threadIdx.x) - kNumThreads;
        const long long first = static_cast<long long>(blockIdx.x) * kExchangeThreads + tid;
        const long long stride = static_cast<long long>(gridDim.x) * kExchangeThreads;
        const int* ready_local = static_cast<const int*>(ar.ready.p[ar.rank]);
        const int* done_local = static_cast<const int*>(ar.done.p[ar.rank]);
        const int panel_rows = ar.panel_tile_rows * kPairBlockM;
        bool ok = true;
        for (int panel = 0; panel < ar.panels; ++panel) {
            const int slot = ar.slot0 + panel;
            if (tid < ar.world) {
                if (!wait_epoch(ready_local + slot * kFlagStride + tid, ar.epoch, p.status, ST_KSPLIT_READY_TIMEOUT,
                                p.wait_limit)) {
                    *exchange_ok = 0;
                }
            }
            ptx::named_barrier_sync(kExchangeBarrierId, kExchangeThreads);
            ok = (*exchange_ok != 0);
            if (ok) {
                // this rank's row shard of the panel; every CTA of the grid takes a slice of it
                const int r0 = panel * panel_rows;
                const int rows = min(p.m - r0, panel_rows);
                const int per = (rows + ar.world - 1) / ar.world;
                const int s0 = min(rows, ar.rank * per);
                const int s1 = min(rows, s0 + per);
                ShardView v;
                v.partial = ar.partial;
                v.out = ar.out;
                v.mc_partial = ar.mc_partial;
                v.mc_out = ar.mc_out;
                v.world = ar.world;
                v.row0 = r0 + s0;
                v.rows = s1 - s0;
                v.n = p.n;
                v.ld_partial = ar.ld_partial;
                v.ld_out = ar.ld_out;
                reduce_shard(v, first, stride);
            }
            // The last CTA to finish its slice publishes the shard as delivered, unless a CTA gave up on its wait.
            __threadfence_system();
            ptx::named_barrier_sync(kExchangeBarrierId, kExchangeThreads);
            if (tid == 0) {
                const int add = ok ? 1 : 1 + kCounterFailed;
                const int after = atomicAdd(ar.exchange_counter + slot, add) + add;
                if ((after & (kCounterFailed - 1)) == static_cast<int>(gridDim.x)) {
                    ar.exchange_counter[slot] = 0;
                    __threadfence_system();
                    if (after < kCounterFailed) {
                        for (int r = 0; r < ar.world; ++r) {
                            st_release_sys(static_cast<int*>(ar.done.p[r]) + slot * kFlagStride + ar.rank, ar.epoch);
                        }
                    }
                }
            }
            if (!ok) {
                break; // the remaining panels would only wait for the same missing rank
            }
        }
        if (ok) {
            // the step is complete here once every owner has delivered every panel into this rank's output
            for (int i = tid; i < ar.panels * ar.world; i += kExchangeThreads) {
                const int slot = ar.slot0 + i / ar.world;
                if (!wait_epoch(done_local + slot * kFlagStride + i % ar.world, ar.epoch, p.status,
                                ST_KSPLIT_DONE_TIMEOUT, p.wait_limit)) {
                    break;
                }
            }
        }
    }

    ptx::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        for (int i = 0; i < 2000; ++i) {
            __nanosleep(1000);
        }
    }
    if constexpr (COMM == COMM_GATHER) {
        // every load of this CTA has landed: the last CTA of the launch tells every rank that this rank is done with
        // the step's rows, so the next step's pushes may overwrite them
        if (threadIdx.x == 0) {
            if (atomicAdd(ga.done_counter, 1) == static_cast<int>(gridDim.x) - 1) {
                *ga.done_counter = 0;
                __threadfence_system();
                for (int r = 0; r < ga.world; ++r) {
                    st_release_sys(static_cast<int*>(ga.flags.p[r]) + p.m_tiles + ga.rank, ga.epoch);
                }
            }
        }
    }
    // Both CTAs are past every access to the other's shared memory, barriers and tensor memory.
    ptx::cluster_arrive_relaxed();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

} // namespace pto_b200
