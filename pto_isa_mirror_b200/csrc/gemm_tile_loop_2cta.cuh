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
// Every wait is bounded as in gemm_tile_loop; the pair leaves through a cluster barrier so neither CTA's shared
// or tensor memory disappears while the other can still touch it.
#pragma once
#include "gemm_tile_loop.cuh"

namespace pto_b200 {

constexpr int kPairBlockM = 256;
constexpr int kPairBlockN = 256;

constexpr int ST_TAIL_TIMEOUT = 5;

__device__ __forceinline__ int ld_acquire_gpu(const int* ptr)
{
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

template <int KIND, int STAGES>
struct PairSmemLayout {
    static constexpr int kABytes = kBlockM * kBlockKBytes;        // this CTA's 128 rows of A
    static constexpr int kBBytes = (kPairBlockN / 2) * kBlockKBytes; // this CTA's 128 columns of B
    static constexpr int kSfaBytes = (KIND == KIND_MXF8) ? 512 : 0;
    static constexpr int kSfbBytes = (KIND == KIND_MXF8) ? 1024 : 0; // scales of all 256 columns, in both CTAs
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kAOff = 0;
    static constexpr int kBOff = STAGES * kABytes;
    static constexpr int kSfaOff = kBOff + STAGES * kBBytes;
    static constexpr int kSfbOff = kSfaOff + STAGES * kSfaBytes;
    static constexpr int kBarOff = kSfbOff + STAGES * kSfbBytes;
    static constexpr int kNumBars = 2 * STAGES + 4;
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

template <int KIND, int STAGES, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
    gemm_tile_loop_2cta(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                        const GemmParams p)
{
    using L = PairSmemLayout<KIND, STAGES>;
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
    const uint32_t cta_rank = ptx::cluster_ctarank();
    const bool leader = (cta_rank == 0);
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&acc_full_bar[a], 1);
            ptx::mbar_init(&acc_empty_bar[a], 8); // four TSTORE warps in each CTA of the pair
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
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
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    ok = bounded_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, ST_PRODUCER_TIMEOUT);
                    if (!ok) {
                        break;
                    }
                    if (leader) {
                        ptx::mbar_arrive_expect_tx(&full_bar[stage], 2u * L::kStageBytes);
                    }
                    const uint32_t full_addr = ptx::map_to_cta(ptx::smem_u32(&full_bar[stage]), 0);
                    ptx::tma_load_2d_pair(smem + L::kAOff + stage * L::kABytes, &tmap_a, full_addr, kb * kBlockKElems,
                                          row_a);
                    ptx::tma_load_2d_pair(smem + L::kBOff + stage * L::kBBytes, &tmap_b, full_addr, kb * kBlockKElems,
                                          row_b);
                    if constexpr (KIND == KIND_MXF8) {
                        // Scale atoms through tensor maps over the re-tiled workspace viewed as rows of 256 bytes
                        // (an atom is two rows): A rows of this CTA (row block 2*mi + rank), B columns of the whole
                        // tile (two atoms). The tensor form lets the bytes complete on the leader's barrier.
                        const int sfa_row = (kb * (2 * p.m_tiles) + 2 * mi + static_cast<int>(cta_rank)) * 2;
                        const int sfb_row = (kb * p.n_tiles + ni) * 4;
                        ptx::tma_load_2d_pair(smem + L::kSfaOff + stage * L::kSfaBytes, &tmap_sfa, full_addr, 0,
                                              sfa_row);
                        ptx::tma_load_2d_pair(smem + L::kSfbOff + stage * L::kSfbBytes, &tmap_sfb, full_addr, 0,
                                              sfb_row);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- TMATMUL / TMATMUL_ACC role (leader only)
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            PairUnit w;
            for (int u = pair; ok && pair_unit(u, p, w); u += num_pairs) {
                ok = bounded_wait(&acc_empty_bar[acc], acc_phase ^ 1u, abort_flag, p.status, ST_MMA_ACC_TIMEOUT);
                if (!ok) {
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kAccCols);
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    ok = bounded_wait(&full_bar[stage], phase, abort_flag, p.status, ST_MMA_FULL_TIMEOUT);
                    if (!ok) {
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_base = ptx::smem_u32(smem + L::kAOff + stage * L::kABytes);
                    const uint32_t b_base = ptx::smem_u32(smem + L::kBOff + stage * L::kBBytes);
                    if constexpr (KIND == KIND_MXF8) {
                        const uint32_t sfa_base = ptx::smem_u32(smem + L::kSfaOff + stage * L::kSfaBytes);
                        const uint32_t sfb_base = ptx::smem_u32(smem + L::kSfbOff + stage * L::kSfbBytes);
                        ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + kSfaCol,
                                                         ptx::make_smem_desc(sfa_base, 0, 128, ptx::kSwizzleNone));
                        ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + kSfbCol,
                                                         ptx::make_smem_desc(sfb_base, 0, 128, ptx::kSwizzleNone));
                        ptx::tmem_cp_32x128b_warpx4_pair(tmem_base + kSfbCol + 4u,
                                                         ptx::make_smem_desc(sfb_base + 512u, 0, 128, ptx::kSwizzleNone));
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
                            ptx::umma_mxf8_pair(d_tmem, a_desc, b_desc, idesc, tmem_base + kSfaCol, tmem_base + kSfbCol,
                                                accumulate);
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
    } else {
        // ---------------------------------------------------------------- TSTORE role (both CTAs)
        const int quarter = warp & 3;
        const int esize = (EPI == EPI_F32 || EPI == EPI_S32) ? 4 : 2;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0) && (((p.ldc * esize) & 15) == 0);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        PairUnit w;
        for (int u = pair; ok && pair_unit(u, p, w); u += num_pairs) {
            const int mi = w.mi, ni = w.ni;
            ok = bounded_wait(&acc_full_bar[acc], acc_phase, abort_flag, p.status, ST_EPILOGUE_TIMEOUT);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) {
                break;
            }
            ptx::tc_fence_after_sync();
            const int row = mi * kPairBlockM + static_cast<int>(cta_rank) * kBlockM + quarter * 32 + lane;
            float s_row = 1.0f;
            if constexpr (EPI == EPI_DEQ_BF16) {
                s_row = (row < p.m) ? __ldg(p.s_row + row) : 0.0f;
            }
            const uint32_t t_row = tmem_base + static_cast<uint32_t>(acc * kAccCols) +
                                   (static_cast<uint32_t>(quarter * 32) << 16);
            // this thread's row of the parked accumulators of a split tile
            uint32_t* ws_row = nullptr;
            int* ws_arrive = nullptr;
            if (w.role != 0) {
                ws_row = p.ws_partial + (static_cast<size_t>(w.tail_idx) * kPairBlockM +
                                         cta_rank * kBlockM + quarter * 32 + lane) * kPairBlockN;
                ws_arrive = p.ws_flags + 2 * w.tail_idx;
            }
            if (w.role == 2) {
                // second K half: wait (bounded) until every store warp of the first half has parked its rows
                bool parked = true;
                if (lane == 0) {
                    const long long t0 = clock64();
                    while (ld_acquire_gpu(ws_arrive) < kTailWarps) {
                        __nanosleep(32);
                        if (*abort_flag != 0 || clock64() - t0 > kWaitLimitCycles) {
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
            }
            // one 32-column chunk of this thread's row: park it (first K half), add the parked half (second K half),
            // then cast / scale and store
            auto finish_chunk = [&](uint32_t (&v)[32], int chunk) {
                const int col0 = ni * kPairBlockN + chunk * 32;
                if (col0 >= p.n) {
                    return;
                }
                if (w.role == 1) {
                    uint4* d4 = reinterpret_cast<uint4*>(ws_row + chunk * 32);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        d4[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    }
                    return;
                }
                if (w.role == 2) {
                    const uint4* s4 = reinterpret_cast<const uint4*>(ws_row + chunk * 32);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint4 q = __ldcg(s4 + i);
                        const uint32_t qa[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if constexpr (EPI == EPI_S32 || EPI == EPI_DEQ_BF16) {
                                v[4 * i + j] += qa[j]; // int32 accumulators: exact
                            } else {
                                v[4 * i + j] = __float_as_uint(__uint_as_float(qa[j]) + __uint_as_float(v[4 * i + j]));
                            }
                        }
                    }
                }
                store_chunk<EPI>(v, p, row, col0, vec_ok, s_row);
            };
            // Accumulator read-back, software-pipelined over 32-column chunks: the TMEM load of the next chunk is in
            // flight while the current one is converted and stored (columns past N are loaded but never stored).
            // Two chunks of registers keep the kernel near 128 registers per thread, so that a reduction CTA of the
            // K-split path still fits beside this CTA on the SM.
            {
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
                    }
                    finish_chunk(vb, g * 2 + 1);
                }
            }
            if (w.role == 1) {
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    atomicAdd(ws_arrive, 1);
                }
            } else if (w.role == 2) {
                __syncwarp();
                if (lane == 0) {
                    // the last reader to leave clears both counters for the next launch
                    if (atomicAdd(ws_arrive + 1, 1) == kTailWarps - 1) {
                        ws_arrive[0] = 0;
                        ws_arrive[1] = 0;
                    }
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (leader) {
                    ptx::mbar_arrive(&acc_empty_bar[acc]);
                } else {
                    ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&acc_empty_bar[acc]), 0));
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
        for (int i = 0; i < 2000; ++i) {
            __nanosleep(1000);
        }
    }
    // Both CTAs are past every access to the other's shared memory, barriers and tensor memory.
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

} // namespace pto_b200
