// Cross-GPU reduction of K-split partials over peer memory (NVLink / NVSwitch), one process per GPU.
//
// The reference reduces its per-rank GEMM outputs tile by tile through symmetric "window" buffers: every rank adds
// its tile into the owner's window, counters tell the owner when a tile is complete, and the owner broadcasts the
// finished tile to every rank (kernels/manual/a2a3/gemm_ar/comm_kernel.cpp:165-210 reduce-scatter, :377-400
// all-gather, :111-123 TNOTIFY counters, :528-590 TTEST/TWAIT). The B200 form keeps that structure per row panel:
//
//   ksplit_signal_kernel   after a rank's GEMM for a panel: publish "my partial of panel p is written" to all ranks
//   ksplit_reduce_kernel   the owner of a row shard waits for every rank's flag, LOADS the shard of every rank's
//                          fp32 partial over peer pointers (plain loads, no multicast), sums in rank order, casts to
//                          bf16 (the TSTORE cast) and STORES the result into every rank's output, then publishes
//                          "my shard of panel p is delivered"
//   ksplit_wait_kernel     end of a step: wait until every owner has delivered every panel into this rank's output
//
// Flags are monotonically increasing epochs (one per step), so nothing is ever reset. Every spin is bounded: on
// expiry the kernel records a code in the library's status word and returns; nothing traps.
#pragma once
#include <cuda_bf16.h>

#include <cstdint>

namespace pto_b200 {

constexpr int kMaxRanks = 8;
constexpr int kFlagStride = kMaxRanks; // flags[slot * kFlagStride + rank]
constexpr long long kPeerWaitLimitCycles = 4000000000ll; // default limit of one wait, about two seconds

enum KsplitStatus : int { ST_KSPLIT_READY_TIMEOUT = 16, ST_KSPLIT_DONE_TIMEOUT = 17 };

struct PeerPointers {
    void* p[kMaxRanks];
};

__device__ __forceinline__ int ld_acquire_sys(const int* ptr)
{
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

// 16-byte load that is coherent at system scope (served by the owning GPU's L2, never by a stale local L1 line)
// and free for the compiler to schedule: many of these are kept in flight per thread to cover NVLink latency.
__device__ __forceinline__ float4 ld_peer_f4(const float* ptr)
{
    float4 v;
    asm("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(ptr));
    return v;
}

// In-switch reduction (NVLS): one load through the multicast address returns the fp32 sum of the same 16 bytes of
// every rank's buffer, added inside the NVSwitch; one store through it writes 8 bytes into every rank's buffer.
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc_ptr)
{
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(mc_ptr)
                 : "memory");
    return v;
}

__device__ __forceinline__ void multimem_st_b64(void* mc_ptr, uint64_t v)
{
    asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(mc_ptr), "l"(v) : "memory");
}

__device__ __forceinline__ void st_release_sys(int* ptr, int v)
{
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}

// Spin until *flag >= epoch. false after `limit` cycles (status word set). (A pause that doubles up to a microsecond
// between two looks, instead of a constant 64 ns, changed no timing of the fused kernels on two GPUs.)
__device__ __forceinline__ bool wait_epoch(const int* flag, int epoch, int* status, int code, long long limit)
{
    if (ld_acquire_sys(flag) >= epoch) {
        return true;
    }
    const long long t0 = clock64();
    while (ld_acquire_sys(flag) < epoch) {
        __nanosleep(64);
        if (clock64() - t0 > limit) {
            atomicCAS(status, 0, code);
            return false;
        }
    }
    return true;
}

// Launched on the GEMM's stream right after the GEMM of one panel: everything this rank wrote before is made
// visible system-wide, then ready[slot][rank] = epoch is stored into every rank's flag array.
__global__ void ksplit_signal_kernel(PeerPointers flag_arrays, int world, int rank, int slot, int epoch)
{
    __threadfence_system();
    if (threadIdx.x < world) {
        int* flags = static_cast<int*>(flag_arrays.p[threadIdx.x]);
        st_release_sys(flags + slot * kFlagStride + rank, epoch);
    }
}

// One row shard of the K-split partials, as seen from the rank that owns it.
struct ShardView {
    PeerPointers partial;    // every rank's fp32 partial buffer [m, ld_partial] (peer pointers, own rank included)
    PeerPointers out;        // every rank's bf16 output [m, ld_out]
    const float* mc_partial; // multicast address of the partial buffers (NVLS), or null: sum with plain peer loads
    void* mc_out;            // multicast address of the output buffers, or null: one plain store per rank
    int world;
    long long row0;          // first row of the shard
    int rows, n;             // shard rows, columns (n % 4 == 0)
    long long ld_partial, ld_out;
};

// Sum the shard over the ranks, cast to bf16 (round to nearest even, the TSTORE cast) and deliver it to every rank.
// The caller's threads share the work: thread `first` of `stride` takes the 16-byte items first, first + stride, ...
__device__ __forceinline__ void reduce_shard(const ShardView& a, long long first, long long stride)
{
    const int n4 = a.n / 4;
    const long long total = static_cast<long long>(a.rows) * n4;
    if (a.mc_partial != nullptr) {
        // NVLS path: the switch adds the ranks' values (its own fixed order) and one store reaches every rank.
        // Four independent loads per thread keep enough requests in flight to cover the switch round trip.
        constexpr int kUnroll = 4;
        for (long long i0 = first; i0 < total; i0 += stride * kUnroll) {
            float4 acc[kUnroll];
            long long off[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const long long i = i0 + u * stride;
                off[u] = -1;
                if (i < total) {
                    const long long row = a.row0 + i / n4;
                    const int c = static_cast<int>(i % n4) * 4;
                    acc[u] = multimem_ld_reduce_f4(a.mc_partial + row * a.ld_partial + c);
                    off[u] = row * a.ld_out + c;
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                if (off[u] >= 0) {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[u].x, acc[u].y);
                    const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[u].z, acc[u].w);
                    const uint64_t packed = static_cast<uint64_t>(*reinterpret_cast<const uint32_t*>(&lo)) |
                                            (static_cast<uint64_t>(*reinterpret_cast<const uint32_t*>(&hi)) << 32);
                    multimem_st_b64(static_cast<__nv_bfloat16*>(a.mc_out) + off[u], packed);
                }
            }
        }
        return;
    }
    for (long long i = first; i < total; i += stride) {
        const long long row = a.row0 + i / n4;
        const int c = static_cast<int>(i % n4) * 4;
        const long long src_off = row * a.ld_partial + c;
        // all loads first (one per rank in flight), then a fixed summation order (rank 0, 1, ...): every
        // element is reduced once, by its owner, so all ranks receive identical bits
        float4 v[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            if (r < a.world) {
                v[r] = ld_peer_f4(static_cast<const float*>(a.partial.p[r]) + src_off);
            }
        }
        float4 acc = v[0];
#pragma unroll
        for (int r = 1; r < kMaxRanks; ++r) {
            if (r < a.world) {
                acc.x += v[r].x;
                acc.y += v[r].y;
                acc.z += v[r].z;
                acc.w += v[r].w;
            }
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        const long long dst_off = row * a.ld_out + c;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
            if (r < a.world) {
                *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.out.p[r]) + dst_off) = packed;
            }
        }
    }
}

// The last block to arrive at a per-slot counter learns whether any block before it failed: a block that gave up adds
// kCounterFailed besides its arrival, so one wrap-free int carries both the arrivals and the failures of a slot.
constexpr int kCounterFailed = 1 << 16;

struct KsplitReduceArgs {
    ShardView shard;
    PeerPointers done;    // every rank's done-flag array
    const int* ready;     // this rank's ready-flag array
    int* cta_counter;     // local scratch: one int per slot, zero between uses
    int* status;
    long long wait_limit; // cycles one flag wait may take
    int rank;
    int slot, epoch;
};

constexpr int kReduceThreads = 512; // 512 x 64 registers: fits beside a resident GEMM CTA

__global__ void __launch_bounds__(kReduceThreads) ksplit_reduce_kernel(const KsplitReduceArgs a)
{
    __shared__ int ok_flag;
    if (threadIdx.x == 0) {
        ok_flag = 1;
    }
    __syncthreads();
    if (threadIdx.x < a.shard.world) {
        if (!wait_epoch(a.ready + a.slot * kFlagStride + threadIdx.x, a.epoch, a.status, ST_KSPLIT_READY_TIMEOUT,
                        a.wait_limit)) {
            ok_flag = 0;
        }
    }
    __syncthreads();
    if (ok_flag != 0) {
        reduce_shard(a.shard, blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x,
                     static_cast<long long>(gridDim.x) * blockDim.x);
    }
    // The last block out publishes the shard as delivered, unless some block of this launch gave up on its wait and
    // skipped its rows: then nothing is published and the peers run into their own bounded wait instead of reading a
    // partly reduced shard.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int before = atomicAdd(a.cta_counter + a.slot, ok_flag != 0 ? 1 : 1 + kCounterFailed);
        const int after = before + (ok_flag != 0 ? 1 : 1 + kCounterFailed);
        if ((after & (kCounterFailed - 1)) == static_cast<int>(gridDim.x)) {
            a.cta_counter[a.slot] = 0;
            __threadfence_system();
            if (after < kCounterFailed) {
                for (int r = 0; r < a.shard.world; ++r) {
                    st_release_sys(static_cast<int*>(a.done.p[r]) + a.slot * kFlagStride + a.rank, a.epoch);
                }
            }
        }
    }
}

// Wait until done[slot][r] >= epoch for slots [slot0, slot0 + slots) and every rank r.
__global__ void ksplit_wait_kernel(const int* done, int world, int slot0, int slots, int epoch, int* status,
                                   long long wait_limit)
{
    for (int i = threadIdx.x; i < slots * world; i += blockDim.x) {
        const int slot = slot0 + i / world;
        const int r = i % world;
        wait_epoch(done + slot * kFlagStride + r, epoch, status, ST_KSPLIT_DONE_TIMEOUT, wait_limit);
    }
}

} // namespace pto_b200
