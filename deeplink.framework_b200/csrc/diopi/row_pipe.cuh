// Row pipeline of the rotary-embedding kernel (rope.cu). A CTA is a set of independent warps; every warp walks over its own
// rows (global warp index, then + total warps, ...) and owns a small ring of shared-memory slots that bulk copies
// (cp.async.bulk, global -> shared, completion counted on an mbarrier) fill ahead of the arithmetic: while a warp works on one
// row, its next row is already on its way from HBM, at no cost in registers or issue slots. There is no CTA-wide barrier
// anywhere: a warp waits on its own mbarrier, reads the row from shared memory (as often as it needs: a reduction pass and an
// output pass), and its first lane refills the slot after a __syncwarp. With a dozen such warps per SM there are a dozen
// independent load -> rotate -> store chains in flight per SM plus as many rows under way. It pays for a kernel without a
// reduction (rotary embedding inside the layer: 4.9 -> 5.6 TB/s); RMSNorm / LayerNorm / softmax measured faster as many small
// one-row CTAs (rowwise.cu), whose rows cost more instructions than a dozen warps per SM can issue in time.
//
// Per row k of a warp (slot s = k % kStages, parity (k / kStages) & 1):
//   all lanes   bounded wait on full[warp][s]
//   all lanes   passes over the slot (16-byte shared loads), results stored to global memory from registers
//   lane 0      after __syncwarp: arms full[warp][s] with the byte count and issues the bulk copy of row k + kStages
// A wait that runs out (2 s) raises the tensor-core kernels' status word; the warp then waits for its copies in flight and
// leaves. Rows must be 16-byte aligned and a multiple of 16 bytes long (the bulk copy's rules).
#pragma once

#include "device_utils.cuh"
#include "gemm_sm100.cuh"

namespace b200 {
namespace rowpipe {

constexpr int kStages = 2;
constexpr int kMaxWarps = 16;
constexpr uint32_t kRingBudget = 192 * 1024;  // shared memory of all rings of a CTA

struct Ctl {
    uint64_t full[kMaxWarps][kStages];
    uint32_t abort_flag;
};

// The rows are read once: the copies carry an evict-first L2 policy, like the streaming loads of the other kernels, so that
// they do not push lines out of L2 that somebody will read again (or dirty lines that are still on their way to HBM).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     sm100::smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(sm100::smem_u32(bar)), "l"(policy)
                 : "memory");
}

__device__ __forceinline__ uint4 lds16(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// One per warp. `ring` is the warp's own kStages * row_bytes bytes of shared memory.
struct WarpRing {
    uint64_t* full;
    unsigned char* ring;
    const char* src;
    uint32_t row_bytes;
    int64_t first, stride, rows;   // this warp's rows: first, first + stride, ... < rows
    uint32_t* abort_flag;

    __device__ __forceinline__ void issue(int k) {
        const int64_t r = first + static_cast<int64_t>(k) * stride;
        if (r < rows) {
            const int s = k % kStages;
            sm100::mbar_arrive_expect_tx(&full[s], row_bytes);
            bulk_load(ring + static_cast<size_t>(s) * row_bytes, src + r * static_cast<int64_t>(row_bytes), row_bytes, &full[s]);
        }
    }
    // The CTA's barriers are initialised (by thread 0, before a __syncthreads) when this runs.
    __device__ __forceinline__ void start() {
        if ((threadIdx.x & 31) == 0) {
            for (int k = 0; k < kStages; ++k) issue(k);
        }
    }
    // Row k has arrived (bounded wait); nullptr when the wait ran out on any lane of the warp.
    __device__ __forceinline__ const unsigned char* acquire(int k) {
        const int s = k % kStages;
        const bool ok = sm100::mbar_wait(&full[s], static_cast<uint32_t>((k / kStages) & 1), abort_flag);
        if (!__all_sync(0xffffffffu, ok ? 1 : 0)) return nullptr;
        return ring + static_cast<size_t>(s) * row_bytes;
    }
    // Every lane has finished reading row k's slot: refill it with row k + kStages.
    __device__ __forceinline__ void release(int k) {
        __syncwarp();
        if ((threadIdx.x & 31) == 0) issue(k + kStages);
    }
};

__device__ __forceinline__ void init_ctl(Ctl* ctl, int warps) {
    if (threadIdx.x == 0) {
        for (int w = 0; w < warps; ++w) {
            for (int s = 0; s < kStages; ++s) sm100::mbar_init(&ctl->full[w][s], 1);
        }
        ctl->abort_flag = 0;
        sm100::fence_barrier_init();
    }
    __syncthreads();
}

__device__ __forceinline__ WarpRing make_ring(Ctl* ctl, unsigned char* smem, const void* src, uint32_t row_bytes, int64_t rows) {
    const int warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    WarpRing r;
    r.full = ctl->full[warp];
    r.ring = smem + static_cast<size_t>(warp) * kStages * row_bytes;
    r.src = static_cast<const char*>(src);
    r.row_bytes = row_bytes;
    r.first = static_cast<int64_t>(blockIdx.x) * warps + warp;
    r.stride = static_cast<int64_t>(gridDim.x) * warps;
    r.rows = rows;
    r.abort_flag = &ctl->abort_flag;
    return r;
}

// A wait ran out: record it and give the copies in flight time to land before the CTA's shared memory is handed on.
__device__ __forceinline__ void leave_after_timeout(uint32_t* status) {
    if ((threadIdx.x & 31) == 0 && status != nullptr) atomicExch(status, 1u);
    const unsigned long long t0 = sm100::globaltimer_ns();
    while (sm100::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
}

// Warps per CTA for rows of row_bytes (plus `extra` bytes of shared memory for parameters): as many rings as fit the budget.
inline int warps_for(int64_t row_bytes, int64_t extra) {
    int64_t w = (static_cast<int64_t>(kRingBudget) - extra) / (kStages * row_bytes);
    if (w > kMaxWarps) w = kMaxWarps;
    return static_cast<int>(w);
}

}  // namespace rowpipe
}  // namespace b200
