// Dense contraction on CTA pairs (tcgen05 cta_group::2): C[b] = alpha * A[b] * B[b] + beta * bias, for large products.
//
// Two CTAs on neighbouring SMs (a cluster of 2) own one 256 x 256 output tile. Each CTA loads only its half of the
// operands per K step - A rows [r*128, r*128+128) and B rows (N) [r*128, r*128+128), 32 KiB instead of the 48 KiB a
// single CTA needs for a 128 x 256 tile - so the same shared memory holds 6 stages instead of 4 (more latency cover)
// and each operand byte staged feeds twice the math. One thread of the leader CTA (cluster rank 0) issues
// tcgen05.mma.cta_group::2 with M = 256: the hardware reads A and B from both CTAs' shared memory at the same offsets
// and accumulates 128 rows x 256 fp32 columns into each CTA's tensor memory. Each CTA runs its own epilogue on its rows.
//
// Hand-over (all waits bounded, see gemm_sm100.cuh):
//   full[s]   (leader's)  both CTAs' TMA loads count their bytes on the leader's barrier; the leader arms it with the
//                         pair's total byte count. Plain per-CTA loads: no cluster multicast anywhere.
//   empty[s]  (each CTA)  the leader commits the MMAs that read stage s to its own and to the partner's barrier
//   acc_full  (each CTA)  the leader commits the tile's last MMA to both CTAs' barriers
//   acc_empty (leader's)  the 8 epilogue warps of the pair arrive (the partner's remotely) when an accumulator is drained
//
// PUSH variant (row-parallel linear of a tensor-parallel group, C = this rank's partial sum): instead of storing the tile
// into a local C, each epilogue warp writes its 32 x 256 piece into the staging block of the rank that owns those rows -
// plain 16-byte stores to peer memory mapped over NVLink, 128 contiguous bytes per row segment - and then raises the
// piece's ready flag there (fence.sys + st.release.sys). The transfer of one tile overlaps the MMAs of the next ones; the
// kernel never waits for a peer except for the (normally long satisfied) permission to overwrite a staging slot. Each
// rank starts its tile order at the rows of the next rank, so that at any moment the ranks push to different owners.
#include <cuda.h>

#include <cstdlib>

#include "device_utils.cuh"
#include "dipu_b200/peer_space.h"
#include "gemm.h"
#include "gemm_sm100.cuh"

namespace b200 {
namespace {

using namespace sm100;

constexpr int BM = 128;      // rows per CTA
constexpr int BN = 256;      // tile columns (128 of them staged per CTA)
constexpr int BNH = BN / 2;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;      // 4 epilogue warps; the EPI = 8 instantiation runs 320
constexpr int kGroupM = 8;   // in units of 256-row pair blocks
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BNH * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStoreBytes = 4 * 2 * 32 * 128;
constexpr int kStages = 6;
constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 512;
static_assert(kSmemBytes <= 232448, "shared memory budget");

struct PairParams {
    int M, N, K, batch;
    int m_pairs, n_blocks, k_blocks;
    int group_m;  // row-pair blocks per tile group (tile order: all tiles of a group before the next group)
    int m_rot;    // the tile order starts at row-pair block m_rot (and wraps around)
    int64_t ldc, stride_cb;
    void* C;
    const void* bias;
    int64_t bias_sb, bias_sr, bias_sc;
    float alpha, beta;
    uint32_t idesc;
    int b_mn_major;
    int bias_vec_ok;
    uint32_t* status;
};

struct PushParams {
    b200PeerSpace space;
    int slot;
    uint32_t epoch;       // this call's number: written into the ready flags
    uint32_t prev_epoch;  // number of the last call that used this slot (0: none); its reduction must be over before we write
    int rows_per_rank;    // M / nranks, a multiple of 128
    unsigned long long wait_ns;  // limit of the wait for the permission to overwrite a peer's staging slot
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_peer16(void* p, const uint4& v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Bounded wait until *flag >= target (flags only grow); raises the CTA's abort flag on time-out.
__device__ __forceinline__ bool flag_wait_ge(const uint32_t* flag, uint32_t target, volatile uint32_t* abort_flag, unsigned long long limit_ns) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(flag) - target) >= 0) return true;
    const unsigned long long t0 = globaltimer_ns();
    while (true) {
        if (static_cast<int32_t>(ld_acquire_sys_u32(flag) - target) >= 0) return true;
        if (*abort_flag != 0) return false;
        if (globaltimer_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            return false;
        }
    }
}

__device__ __forceinline__ void pair_tile_coords(int tile, const PairParams& p, int* b, int* mp, int* nb) {
    const int per_batch = p.m_pairs * p.n_blocks;
    *b = tile / per_batch;
    const int t = tile - *b * per_batch;
    const int group_sz = p.group_m * p.n_blocks;
    const int g = t / group_sz;
    const int first = g * p.group_m;
    const int rows = min(p.m_pairs - first, p.group_m);
    const int r = t - g * group_sz;
    *mp = first + r % rows + p.m_rot;
    if (*mp >= p.m_pairs) *mp -= p.m_pairs;
    *nb = r / rows;
}

// EPI = epilogue warps per CTA: 4 (one per 32-lane quarter of tensor memory) or 8 (two per quarter, each draining half of
// the tile's columns). A 256 x 256 tile takes the tensor cores 0.27 us per 64-deep K block and one warp per quarter about
// 3 us to drain: with K loops of up to 8 blocks (the row-parallel shards of an 8-way tensor-parallel layer, K = 512) the
// drain, not the product, paces the kernel unless it is spread over eight warps.
template <typename TOut, bool PUSH, int EPI>
__global__ void __launch_bounds__(64 + 32 * EPI, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                    const PairParams p, const __grid_constant__ PushParams q) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kStages * kABytes;
    uint8_t* smem_c = smem + kStages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_c + kStoreBytes);
    uint64_t* full_bar = bars;                    // [kStages] used in the leader only
    uint64_t* empty_bar = bars + kStages;         // [kStages] one set per CTA
    uint64_t* acc_full = bars + 2 * kStages;      // [2] one set per CTA
    uint64_t* acc_empty = bars + 2 * kStages + 2; // [2] used in the leader only
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;
    const int total_tiles = p.batch * p.m_pairs * p.n_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);   // the leader's arrive.expect_tx; bytes from both CTAs
            mbar_init(&empty_bar[s], 1);  // one commit from the leader
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 2 * EPI);  // the epilogue warps of both CTAs of the pair
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        prefetch_tensormap(&map_c);
    }
    __syncthreads();
    // barriers of both CTAs must exist before either CTA signals the other's
    cluster_sync_all();
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // shared::cluster addresses of the leader's barriers and of the partner's copies of the per-CTA ones
    const uint32_t leader_full0 = map_to_cta(smem_u32(&full_bar[0]), 0);
    const uint32_t leader_acc_empty0 = map_to_cta(smem_u32(&acc_empty[0]), 0);

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs: each loads its own halves) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters) {
                int b, mp, nb;
                pair_tile_coords(tile, p, &b, &mp, &nb);
                const int row0 = mp * (2 * BM) + static_cast<int>(rank) * BM;
                const int col0 = nb * BN + static_cast<int>(rank) * BNH;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * kStageBytes);
                    const uint32_t bar = leader_full0 + stage * 8;
                    tma_load_3d_pair(smem_a + stage * kABytes, &map_a, bar, kb * BK, row0, b);
                    if (!p.b_mn_major) {
                        tma_load_3d_pair(smem_b + stage * kBBytes, &map_b, bar, kb * BK, col0, b);
                    } else {
#pragma unroll
                        for (int g = 0; g < BNH / 64; ++g) {
                            tma_load_3d_pair(smem_b + stage * kBBytes + g * (64 * BK * 2), &map_b, bar, col0 + g * 64, kb * BK, b);
                        }
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t peer_empty0 = map_to_cta(smem_u32(&empty_bar[0]), 1);
            const uint32_t peer_acc_full0 = map_to_cta(smem_u32(&acc_full[0]), 1);
            const uint32_t own_empty0 = map_to_cta(smem_u32(&empty_bar[0]), 0);
            const uint32_t own_acc_full0 = map_to_cta(smem_u32(&acc_full[0]), 0);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters, ++local) {
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1u;
                if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + stage * kABytes);
                    const uint32_t b_addr = smem_u32(smem_b + stage * kBBytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t da = make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
                        const uint64_t db = p.b_mn_major ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                                         : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
                        umma_f16_ss_pair(d_tmem, da, db, p.idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    // the stage is free in both CTAs once these MMAs have read it
                    umma_commit_pair(own_empty0 + stage * 8);
                    umma_commit_pair(peer_empty0 + stage * 8);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) {
                    umma_commit_pair(own_acc_full0 + acc * 8);
                    umma_commit_pair(peer_acc_full0 + acc * 8);
                }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs, each CTA on its own 128 rows) ----------------
        const int quarter = warp & 3;
        int local = 0;
        uint32_t store_seq = 0;
        uint32_t checked = 0;  // PUSH: owners whose staging slot is known to be free for this call
        uint32_t* pending_flag = nullptr;  // PUSH: ready flag of the piece pushed last, not raised yet
        bool ok = true;
        constexpr int PIECE_COLS = 128 / static_cast<int>(sizeof(TOut));
        constexpr int LOADS = PIECE_COLS / 32;
        // staging for the TMA store: two 4 KiB buffers per warp with four warps, one with eight (the same 32 KiB)
        uint8_t* stage_base = smem_c + (warp - 2) * ((EPI == 4 ? 2 : 1) * 32 * 128);
        constexpr int kPieces = BN / PIECE_COLS;
        const int c_begin = EPI == 4 ? 0 : ((warp - 2) >> 2) * (kPieces / 2);
        const int c_end = EPI == 4 ? kPieces : c_begin + kPieces / 2;
        for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters, ++local) {
            int b, mp, nb;
            pair_tile_coords(tile, p, &b, &mp, &nb);
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1u;
            if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            if constexpr (PUSH) {
                // st.release.sys orders the whole warp's stores of the previous tile (they were followed by __syncwarp) before
                // the flag, at system scope
                if (pending_flag != nullptr && lane == 0) st_release_sys_u32(pending_flag, q.epoch);
                pending_flag = nullptr;
            }
            const int row_base = mp * (2 * BM) + static_cast<int>(rank) * BM + quarter * 32;
            const int row = row_base + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
            int owner = 0, local_row0 = 0;
            uint8_t* push_dst = nullptr;  // PUSH: where this warp's 32 rows start in the owner's staging slot (column 0)
            if constexpr (PUSH) {
                owner = row_base / q.rows_per_rank;
                if (((checked >> owner) & 1u) == 0) {
                    int fine = 1;
                    if (lane == 0) {
                        fine = flag_wait_ge(q.space.flags[q.space.rank] + b200_peer_sfree_off(&q.space, q.slot, owner), q.prev_epoch, abort_flag, q.wait_ns) ? 1 : 0;
                    }
                    fine = __shfl_sync(0xffffffffu, fine, 0);
                    if (!fine) { ok = false; break; }
                    checked |= 1u << owner;
                }
                local_row0 = row_base - owner * q.rows_per_rank;
                push_dst = static_cast<uint8_t*>(q.space.stage[owner]) + static_cast<size_t>(q.slot) * q.space.slot_bytes +
                           (static_cast<size_t>(q.space.rank) * q.rows_per_rank + local_row0) * p.N * sizeof(TOut);
            }
            if (row_base < p.M) {
#pragma unroll 1
                for (int c = c_begin; c < c_end; ++c) {
                    const int col0 = nb * BN + c * PIECE_COLS;
                    if (col0 >= p.N) break;  // warp-uniform
                    uint8_t* buf = stage_base + (EPI == 4 ? (store_seq & 1) * (32 * 128) : 0);
                    if constexpr (!PUSH) {
                        if (lane == 0) {
                            if constexpr (EPI == 4) tma_store_wait_read<1>();
                            else tma_store_wait_read<0>();
                        }
                        __syncwarp();
                    }
                    uint32_t r[LOADS][32];
#pragma unroll
                    for (int l = 0; l < LOADS; ++l) tmem_ld_32x32(t_row + c * PIECE_COLS + l * 32, r[l]);
                    tmem_ld_wait();
#pragma unroll
                    for (int l = 0; l < LOADS; ++l) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[l][j]) * p.alpha;
                        if (p.bias != nullptr && row < p.M) {
                            const TOut* brow = static_cast<const TOut*>(p.bias) + static_cast<int64_t>(b) * p.bias_sb + static_cast<int64_t>(row) * p.bias_sr;
                            const int cbase = col0 + l * 32;
                            if (p.bias_vec_ok && cbase + 32 <= p.N) {
                                constexpr int BV = 16 / static_cast<int>(sizeof(TOut));
#pragma unroll
                                for (int j = 0; j < 32; j += BV) {
                                    const Vec16<TOut> bv = ld16(brow + cbase + j);
#pragma unroll
                                    for (int e = 0; e < BV; ++e) v[j + e] += p.beta * to_f32(bv.v[e]);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    const int col = cbase + j;
                                    if (col < p.N) v[j] += p.beta * to_f32(brow[static_cast<int64_t>(col) * p.bias_sc]);
                                }
                            }
                        }
                        constexpr int V = 16 / static_cast<int>(sizeof(TOut));
#pragma unroll
                        for (int j = 0; j < 32; j += V) {
                            Vec16<TOut> o;
#pragma unroll
                            for (int e = 0; e < V; ++e) o.v[e] = from_f32<TOut>(v[j + e]);
                            const int chunk = (l * 32 + j) / V;
                            *reinterpret_cast<uint4*>(buf + lane * 128 + ((chunk ^ (lane & 7)) * 16)) = *reinterpret_cast<const uint4*>(&o);
                        }
                    }
                    if constexpr (PUSH) {
                        // read the piece back row-wise: 8 lanes cover the 128 bytes of a row segment, 4 rows per instruction
                        __syncwarp();
                        const int sub = lane & 7, rsel = lane >> 3;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = i * 4 + rsel;
                            const uint4 w = *reinterpret_cast<const uint4*>(buf + rr * 128 + ((sub ^ (rr & 7)) * 16));
                            st_peer16(push_dst + (static_cast<size_t>(rr) * p.N + col0) * sizeof(TOut) + sub * 16, w);
                        }
                        __syncwarp();
                    } else {
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(&map_c, buf, col0, row_base, b);
                            tma_store_commit();
                        }
                    }
                    ++store_seq;
                }
            }
            if constexpr (PUSH) {
                // The piece is on its way. Its flag is raised when the next tile's accumulator is ready (or after the
                // last tile): by then the stores have long been acknowledged and the release costs next to nothing.
                const uint32_t unit = static_cast<uint32_t>(local_row0 / B200_PEER_PIECE_ROWS) * p.n_blocks + nb;
                pending_flag = q.space.flags[owner] + b200_peer_ready_off(&q.space, q.slot, q.space.rank, unit);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + acc * 8);
        }
        if constexpr (PUSH) {
            if (ok && pending_flag != nullptr && lane == 0) st_release_sys_u32(pending_flag, q.epoch);
        }
        if (lane == 0) tma_store_wait_all<0>();
    }

    // ---------------- teardown: every thread of both CTAs comes through here, also after a timed-out wait ----------------
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();  // the partner's shared / tensor memory is in use by the leader's MMAs until both are done
    tc_fence_after();
    if (*abort_flag != 0) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0) atomicExch(p.status, 1u);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

template <typename TOut, bool PUSH, int EPI = 4>
cudaError_t launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const PairParams& p, const PushParams& q, int grid,
                        cudaStream_t stream) {
    if (cudaError_t e = tc_ensure_smem_attr(reinterpret_cast<const void*>(gemm_tc_pair_kernel<TOut, PUSH, EPI>), kSmemBytes); e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(64 + 32 * EPI);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<TOut, PUSH, EPI>, ma, mb, mc, p, q);
}

// Tensor maps of A and B and the tile geometry: shared by the storing and the pushing launch.
diopiError_t pair_setup(const GemmProblem& g, CUtensorMap* ma, CUtensorMap* mb, PairParams* pp) {
    const bool is_bf16 = g.ab_dtype == diopi_dtype_bfloat16;
    const bool b_mn = g.b_sk != 1;
    B200_CHECK(tc_encode_map(ma, g.ab_dtype, g.A, g.K, g.M, g.batch, g.a_sm, g.batch > 1 ? g.a_sb : g.a_sm * g.M, BM),
               "gemm: cuTensorMapEncodeTiled failed for A");
    if (!b_mn) {
        B200_CHECK(tc_encode_map(mb, g.ab_dtype, g.B, g.K, g.N, g.batch, g.b_sn, g.batch > 1 ? g.b_sb : g.b_sn * g.N, BNH),
                   "gemm: cuTensorMapEncodeTiled failed for B (K-major)");
    } else {
        B200_CHECK(tc_encode_map(mb, g.ab_dtype, g.B, g.N, g.K, g.batch, g.b_sk, g.batch > 1 ? g.b_sb : g.b_sk * g.K, BK),
                   "gemm: cuTensorMapEncodeTiled failed for B (MN-major)");
    }
    PairParams& p = *pp;
    p.M = static_cast<int>(g.M); p.N = static_cast<int>(g.N); p.K = static_cast<int>(g.K); p.batch = static_cast<int>(g.batch);
    p.m_pairs = static_cast<int>((g.M + 2 * BM - 1) / (2 * BM));
    p.n_blocks = static_cast<int>((g.N + BN - 1) / BN);
    // read once: the environment is not consulted on the launch path
    static const int group_m_env = [] {
        const char* e = std::getenv("B200_GEMM_GROUP_M");
        const int v = e != nullptr ? std::atoi(e) : 0;
        return (v >= 1 && v <= 64) ? v : 0;
    }();
    p.group_m = group_m_env != 0 ? group_m_env : kGroupM;
    p.m_rot = 0;
    p.k_blocks = static_cast<int>((g.K + BK - 1) / BK);
    p.ldc = g.c_sm; p.stride_cb = g.c_sb; p.C = g.C;
    p.bias = g.bias; p.bias_sb = g.bias_sb; p.bias_sr = g.bias_sm; p.bias_sc = g.bias_sn;
    p.alpha = g.alpha; p.beta = g.beta;
    p.idesc = make_idesc_f16(is_bf16 ? 1 : 0, b_mn, 2 * BM, BN);
    p.b_mn_major = b_mn ? 1 : 0;
    const int64_t c_es = dtype_size(g.c_dtype);
    p.bias_vec_ok = (g.bias != nullptr && g.bias_sn == 1 && (reinterpret_cast<uintptr_t>(g.bias) & 15u) == 0 && (g.bias_sm * c_es) % 16 == 0 &&
                     (g.bias_sb * c_es) % 16 == 0) ? 1 : 0;
    p.status = g.status_override != nullptr ? g.status_override : tc_status_word();
    B200_CHECK(p.status != nullptr, "gemm: could not allocate the kernel status word");
    return diopiSuccess;
}

unsigned long long g_push_wait_ns = kWaitLimitNs;

int pair_grid(const PairParams& p) {
    const int64_t total = static_cast<int64_t>(p.batch) * p.m_pairs * p.n_blocks;
    int64_t clusters = sm_count() / 2;
    if (clusters > total) clusters = total;
    return static_cast<int>(clusters * 2);
}

}  // namespace

// Large products with a TMA-storable output: at least two 256-row blocks and enough 256 x 256 tiles to fill the SM pairs.
bool gemm_tc2_applies(const GemmProblem& g) {
    static const bool disabled = std::getenv("B200_GEMM_NO_PAIR") != nullptr;
    if (disabled) return false;
    if (g.M < 256 || g.N < 256 || g.K < 256) return false;
    const int64_t c_es = dtype_size(g.c_dtype);
    const bool c_ok = (reinterpret_cast<uintptr_t>(g.C) & 15u) == 0 && (g.c_sm * c_es) % 16 == 0 && (g.batch == 1 || (g.c_sb * c_es) % 16 == 0);
    if (!c_ok) return false;
    const int64_t tiles = g.batch * ((g.M + 255) / 256) * ((g.N + 255) / 256);
    return tiles >= sm_count() / 2 && tiles <= 0x3fffffffLL;
}

diopiError_t gemm_tc2_launch(const GemmProblem& g, cudaStream_t stream) {
    CUtensorMap ma, mb, mc;
    PairParams p;
    if (diopiError_t err = pair_setup(g, &ma, &mb, &p); err != diopiSuccess) return err;
    B200_CHECK(tc_encode_map(&mc, g.c_dtype, g.C, g.N, g.M, g.batch, g.c_sm, g.batch > 1 ? g.c_sb : g.c_sm * g.M, 32),
               "gemm: cuTensorMapEncodeTiled failed for C");
    PushParams q = {};
    const int grid = pair_grid(p);
    cudaError_t e;
    // short K loops: eight epilogue warps, so that draining a tile does not take longer than computing the next one
    const bool wide_epilogue = p.k_blocks <= 8;
    if (g.c_dtype == diopi_dtype_bfloat16) e = wide_epilogue ? launch_pair<bf16, false, 8>(ma, mb, mc, p, q, grid, stream) : launch_pair<bf16, false>(ma, mb, mc, p, q, grid, stream);
    else if (g.c_dtype == diopi_dtype_float16) e = wide_epilogue ? launch_pair<fp16, false, 8>(ma, mb, mc, p, q, grid, stream) : launch_pair<fp16, false>(ma, mb, mc, p, q, grid, stream);
    else e = wide_epilogue ? launch_pair<float, false, 8>(ma, mb, mc, p, q, grid, stream) : launch_pair<float, false>(ma, mb, mc, p, q, grid, stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        B200_FAIL("gemm: tcgen05 pair kernel launch failed: %s", cudaGetErrorString(e));
    }
    return diopiSuccess;
}

void gemm_tc2_set_push_wait_limit_ns(unsigned long long ns) { g_push_wait_ns = ns == 0 ? kWaitLimitNs : ns; }

// This rank's partial product, pushed tile by tile into the staging slots of the ranks that own the rows. g.C is not used.
diopiError_t gemm_tc2_push_launch(const GemmProblem& g, const b200PeerSpace& space, int slot, uint32_t epoch, uint32_t prev_epoch,
                                  cudaStream_t stream) {
    const int n = space.nranks;
    B200_CHECK(n >= 1 && n <= B200_PEER_MAX_RANKS && space.rank >= 0 && space.rank < n, "mm push: bad peer space (rank %d of %d)", space.rank, n);
    B200_CHECK(slot >= 0 && slot < space.slots, "mm push: slot %d outside [0, %d)", slot, space.slots);
    B200_CHECK(g.batch == 1 && g.bias == nullptr && g.c_dtype == g.ab_dtype, "mm push: one plain product with the operands' dtype as result");
    B200_CHECK(g.M % (2 * BM) == 0 && g.M % (static_cast<int64_t>(BM) * n) == 0 && g.N % BN == 0 && g.K >= BK,
               "mm push: rows must be a multiple of %d x ranks and columns of %d (got %lld x %lld, %d ranks)", BM, BN, (long long)g.M, (long long)g.N, n);
    const int64_t es = dtype_size(g.ab_dtype);
    B200_CHECK(static_cast<uint64_t>(g.M * g.N * es) <= space.slot_bytes, "mm push: result of %lld bytes exceeds the slot size %llu",
               (long long)(g.M * g.N * es), (unsigned long long)space.slot_bytes);
    const int64_t units = (g.M / n / B200_PEER_PIECE_ROWS) * (g.N / B200_PEER_PIECE_COLS);
    B200_CHECK(units <= static_cast<int64_t>(space.max_units), "mm push: %lld pieces per rank exceed the space's %u", (long long)units, space.max_units);
    CUtensorMap ma, mb;
    PairParams p;
    if (diopiError_t err = pair_setup(g, &ma, &mb, &p); err != diopiSuccess) return err;
    // each rank starts at the rows of the next rank and ends with its own
    const int64_t start_row = (static_cast<int64_t>(space.rank + 1) % n) * (g.M / n);
    p.m_rot = static_cast<int>(start_row / (2 * BM));
    PushParams q;
    q.space = space;
    q.slot = slot;
    q.epoch = epoch;
    q.prev_epoch = prev_epoch;
    q.rows_per_rank = static_cast<int>(g.M / n);
    q.wait_ns = g_push_wait_ns;
    const int grid = pair_grid(p);
    cudaError_t e = g.ab_dtype == diopi_dtype_bfloat16 ? launch_pair<bf16, true>(ma, mb, ma, p, q, grid, stream)
                                                       : launch_pair<fp16, true>(ma, mb, ma, p, q, grid, stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        B200_FAIL("mm push: tcgen05 pair kernel launch failed: %s", cudaGetErrorString(e));
    }
    return diopiSuccess;
}

}  // namespace b200
