// Dense contraction on the 5th-generation tensor cores: C[b] = alpha * A[b] * B[b] + beta * bias.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer   - streams 128 x 64 tiles of A and BN x 64 tiles of B (bf16 / fp16) into a ring of
//                                128-byte-swizzled shared-memory stages (cp.async.bulk.tensor, per-CTA loads only)
//   warp 1      MMA issuer     - one thread issues tcgen05.mma (M=128, N=BN, K=16) accumulating fp32 in tensor
//                                memory; two accumulators of BN columns each are double-buffered so the epilogue of
//                                tile i overlaps the main loop of tile i+1
//   warps 2..5  epilogue       - tcgen05.ld the accumulator (each warp its own 32-lane quarter), scale / add bias,
//                                convert, stage 32 x 128-byte pieces in swizzled shared memory and write them with TMA
//                                stores (full 128-byte lines per row, ragged edges clipped by the hardware); outputs whose
//                                pitch or base is not 16-byte aligned are stored straight from registers instead
// Stages and accumulators are handed over with mbarriers; every wait is bounded (see gemm_sm100.cuh) and a
// time-out is reported through the status word instead of hanging.
//
// Operand layouts (taken from the tensors' strides, no copies):
//   A  [batch, M, K]  K contiguous
//   B  [batch, N, K]  K contiguous  ("K-major": the transposed view of an [N,K] weight that F.linear passes), or
//      [batch, K, N]  N contiguous  ("MN-major": a plain [K,N] matrix, e.g. V in P*V)
//   C  [batch, M, N]  N contiguous, row pitch ldc
// Tile order groups 8 row-blocks so that a wave of CTAs shares A and B tiles in L2.
#include <cuda.h>

#include <mutex>
#include <set>
#include <utility>

#include "gemm.h"
#include "diopi/functions_b200.h"
#include "gemm_sm100.cuh"
#include "device_utils.cuh"

namespace b200 {
namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;          // 64 two-byte elements = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kGroupM = 8;
constexpr int kSmemLimit = 232448;  // 227 KiB per CTA

template <int BN, int EPI = 4>
struct TileCfg {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStoreBytes = EPI /*warps*/ * 2 /*buffers*/ * 32 /*rows*/ * 128 /*bytes*/;  // epilogue staging
    static constexpr int kStagesRaw = (kSmemLimit - 1024 - 512 - kStoreBytes) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
    static constexpr int kTmemCols = (2 * BN) < 32 ? 32 : (2 * BN);
    static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

struct TcParams {
    int M, N, K, batch;
    int m_blocks, n_blocks, k_blocks;
    int64_t ldc, stride_cb;
    void* C;
    const void* bias;  // same dtype as C, may be nullptr
    int64_t bias_sb, bias_sr, bias_sc;
    float alpha, beta;
    uint32_t idesc;
    int b_mn_major;
    int c_vec_ok;
    int tma_store;  // epilogue writes through map_c
    int rotate_k;   // start each tile's K loop at a tile-dependent block (see the producer)
    int bias_vec_ok;  // additive input: unit column stride, 16-byte aligned rows
    uint32_t* status;
};

__device__ __forceinline__ void tile_coords(int tile, const TcParams& p, int* b, int* mb, int* nb) {
    const int per_batch = p.m_blocks * p.n_blocks;
    *b = tile / per_batch;
    const int t = tile - *b * per_batch;
    const int group_sz = kGroupM * p.n_blocks;
    const int g = t / group_sz;
    const int first_m = g * kGroupM;
    const int rows = min(p.m_blocks - first_m, kGroupM);
    const int r = t - g * group_sz;
    *mb = first_m + r % rows;
    *nb = r / rows;
}

template <typename TOut>
__device__ __forceinline__ void store_chunk(const TcParams& p, const uint32_t (&acc)[32], int b, int row, int col0) {
    if (row >= p.M) return;
    TOut* crow = static_cast<TOut*>(p.C) + static_cast<int64_t>(b) * p.stride_cb + static_cast<int64_t>(row) * p.ldc;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]) * p.alpha;
    if (p.bias != nullptr) {
        const TOut* brow = static_cast<const TOut*>(p.bias) + static_cast<int64_t>(b) * p.bias_sb + static_cast<int64_t>(row) * p.bias_sr;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (col0 + j < p.N) v[j] += p.beta * to_f32(brow[static_cast<int64_t>(col0 + j) * p.bias_sc]);
        }
    }
    if (p.c_vec_ok && col0 + 32 <= p.N) {
        constexpr int V = 16 / sizeof(TOut);
#pragma unroll
        for (int j = 0; j < 32; j += V) {
            Vec16<TOut> o;
#pragma unroll
            for (int e = 0; e < V; ++e) o.v[e] = from_f32<TOut>(v[j + e]);
            st16(crow + col0 + j, o);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (col0 + j < p.N) crow[col0 + j] = from_f32<TOut>(v[j]);
        }
    }
}

// EPI: epilogue warps, 4 or 8. With 8, two warps share each 32-lane quarter of the accumulator and take half of the tile's
// columns each: for products with a short K loop (Q K^T: two K blocks per 64 KiB output tile) the epilogue, not the
// tensor pipe, is the critical path, and its per-piece latency chain (TMEM load, convert, stage, bulk store) needs more
// warps in flight to keep the store stream busy.
template <int BN, typename TOut, int EPI>
__global__ void __launch_bounds__(64 + 32 * EPI, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
               const TcParams p) {
    using Cfg = TileCfg<BN, EPI>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle patterns repeat every 1024 bytes: stage buffers must start on that boundary
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * Cfg::kABytes;
    uint8_t* smem_c = smem + STAGES * Cfg::kStageBytes;  // [4 warps][2 buffers][32 rows x 128 bytes], 1024-byte aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_c + Cfg::kStoreBytes);
    uint64_t* full_bar = bars;                     // [STAGES] producer -> MMA
    uint64_t* empty_bar = bars + STAGES;           // [STAGES] MMA -> producer
    uint64_t* acc_full = bars + 2 * STAGES;        // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * STAGES + 2;   // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = p.batch * p.m_blocks * p.n_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], EPI);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        if (p.tma_store) prefetch_tensormap(&map_c);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int b, mb, nb;
                tile_coords(tile, p, &b, &mb, &nb);
                // When there is a single row-block (decode: M <= 128) every CTA would read the same A tile at the same moment
                // and the L2 slice holding it becomes the bottleneck. Starting each tile's K loop at a different block
                // spreads those reads over the whole A matrix; the sum is the same up to fp32 association.
                const int rot = p.rotate_k ? static_cast<int>((static_cast<unsigned>(tile) * 7u) % static_cast<unsigned>(p.k_blocks)) : 0;
                for (int it = 0; it < p.k_blocks; ++it) {
                    int kb = it + rot;
                    if (kb >= p.k_blocks) kb -= p.k_blocks;
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
                    tma_load_3d(smem_a + stage * Cfg::kABytes, &map_a, &full_bar[stage], kb * BK, mb * BM, b);
                    if (!p.b_mn_major) {
                        tma_load_3d(smem_b + stage * Cfg::kBBytes, &map_b, &full_bar[stage], kb * BK, nb * BN, b);
                    } else {
#pragma unroll
                        for (int g = 0; g < BN / 64; ++g) {
                            tma_load_3d(smem_b + stage * Cfg::kBBytes + g * (64 * BK * 2), &map_b, &full_bar[stage], nb * BN + g * 64, kb * BK, b);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1u;
                if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + stage * Cfg::kABytes);
                    const uint32_t b_addr = smem_u32(smem_b + stage * Cfg::kBBytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major operand: 8-row groups are 1024 bytes apart, a K step of 16 elements moves 32 bytes inside
                        // the swizzled row. MN-major B: 64-column groups are 8192 bytes apart (leading offset), 8-row K
                        // groups 1024 bytes apart, a K step of 16 rows moves 2048 bytes.
                        const uint64_t da = make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
                        const uint64_t db = p.b_mn_major ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                                         : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
                        umma_f16_ss(d_tmem, da, db, p.idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(&acc_full[acc]);
            }
        }
    } else {
        // ---------------- epilogue (warps 2 .. 2+EPI-1) ----------------
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are the ones this warp may read
        const int half = (warp - 2) >> 2;  // with eight warps: which half of the tile's columns this warp converts
        int local = 0;
        uint32_t store_seq = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            int b, mb, nb;
            tile_coords(tile, p, &b, &mb, &nb);
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1u;
            if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int row = mb * BM + quarter * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
            if (mb * BM + quarter * 32 >= p.M) {
                // this warp's 32 accumulator rows lie beyond the matrix (few-row products): nothing to read or store
            } else if (p.tma_store) {
                // One piece = 32 rows x 128 bytes (64 two-byte or 32 four-byte columns), double-buffered per warp.
                constexpr int PIECE_COLS = 128 / static_cast<int>(sizeof(TOut));
                constexpr int LOADS = PIECE_COLS / 32;
                uint8_t* stage_base = smem_c + (warp - 2) * (2 * 32 * 128);
                constexpr int PIECES = BN / PIECE_COLS;
                const int c_begin = EPI == 8 ? half * (PIECES / 2) : 0;
                const int c_end = EPI == 8 ? c_begin + PIECES / 2 : PIECES;
#pragma unroll 1
                for (int c = c_begin; c < c_end; ++c) {
                    const int col0 = nb * BN + c * PIECE_COLS;
                    if (col0 >= p.N) break;  // warp-uniform
                    uint8_t* buf = stage_base + (store_seq & 1) * (32 * 128);
                    // the store issued from this buffer two pieces ago must have finished reading it
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                    // all TMEM loads of the piece are issued before the single wait: their latencies overlap
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
                                // dense row of the additive input (a [S, S] mask, a full matrix): 16-byte loads
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
                        // 16-byte chunk k of row `lane` lives at chunk position k ^ (lane & 7): the 128-byte swizzle the
                        // store's tensor map expects, and conflict-free for the warp's writes
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
                    fence_proxy_async();  // make the generic-proxy writes visible to the bulk copy engine
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&map_c, buf, col0, mb * BM + quarter * 32, b);
                        tma_store_commit();
                    }
                    ++store_seq;
                }
            } else {
                const int s_begin = EPI == 8 ? half * (BN / 64) : 0;
                const int s_end = EPI == 8 ? s_begin + BN / 64 : BN / 32;
#pragma unroll 1
                for (int c = s_begin; c < s_end; ++c) {
                    const int col0 = nb * BN + c * 32;
                    if (col0 >= p.N) break;  // warp-uniform
                    uint32_t r[32];
                    tmem_ld_32x32(t_row + c * 32, r);
                    tmem_ld_wait();
                    store_chunk<TOut>(p, r, b, row, col0);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
        // all stores of this warp must be complete before the CTA's shared memory goes away
        if (p.tma_store && lane == 0) tma_store_wait_all<0>();
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag != 0) {
        // A wait timed out. Give copies and MMAs that are still in flight time to land before the CTA's shared and
        // tensor memory are released, then report.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0) atomicExch(p.status, 1u);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();  // the issuing lane took a different path: reconverge before the warp-wide dealloc
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---- split-K variant for a single row-block (M <= 128: decode) -------------------------------------------------------------
// With few rows the product is bound by streaming the weight matrix once; a tile per CTA leaves most SMs idle (N / BN
// tiles) and shrinking BN makes every CTA re-read all of A. Here a cluster of S CTAs shares one 128 x BN output tile,
// each CTA contracting its own slice of K (so A is read N/BN times in total, B exactly once, and tiles x S CTAs stream).
// The fp32 partial tiles are exchanged through distributed shared memory: every CTA parks its accumulator in its own
// shared memory (the drained pipeline stages), the cluster synchronises, CTA r sums its share of the tile's 16-byte column
// chunks over all S partials in rank order and writes them out. No global workspace, one launch, deterministic.
// S is any cluster size from 1 to 8 (the planner picks tiles x S close to the SM count; S = 1 is a wide product whose
// tiles alone occupy the SMs, each CTA streaming its whole K extent). With swiglu != 0 the tile's columns are (gate, up)
// pairs and the output is silu(gate) * up, half as wide: the SiLU and the product of the feed-forward block ride in the
// epilogue of ONE product over the interleaved gate / up weight instead of two products and two element-wise kernels.
struct SplitKParams {
    int M, N, K, batch;
    int n_blocks, k_blocks, kb_per_cta, splits;
    int64_t ldc, stride_cb;
    void* C;
    const void* bias;
    int64_t bias_sb, bias_sr, bias_sc;
    float alpha, beta;
    uint32_t idesc;
    int b_mn_major;
    int swiglu;
    uint32_t* status;
};

template <int BN, typename TOut>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_splitk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const SplitKParams p) {
    using Cfg = TileCfg<BN>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * Cfg::kABytes;
    float* partial = reinterpret_cast<float*>(smem);  // [128][BN] fp32 over the drained stages, 16-byte chunks swizzled per row
    static_assert(STAGES * Cfg::kStageBytes >= BM * BN * 4, "stage memory must hold the fp32 partial tile");
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes + Cfg::kStoreBytes);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ks = cluster_ctarank();           // this CTA's K slice
    const int tile = blockIdx.x / p.splits;           // (batch, n-block) shared by the cluster
    const int b = tile / p.n_blocks;
    const int nb = tile - b * p.n_blocks;
    const int kb0 = static_cast<int>(ks) * p.kb_per_cta;
    const int kb1 = min(p.k_blocks, kb0 + p.kb_per_cta);
    const int my_kb = max(kb1 - kb0, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, BN < 32 ? 32 : BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Launched as a programmatic dependent (launch_splitk), this CTA may have been set up while the kernel before it in the stream
    // was still running; nothing of that kernel has been read and nothing written up to here.
    grid_dependency_wait();
    grid_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int it = 0; it < my_kb; ++it) {
                const int kb = kb0 + it;
                if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) break;
                mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
                tma_load_3d(smem_a + stage * Cfg::kABytes, &map_a, &full_bar[stage], kb * BK, 0, b);
                if (!p.b_mn_major) {
                    tma_load_3d(smem_b + stage * Cfg::kBBytes, &map_b, &full_bar[stage], kb * BK, nb * BN, b);
                } else {
#pragma unroll
                    for (int g = 0; g < BN / 64; ++g) {
                        tma_load_3d(smem_b + stage * Cfg::kBBytes + g * (64 * BK * 2), &map_b, &full_bar[stage], nb * BN + g * 64, kb * BK, b);
                    }
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int it = 0; it < my_kb; ++it) {
                if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem_a + stage * Cfg::kABytes);
                const uint32_t b_addr = smem_u32(smem_b + stage * Cfg::kBBytes);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t da = make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
                    const uint64_t db = p.b_mn_major ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                                     : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
                    umma_f16_ss(tmem_base, da, db, p.idesc, (it | k) != 0 ? 1u : 0u);
                }
                umma_commit(&empty_bar[stage]);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) {
                if (my_kb > 0) umma_commit(acc_full);
                else mbar_arrive(acc_full);  // empty K slice: nothing to wait for
            }
        }
    } else {
        // epilogue part 1: accumulator -> this CTA's shared memory (rows that exist only)
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        if (mbar_wait(acc_full, 0, abort_flag)) {
            tc_fence_after();
            if (quarter * 32 < p.M) {  // warp-uniform: this quarter holds real rows
                const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    if (my_kb > 0) {
                        tmem_ld_32x32(t_row + c * 32, r);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = 0u;  // empty K slice: contributes zeros
                    }
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int chunk = (c * 32 + j) / 4;
                        float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        *reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(partial) + static_cast<size_t>(row) * (BN * 4) +
                                                   ((chunk ^ (row & 7)) * 16)) = v;
                    }
                }
            }
            tc_fence_before();
        }
    }

    // every thread of every CTA of the cluster passes here, also after a timed-out wait
    __syncthreads();
    __syncwarp();  // lanes that ran a role loop rejoin their warp before the warp-aligned cluster barrier
    cluster_sync_all();

    if (warp >= 2 && *abort_flag == 0) {
        // epilogue part 2: this CTA owns the 16-byte column chunks [c0, c1) of the tile: sum them over the S partials
        constexpr int kChunks = BN / 4;
        const int c0 = (static_cast<int>(ks) * kChunks) / p.splits, c1 = ((static_cast<int>(ks) + 1) * kChunks) / p.splits;
        const int chunks_per_row = c1 - c0;
        const int rows = min(p.M, BM);
        const int items = rows * chunks_per_row;
        const uint32_t local_base = smem_u32(partial);
        for (int i = threadIdx.x - 64; i < items; i += 128) {
            const int row = i / chunks_per_row;
            const int chunk = c0 + (i - row * chunks_per_row);
            const uint32_t off = static_cast<uint32_t>(row) * (BN * 4) + ((chunk ^ (row & 7)) * 16);
            // all partials of the chunk are requested before the first one is used: a remote shared-memory load takes several
            // hundred cycles, and a loop that adds them one by one would wait that long per CTA of the cluster
            float4 v[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (s < p.splits) v[s] = ld_cluster_f4(map_to_cta(local_base + off, static_cast<uint32_t>(s)));
            }
            float4 acc = v[0];
#pragma unroll
            for (int s = 1; s < 8; ++s) {
                if (s < p.splits) {
                    acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w;
                }
            }
            const int col = nb * BN + chunk * 4;
            TOut* crow = static_cast<TOut*>(p.C) + static_cast<int64_t>(b) * p.stride_cb + static_cast<int64_t>(row) * p.ldc;
            if (p.swiglu) {
                // columns (col, col + 1) and (col + 2, col + 3) are (gate, up) pairs: two outputs at col / 2
                const float g0 = acc.x * p.alpha, u0 = acc.y * p.alpha, g1 = acc.z * p.alpha, u1 = acc.w * p.alpha;
                const int oc = col >> 1;
                if (col + 1 < p.N) crow[oc] = from_f32<TOut>(g0 / (1.f + __expf(-g0)) * u0);
                if (col + 3 < p.N) crow[oc + 1] = from_f32<TOut>(g1 / (1.f + __expf(-g1)) * u1);
                continue;
            }
            float o[4] = {acc.x * p.alpha, acc.y * p.alpha, acc.z * p.alpha, acc.w * p.alpha};
            if (p.bias != nullptr) {
                const TOut* brow = static_cast<const TOut*>(p.bias) + static_cast<int64_t>(b) * p.bias_sb + static_cast<int64_t>(row) * p.bias_sr;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (col + j < p.N) o[j] += p.beta * to_f32(brow[static_cast<int64_t>(col + j) * p.bias_sc]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (col + j < p.N) crow[col + j] = from_f32<TOut>(o[j]);
            }
        }
    }

    // no CTA may leave while its shared memory can still be read by a peer
    __syncwarp();
    cluster_sync_all();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag != 0) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0) atomicExch(p.status, 1u);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, BN < 32 ? 32 : BN);
    }
}

// ---- host side -------------------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeFn>(sym);
        }
        (void)cudaGetLastError();
    });
    return fn;
}

// 3-D map over [batch, rows, inner] with a [1, box_rows, 128 bytes] box and 128-byte swizzle.
bool encode_map(CUtensorMap* map, diopiDtype_t dtype, const void* base, int64_t inner, int64_t rows, int64_t batch, int64_t row_pitch_elems,
                int64_t batch_pitch_elems, int box_rows) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const int es = dtype == diopi_dtype_float32 ? 4 : 2;
    const CUtensorMapDataType dt = dtype == diopi_dtype_float32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (dtype == diopi_dtype_bfloat16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_pitch_elems * es), static_cast<cuuint64_t>(batch_pitch_elems * es)};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(box_rows), 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

cudaError_t ensure_smem_attr(const void* kernel, int bytes) {
    static std::mutex mu;
    static std::set<std::pair<int, const void*>> done;
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_pair(dev, kernel);
    if (done.count(key) != 0) return cudaSuccess;
    if (cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); e != cudaSuccess) return e;
    done.insert(key);
    return cudaSuccess;
}

uint32_t* status_word() {
    // one status word per device, kept for the life of the process: allocated by diopiB200Init when the host announces the
    // device, or on first use when it did not
    static uint32_t* words[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (words[dev] == nullptr) {
        uint32_t* w = nullptr;
        if (cudaMalloc(&w, sizeof(uint32_t)) != cudaSuccess) return nullptr;
        cudaMemset(w, 0, sizeof(uint32_t));
        words[dev] = w;
    }
    return words[dev];
}

template <int BN, typename TOut, int EPI>
cudaError_t launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const TcParams& p, int grid, cudaStream_t stream) {
    using Cfg = TileCfg<BN, EPI>;
    if (cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(gemm_tc_kernel<BN, TOut, EPI>), Cfg::kSmemBytes); e != cudaSuccess) return e;
    gemm_tc_kernel<BN, TOut, EPI><<<grid, 64 + 32 * EPI, Cfg::kSmemBytes, stream>>>(ma, mb, mc, p);
    return cudaPeekAtLastError();
}

template <typename TOut>
cudaError_t launch_tc_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const TcParams& p, int grid,
                         cudaStream_t stream) {
    // eight epilogue warps where the K loop is too short to hide the epilogue (and the tile is wide enough to split)
    const bool wide_epilogue = p.k_blocks <= 8 && bn >= 128;
    switch (bn) {
        case 256: return wide_epilogue ? launch_tc<256, TOut, 8>(ma, mb, mc, p, grid, stream) : launch_tc<256, TOut, 4>(ma, mb, mc, p, grid, stream);
        case 128: return wide_epilogue ? launch_tc<128, TOut, 8>(ma, mb, mc, p, grid, stream) : launch_tc<128, TOut, 4>(ma, mb, mc, p, grid, stream);
        case 64: return launch_tc<64, TOut, 4>(ma, mb, mc, p, grid, stream);
        default: return launch_tc<32, TOut, 4>(ma, mb, mc, p, grid, stream);
    }
}

template <int BN, typename TOut>
cudaError_t launch_splitk(const CUtensorMap& ma, const CUtensorMap& mb, const SplitKParams& p, int grid, cudaStream_t stream) {
    using Cfg = TileCfg<BN>;
    if (cudaError_t e = ensure_smem_attr(reinterpret_cast<const void*>(gemm_tc_splitk_kernel<BN, TOut>), Cfg::kSmemBytes); e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(p.splits);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // Programmatic dependent launch: in a decode step these products are 10 - 30 us kernels between other short kernels, and the
    // set-up of one (launch, barriers, tensor memory, descriptor fetch) overlaps the tail of the kernel before it (back-to-back
    // [64, 4096] x [4096, 4096]: 17.1 -> 13.2 us per product; requesting the first weight tiles into L2 during that overlap
    // measured no further gain). The kernel reads and writes global data only after griddepcontrol.wait.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_splitk_kernel<BN, TOut>, ma, mb, p);
}

template <typename TOut>
cudaError_t launch_splitk_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const SplitKParams& p, int grid, cudaStream_t stream) {
    switch (bn) {
        case 256: return launch_splitk<256, TOut>(ma, mb, p, grid, stream);
        case 128: return launch_splitk<128, TOut>(ma, mb, p, grid, stream);
        default: return launch_splitk<64, TOut>(ma, mb, p, grid, stream);
    }
}

// Plan of the single-row-block kernel (M <= 128): tile width (256, 128 or 64 columns) and cluster size (1 to 4 CTAs sharing
// a tile's K extent). The pair that puts the most CTAs on the device without exceeding one CTA per SM wins; among equals the
// larger cluster (wider tiles re-read A less often). Clusters of 8 measured slower than clusters of 4 on narrower tiles
// ([64, 4096] x [4096, 4096]: 25.5 against 15.8 us; K = 11008: 38.6 against 25.3 us), so 4 is the limit.
// Returns false when plain tiling is the better choice: more tiles than SMs even at 256 columns (the persistent kernel walks
// them), or a single CTA per tile without a fused epilogue (the persistent kernel's TMA-store epilogue serves that).
bool plan_splitk(const GemmProblem& g, int sms, int* bn_out, int* splits_out) {
    if (g.M > BM) return false;
    const int64_t k_blocks = (g.K + BK - 1) / BK;
    int best_bn = 0, best_splits = 0;
    int64_t best_ctas = 0;
    for (int bn = 256; bn >= 64; bn >>= 1) {
        if (bn > 64 && g.N <= bn / 2) continue;  // a tile twice as wide as the product
        const int64_t tiles = ((g.N + bn - 1) / bn) * g.batch;
        if (tiles > sms) continue;
        int64_t splits = sms / tiles;
        if (splits > 4) splits = 4;
        if (splits > k_blocks) splits = k_blocks;
        if (splits < 1) splits = 1;
        const int64_t ctas = tiles * splits;
        if (ctas > best_ctas || (ctas == best_ctas && splits > best_splits)) {
            best_ctas = ctas;
            best_bn = bn;
            best_splits = static_cast<int>(splits);
        }
    }
    if (best_bn == 0) return false;
    if (best_splits < 2 && g.epilogue == GemmProblem::kPlain) return false;
    *bn_out = best_bn;
    *splits_out = best_splits;
    return true;
}

}  // namespace

bool tc_encode_map(::CUtensorMap_st* map, diopiDtype_t dtype, const void* base, int64_t inner, int64_t rows, int64_t batch, int64_t row_pitch_elems,
                   int64_t batch_pitch_elems, int box_rows) {
    return encode_map(reinterpret_cast<CUtensorMap*>(map), dtype, base, inner, rows, batch, row_pitch_elems, batch_pitch_elems, box_rows);
}
// 4-D map over a [d3, d2, d1, inner] view (pitches in elements) with a [1, box2, box1, 128 bytes] box and 128-byte swizzle.
bool tc_encode_map4(::CUtensorMap_st* map, diopiDtype_t dtype, const void* base, const int64_t dims[4], const int64_t pitch_elems[3], int box1,
                    int box2) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const int es = dtype == diopi_dtype_float32 ? 4 : 2;
    const CUtensorMapDataType dt = dtype == diopi_dtype_float32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (dtype == diopi_dtype_bfloat16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    const cuuint64_t d[4] = {static_cast<cuuint64_t>(dims[0]), static_cast<cuuint64_t>(dims[1]), static_cast<cuuint64_t>(dims[2]),
                             static_cast<cuuint64_t>(dims[3])};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(pitch_elems[0] * es), static_cast<cuuint64_t>(pitch_elems[1] * es),
                                   static_cast<cuuint64_t>(pitch_elems[2] * es)};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(box1), static_cast<cuuint32_t>(box2), 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    const CUresult r = fn(reinterpret_cast<CUtensorMap*>(map), dt, 4, const_cast<void*>(base), d, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}
uint32_t* tc_status_word() { return status_word(); }
cudaError_t tc_ensure_smem_attr(const void* kernel, int bytes) { return ensure_smem_attr(kernel, bytes); }

bool gemm_tc_eligible(const GemmProblem& g) {
    if (!(g.ab_dtype == diopi_dtype_bfloat16 || g.ab_dtype == diopi_dtype_float16)) return false;
    if (!(g.c_dtype == g.ab_dtype || g.c_dtype == diopi_dtype_float32)) return false;
    if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.batch <= 0) return false;
    if (g.M > 0x7fffffffLL || g.N > 0x7fffffffLL || g.K > 0x7fffffffLL) return false;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    auto pitch_ok = [](int64_t elems) { return elems > 0 && (elems * 2) % 16 == 0 && elems * 2 < (1ll << 40); };
    // A: K contiguous
    if (g.a_sk != 1 || !al16(g.A) || !pitch_ok(g.a_sm)) return false;
    if (g.batch > 1 && !pitch_ok(g.a_sb)) return false;
    if (g.a_sm < g.K) return false;
    // B: K contiguous or N contiguous
    if (!al16(g.B)) return false;
    if (g.b_sk == 1) {
        if (!pitch_ok(g.b_sn) || g.b_sn < g.K) return false;
    } else if (g.b_sn == 1) {
        if (!pitch_ok(g.b_sk) || g.b_sk < g.N) return false;
    } else {
        return false;
    }
    if (g.batch > 1 && !pitch_ok(g.b_sb)) return false;
    if (g.c_sn != 1 || g.c_sm < g.N) return false;
    if (g.bias != nullptr && g.bias_dtype != g.c_dtype) return false;
    const int64_t tiles = g.batch * ((g.M + BM - 1) / BM) * ((g.N + 31) / 32);
    if (tiles > 0x7fffffffLL) return false;
    return get_encode_fn() != nullptr;
}

diopiError_t gemm_tc_launch(const GemmProblem& g, cudaStream_t stream) {
    const bool is_bf16 = g.ab_dtype == diopi_dtype_bfloat16;
    const bool b_mn = g.b_sk != 1;
    const int sms = sm_count();
    const int64_t m_blocks = (g.M + BM - 1) / BM;
    // widest tile that still yields at least one tile per SM; MN-major B needs whole 64-column swizzle groups
    int bn = 256;
    const int min_bn = b_mn ? 64 : 32;
    while (bn > min_bn && (g.N <= bn / 2 || g.batch * m_blocks * ((g.N + bn - 1) / bn) < sms)) bn >>= 1;
    const int64_t n_blocks = (g.N + bn - 1) / bn;

    if (g.epilogue == GemmProblem::kPlain && gemm_tc2_applies(g)) return gemm_tc2_launch(g, stream);
    int sk_bn = 0, sk_splits = 0;
    const bool planned = plan_splitk(g, sms, &sk_bn, &sk_splits);
    B200_CHECK(planned || g.epilogue == GemmProblem::kPlain,
               "gemm: the fused gate / up epilogue is served for up to %d rows and at most %d tiles of 256 columns (got %lld x %lld)", BM, sms,
               (long long)g.M, (long long)g.N);
    if (planned) {
        const bool b_mn_sk = b_mn;
        CUtensorMap sa, sb;
        B200_CHECK(encode_map(&sa, g.ab_dtype, g.A, g.K, g.M, g.batch, g.a_sm, g.batch > 1 ? g.a_sb : g.a_sm * g.M, BM),
                   "gemm: cuTensorMapEncodeTiled failed for A");
        if (!b_mn_sk) {
            B200_CHECK(encode_map(&sb, g.ab_dtype, g.B, g.K, g.N, g.batch, g.b_sn, g.batch > 1 ? g.b_sb : g.b_sn * g.N, sk_bn),
                       "gemm: cuTensorMapEncodeTiled failed for B (K-major)");
        } else {
            B200_CHECK(encode_map(&sb, g.ab_dtype, g.B, g.N, g.K, g.batch, g.b_sk, g.batch > 1 ? g.b_sb : g.b_sk * g.K, BK),
                       "gemm: cuTensorMapEncodeTiled failed for B (MN-major)");
        }
        SplitKParams q;
        q.M = static_cast<int>(g.M); q.N = static_cast<int>(g.N); q.K = static_cast<int>(g.K); q.batch = static_cast<int>(g.batch);
        q.n_blocks = static_cast<int>((g.N + sk_bn - 1) / sk_bn);
        q.k_blocks = static_cast<int>((g.K + BK - 1) / BK);
        q.splits = sk_splits;
        q.kb_per_cta = (q.k_blocks + sk_splits - 1) / sk_splits;
        q.ldc = g.c_sm; q.stride_cb = g.c_sb; q.C = g.C;
        q.bias = g.bias; q.bias_sb = g.bias_sb; q.bias_sr = g.bias_sm; q.bias_sc = g.bias_sn;
        q.alpha = g.alpha; q.beta = g.beta;
        q.idesc = make_idesc_f16(is_bf16 ? 1 : 0, b_mn_sk, BM, sk_bn);
        q.b_mn_major = b_mn_sk ? 1 : 0;
        q.swiglu = g.epilogue == GemmProblem::kSwiGLU ? 1 : 0;
        q.status = g.status_override != nullptr ? g.status_override : status_word();
        B200_CHECK(q.status != nullptr, "gemm: could not allocate the kernel status word");
        const int grid_sk = q.batch * q.n_blocks * sk_splits;
        cudaError_t ek;
        if (g.c_dtype == diopi_dtype_bfloat16) ek = launch_splitk_bn<bf16>(sk_bn, sa, sb, q, grid_sk, stream);
        else if (g.c_dtype == diopi_dtype_float16) ek = launch_splitk_bn<fp16>(sk_bn, sa, sb, q, grid_sk, stream);
        else ek = launch_splitk_bn<float>(sk_bn, sa, sb, q, grid_sk, stream);
        if (ek != cudaSuccess) {
            (void)cudaGetLastError();
            B200_FAIL("gemm: split-K tcgen05 kernel launch failed: %s", cudaGetErrorString(ek));
        }
        return diopiSuccess;
    }

    CUtensorMap ma, mb, mc;
    B200_CHECK(encode_map(&ma, g.ab_dtype, g.A, g.K, g.M, g.batch, g.a_sm, g.batch > 1 ? g.a_sb : g.a_sm * g.M, BM),
               "gemm: cuTensorMapEncodeTiled failed for A");
    if (!b_mn) {
        B200_CHECK(encode_map(&mb, g.ab_dtype, g.B, g.K, g.N, g.batch, g.b_sn, g.batch > 1 ? g.b_sb : g.b_sn * g.N, bn),
                   "gemm: cuTensorMapEncodeTiled failed for B (K-major)");
    } else {
        B200_CHECK(encode_map(&mb, g.ab_dtype, g.B, g.N, g.K, g.batch, g.b_sk, g.batch > 1 ? g.b_sb : g.b_sk * g.K, BK),
                   "gemm: cuTensorMapEncodeTiled failed for B (MN-major)");
    }
    TcParams p;
    p.M = static_cast<int>(g.M); p.N = static_cast<int>(g.N); p.K = static_cast<int>(g.K); p.batch = static_cast<int>(g.batch);
    p.m_blocks = static_cast<int>(m_blocks); p.n_blocks = static_cast<int>(n_blocks); p.k_blocks = static_cast<int>((g.K + BK - 1) / BK);
    p.ldc = g.c_sm; p.stride_cb = g.c_sb; p.C = g.C;
    p.bias = g.bias; p.bias_sb = g.bias_sb; p.bias_sr = g.bias_sm; p.bias_sc = g.bias_sn;
    p.alpha = g.alpha; p.beta = g.beta;
    p.idesc = make_idesc_f16(is_bf16 ? 1 : 0, b_mn, BM, bn);
    p.b_mn_major = b_mn ? 1 : 0;
    const int64_t c_es = dtype_size(g.c_dtype);
    p.c_vec_ok = ((reinterpret_cast<uintptr_t>(g.C) & 15u) == 0 && (g.c_sm * c_es) % 16 == 0 && (g.batch == 1 || (g.c_sb * c_es) % 16 == 0)) ? 1 : 0;
    // TMA-store epilogue whenever the output obeys the 16-byte rules; the map is encoded even when unused (kernel parameter)
    p.tma_store = (p.c_vec_ok && bn * c_es >= 128) ? 1 : 0;  // a piece is 128 bytes wide: narrower tiles store from registers
    if (p.tma_store) {
        p.tma_store = encode_map(&mc, g.c_dtype, g.C, g.N, g.M, g.batch, g.c_sm, g.batch > 1 ? g.c_sb : g.c_sm * g.M, 32) ? 1 : 0;
    }
    if (!p.tma_store) mc = ma;
    p.rotate_k = (m_blocks == 1 && p.k_blocks > 1) ? 1 : 0;
    p.bias_vec_ok = (g.bias != nullptr && g.bias_sn == 1 && (reinterpret_cast<uintptr_t>(g.bias) & 15u) == 0 && (g.bias_sm * c_es) % 16 == 0 &&
                     (g.bias_sb * c_es) % 16 == 0) ? 1 : 0;
    p.status = g.status_override != nullptr ? g.status_override : status_word();
    B200_CHECK(p.status != nullptr, "gemm: could not allocate the kernel status word");
    const int64_t total = static_cast<int64_t>(p.batch) * m_blocks * n_blocks;
    const int grid = static_cast<int>(total < sms ? total : sms);
    cudaError_t e;
    if (g.c_dtype == diopi_dtype_bfloat16) e = launch_tc_bn<bf16>(bn, ma, mb, mc, p, grid, stream);
    else if (g.c_dtype == diopi_dtype_float16) e = launch_tc_bn<fp16>(bn, ma, mb, mc, p, grid, stream);
    else e = launch_tc_bn<float>(bn, ma, mb, mc, p, grid, stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        B200_FAIL("gemm: tcgen05 kernel launch failed: %s", cudaGetErrorString(e));
    }
    return diopiSuccess;
}

}  // namespace b200

// One-time set-up on the current device, for hosts that want it out of the first operator call: allocates and clears the
// status word of the tensor-core kernels (a cudaMalloc and a synchronising memset that otherwise happen inside the first
// product). Call it where the host initialises a device (DIPU: initializeVendor / the first setDevice); calling it again is
// free. Operators work without it.
extern "C" DIOPI_API diopiError_t diopiB200Init(void) {
    using namespace b200;
    B200_CHECK(status_word() != nullptr, "diopiB200Init: could not allocate the kernels' status word on the current device");
    return diopiSuccess;
}

extern "C" DIOPI_API void diopiB200SetPushWaitLimitNs(unsigned long long ns) { b200::gemm_tc2_set_push_wait_limit_ns(ns); }

// Status of the tensor-core kernels on the current device: 0 = no wait has ever timed out.
// Synchronises the device. Not part of DIOPI; exported for tests and health checks.
extern "C" DIOPI_API int diopiB200GemmStatus(void) {
    uint32_t* w = b200::status_word();
    if (w == nullptr) return -1;
    uint32_t v = 0;
    if (cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return static_cast<int>(v);
}

// ---- matrix product that allocates nothing ---------------------------------------------------------------------------
// The tensor-core kernel's only scratch is its status word. diopiMm keeps it in memory obtained with cudaMalloc on
// first use; here it lives in a static block of the library image, so the entry point below never allocates.
namespace {
constexpr int kNoAllocScratchWords = 64;  // 256 bytes; word 0 is the status word, the rest is reserved
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocScratchWords];

std::mutex g_noalloc_mu;
uint32_t* g_noalloc_ptr[64] = {nullptr};

// Device address of the static block on the current device. In host code the array's name is only a handle for the
// runtime, not an address a kernel could use: the address has to be asked for, once per device.
uint32_t* noalloc_scratch_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        b200::set_last_error("diopiB200MmNoAlloc: cannot determine the current device");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
        uint32_t* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            b200::set_last_error("diopiB200MmNoAlloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return nullptr;
        }
        g_noalloc_ptr[dev] = ptr;
    }
    return g_noalloc_ptr[dev];
}
}  // namespace

extern "C" DIOPI_API diopiError_t diopiB200MmNoAlloc(diopiStreamHandle_t stream, void* out, const void* mat1, const void* mat2, int64_t m,
                                                     int64_t n, int64_t k, int64_t ld1, int64_t ld2, int mat2_is_nk, int64_t ldo,
                                                     diopiDtype_t dtype) {
    using namespace b200;
    B200_CHECK(out != nullptr && mat1 != nullptr && mat2 != nullptr, "diopiB200MmNoAlloc: NULL operand");
    B200_CHECK(dtype == diopi_dtype_bfloat16 || dtype == diopi_dtype_float16, "diopiB200MmNoAlloc: dtype must be bfloat16 or float16, got %s",
               dtype_name(dtype));
    const int64_t lim = 0x7fffffffLL;
    B200_CHECK(m >= 1 && n >= 1 && k >= 1 && m <= lim && n <= lim && k <= lim,
               "diopiB200MmNoAlloc: dimensions must lie in [1, 2^31): got m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
    GemmProblem g;
    g.batch = 1; g.M = m; g.N = n; g.K = k;
    g.A = mat1; g.a_sm = ld1; g.a_sk = 1;
    g.B = mat2;
    if (mat2_is_nk) { g.b_sn = ld2; g.b_sk = 1; } else { g.b_sk = ld2; g.b_sn = 1; }
    g.C = out; g.c_sm = ldo; g.c_sn = 1;
    g.ab_dtype = dtype; g.c_dtype = dtype;
    B200_CHECK(gemm_tc_eligible(g),
               "diopiB200MmNoAlloc: operands do not meet the tensor-core kernel's layout rules (16-byte aligned pointers, pitches that are "
               "multiples of 8 elements and at least the row length); this entry point has no other path");
    uint32_t* scratch = noalloc_scratch_ptr();
    if (scratch == nullptr) return diopiErrorOccurred;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the block keeps whatever the previous call left: the status word must start at zero
    B200_CUDA(cudaMemsetAsync(scratch, 0, sizeof(uint32_t), s));
    g.status_override = scratch;
    return gemm_tc_launch(g, s);
}

extern "C" DIOPI_API int diopiB200NoAllocStatus(void) {
    uint32_t* scratch = noalloc_scratch_ptr();
    if (scratch == nullptr) return -1;
    uint32_t v = 0;
    if (cudaMemcpy(&v, scratch, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    return static_cast<int>(v);
}
