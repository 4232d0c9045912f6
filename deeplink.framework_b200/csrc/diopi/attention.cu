// Fused attention for the prefill step: out = softmax(scale * Q K^T + causal mask) V in one kernel, without the
// [heads, Sq, Skv] score tensor ever reaching HBM. This is the fused form of the bmm -> div -> add(mask) -> softmax ->
// bmm sequence of dicp/test/model/llama/model.py:146-150; the reference's own CPU restatement of the fused operator is
// dicp/dicp/vendor/AscendGraph/ext_ops.py:52-86 (prompt_attention_inference: causal, grouped K/V heads).
//
// One CTA per (batch, head, 256 query rows), 384 threads:
//   warp 0       TMA producer: the two 128-row Q tiles once, then K and V blocks of 128 keys through a 3-slot ring, the keys
//                one block ahead of the values (K0, K1, V0, K2, V1, ...)
//   warp 1, 3    MMA issuers (one thread each) for Q tile 0 and Q tile 1: S_t = Q_t K_j^T and O_t += P_t V_j with
//                tcgen05.mma, accumulators in TMEM. tcgen05.mma holds its issuing thread while the product is taken, so
//                with one issuer per tile the barrier polls and commits of one overlap the products of the other
//   warp 2       TMEM allocation (512 columns: S_0, S_1, O_0, O_1, 128 fp32 columns each)
//   warps 4..7   softmax of Q tile 0, warps 8..11 of Q tile 1: one thread per query row reads its 128 scores from
//                TMEM, keeps the running maximum and sum, writes P (bf16 / fp16) into swizzled shared memory as the A
//                operand of the second product, and rescales O in TMEM only when the maximum grew by more than 2^8
// Hand-over per tile and block j: as soon as the softmax warps hold S_j in registers (s_free) the issuer sends S_(j+1), so
// the next scores are ready before the softmax of block j is over and the softmax warps never wait for the tensor core;
// P_j is written after P V_(j-1) has completed (pv_done), then p_full releases P V_j. The special-function unit (4 lanes
// per cycle and scheduler) is what the softmax is bound by: the two warps of a scheduler (same TMEM quarter, one per tile)
// take turns at the exponentials, so that one warp's other phases (score load, maximum, P store, barriers) run in the
// shadow of its partner's exponentials. Causal blocks above the diagonal are skipped; only diagonal blocks pay for the
// element mask.
// Every wait is bounded (gemm_sm100.cuh); a time-out ends the kernel and is reported through the status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdlib>

#include "common.h"
#include "gemm.h"
#include "gemm_sm100.cuh"
#include "device_utils.cuh"

namespace b200 {
namespace {

using namespace sm100;

constexpr int kHeadDim = 128;
constexpr int kTileQ = 128;            // query rows per tile (one TMEM lane each)
constexpr int kTilesPerCta = 2;
constexpr int kBlockKv = 128;          // keys per block
constexpr int kRing = 3;               // K / V slots
constexpr int kTileBytes = 128 * 128 * 2;  // one 128 x 128 two-byte tile = two 128-byte-swizzled halves of 16 KiB
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int kAttnSmem = (kTilesPerCta * 2 + kRing) * kTileBytes + 1024 /*alignment*/ + 256 /*barriers*/ + 1024 /*row exchange*/ + 256 /*votes*/;
static_assert(kAttnSmem <= 232448, "shared memory budget");
constexpr float kRescaleThreshold = 8.f;   // log2 units: P stays below 2^8

struct AttnParams {
    int B, Hq, Hkv, Sq, Skv;
    int q_blocks;        // ceil(Sq / 256)
    int causal;
    int causal_off;      // Skv - Sq: key k is visible to query q iff k <= q + causal_off
    float scale_log2;    // softmax scale * log2(e)
    uint32_t idesc_s, idesc_pv;
    float* lse;          // optional [B, Hq, Sq] (any pitches), natural-log sum of exponentials
    int64_t lse_sb, lse_sh, lse_sq;
    // per operand: 1 = the tensor map's dimensions are (dim, head, row, batch), 0 = (dim, row, head, batch); the
    // dimension with the smaller pitch comes first
    int q_hfirst, k_hfirst, v_hfirst, o_hfirst;
    uint32_t* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Number of 128-key blocks a Q tile starting at row q_lo has to visit.
__device__ __forceinline__ int blocks_of_tile(const AttnParams& p, int q_lo) {
    if (q_lo >= p.Sq) return 0;
    int kv_end = p.Skv;
    if (p.causal) {
        const int q_hi = min(q_lo + kTileQ - 1, p.Sq - 1);
        kv_end = min(p.Skv, q_hi + p.causal_off + 1);
    }
    return kv_end <= 0 ? 0 : (kv_end + kBlockKv - 1) / kBlockKv;
}

// Named barrier over `count` threads (two partner warps of a row group); barrier 0 is the CTA-wide one.
__device__ __forceinline__ void pair_barrier(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }

// Position of block j's keys / values in the producer's load order (K0, K1, V0, K2, V1, ..., K(n-1), V(n-2), V(n-1)).
__device__ __forceinline__ int load_of_k(int j) { return j == 0 ? 0 : 2 * j - 1; }
__device__ __forceinline__ int load_of_v(int j, int n) { return min(2 * j + 2, 2 * n - 1); }

// SPLIT = threads per query row (1 or 2). With 2, the two threads of a row own 64 score columns each (warps w and w + 4 of
// the tile's eight softmax warps share a 32-lane quarter of tensor memory), which halves the length of the serial
// load -> max -> exponentiate -> pack chain that separates a tile's score product from its P V product. Row maxima and
// row sums cross the pair through one shared-memory slot per row and a 64-thread named barrier.
template <typename T, int SPLIT>
__global__ void __launch_bounds__(128 + 256 * SPLIT, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const __grid_constant__ CUtensorMap map_o, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* smem_q = smem;                                   // [tile][half][128 rows][128 B]
    uint8_t* smem_p = smem + kTilesPerCta * kTileBytes;       // [tile][half][128 rows][128 B]
    uint8_t* smem_kv = smem + 2 * kTilesPerCta * kTileBytes;  // [slot][half][128 rows][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 * kTilesPerCta + kRing) * kTileBytes);
    uint64_t* q_full = bars;               // [1]
    uint64_t* kv_full = bars + 1;          // [kRing] producer -> MMA
    uint64_t* kv_empty = bars + 1 + kRing; // [kRing] MMA -> producer
    uint64_t* s_full = bars + 1 + 2 * kRing;   // [2] MMA -> softmax: scores of the block are in TMEM
    uint64_t* p_full = s_full + 2;             // [2] softmax -> MMA: P is in shared memory, S may be overwritten
    uint64_t* pv_done = p_full + 2;            // [2] MMA -> softmax: O holds the block, P may be overwritten
    uint64_t* s_free = pv_done + 2;            // [2] softmax -> MMA: the scores are in registers, S may be overwritten
    uint64_t* turn = s_free + 2;               // [4 quarters][2] softmax warp -> its partner of the other tile: exponentials done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(turn + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);      // [tile][128 rows]: pair exchange (SPLIT = 2)
    volatile uint8_t* xfail = reinterpret_cast<uint8_t*>(bars) + 256 + 1024;            // [tile][128 rows]: a wait of the pair failed

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // heavy (late) query blocks of a head first; the blocks of one head are neighbours so that its K / V stay in L2
    const int bh = blockIdx.x / p.q_blocks;
    const int qb = p.q_blocks - 1 - (blockIdx.x - bh * p.q_blocks);
    const int b = bh / p.Hq;
    const int h = bh - b * p.Hq;
    const int hk = h / (p.Hq / p.Hkv);
    const int q0 = qb * (kTilesPerCta * kTileQ);
    const int n0 = blocks_of_tile(p, q0);
    const int n1 = blocks_of_tile(p, q0 + kTileQ);
    const int nmax = max(n0, n1);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kRing; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 2);  // one arrival per Q tile (a tile that is alone on a block arrives twice)
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], 4 * SPLIT);  // one arrival per softmax warp of the tile
            mbar_init(&pv_done[t], 1);
            mbar_init(&s_free[t], 4 * SPLIT);
        }
        for (int i = 0; i < 8; ++i) mbar_init(&turn[i], 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        prefetch_tensormap(&map_o);
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    if (threadIdx.x < 256) xfail[threadIdx.x] = 0;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, kTilesPerCta * kTileBytes);
            for (int t = 0; t < kTilesPerCta; ++t) {
                for (int g = 0; g < 2; ++g) {
                    // rows beyond Sq are filled with zeros by the copy engine
                    const int row = q0 + t * kTileQ;
                    tma_load_4d(smem_q + t * kTileBytes + g * kHalfBytes, &map_q, q_full, g * 64, p.q_hfirst ? h : row, p.q_hfirst ? row : h, b);
                }
            }
            // Order: K0, then for every block i: K(i+1) if there is one, V(i). The keys run a block ahead of the values because
            // a tile's next score product is issued as soon as its softmax has read the current scores out of tensor memory,
            // long before the probabilities for the current values are ready.
            for (int r = 0; r < 2 * nmax; ++r) {
                const int slot = r % kRing;
                const uint32_t phase = static_cast<uint32_t>(r / kRing) & 1u;
                if (!mbar_wait(&kv_empty[slot], phase ^ 1u, abort_flag)) break;
                mbar_arrive_expect_tx(&kv_full[slot], kTileBytes);
                const bool is_v = r == 2 * nmax - 1 || (r != 0 && (r & 1) == 0);
                const int blk = is_v ? (r == 2 * nmax - 1 ? nmax - 1 : (r - 2) / 2) : (r + 1) / 2;
                const CUtensorMap* m = is_v ? &map_v : &map_k;
                const int hfirst = is_v ? p.v_hfirst : p.k_hfirst;
                const int row = blk * kBlockKv;
                for (int g = 0; g < 2; ++g) {
                    tma_load_4d(smem_kv + slot * kTileBytes + g * kHalfBytes, m, &kv_full[slot], g * 64, hfirst ? hk : row, hfirst ? row : hk, b);
                }
            }
        }
    } else if (warp == 1 || warp == 3) {
        // ---------------- MMA issuers: warp 1 for Q tile 0, warp 3 for Q tile 1 ----------------
        // tcgen05.mma keeps the issuing thread until the product has been taken by the tensor core, so one thread issuing for
        // both tiles also serialises its own bookkeeping (barrier polls, commits) with the products. With one issuer per
        // tile the bookkeeping of one overlaps the products of the other. Per tile and block j: S(j+1) goes as soon as the
        // softmax warps have pulled S(j) into registers (s_free) and K(j+1) has landed - the next scores are computed while
        // the softmax is still exponentiating the current ones; P V(j) goes when the probabilities are in shared memory
        // (p_full) and V(j) has landed. Every K / V slot gets two arrivals, one per tile.
        if (lane == 0) {
            const int t = warp == 1 ? 0 : 1;
            const int n_t = t == 0 ? n0 : n1;
            const int n_o = t == 0 ? n1 : n0;
            // Q is always waited for, also when no block is visible: no copy may still be in flight when the CTA ends
            bool ok = mbar_wait(q_full, 0, abort_flag) && n_t > 0;
            auto issue_s = [&](int slot) {
                const uint32_t qa = smem_u32(smem_q + t * kTileBytes);
                const uint32_t ka = smem_u32(smem_kv + slot * kTileBytes);
#pragma unroll
                for (int k = 0; k < kHeadDim / 16; ++k) {
                    const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
                    umma_f16_ss(tmem_base + t * 128, make_smem_desc_sw128(qa + off, 16, 1024), make_smem_desc_sw128(ka + off, 16, 1024), p.idesc_s,
                                k != 0 ? 1u : 0u);
                }
            };
            auto issue_pv = [&](int slot, bool accumulate) {
                const uint32_t pa = smem_u32(smem_p + t * kTileBytes);
                const uint32_t va = smem_u32(smem_kv + slot * kTileBytes);
#pragma unroll
                for (int k = 0; k < kBlockKv / 16; ++k) {
                    // V is N-contiguous: 16 keys are 16 rows of 128 bytes; the two 64-column halves lie kHalfBytes apart
                    umma_f16_ss(tmem_base + 256 + t * 128, make_smem_desc_sw128(pa + (k >> 2) * kHalfBytes + (k & 3) * 32, 16, 1024),
                                make_smem_desc_sw128(va + k * 2048, kHalfBytes, 1024), p.idesc_pv, (accumulate || k != 0) ? 1u : 0u);
                }
            };
            // hands block j's slot back: once for this tile, once more for the other tile if it never visits block j
            auto release = [&](int slot, int j) {
                umma_commit(&kv_empty[slot]);
                if (n_o <= j) umma_commit(&kv_empty[slot]);
            };
            auto scores = [&](int j) -> bool {
                const int r = load_of_k(j);
                if (j > 0 && !mbar_wait(&s_free[t], static_cast<uint32_t>(j - 1) & 1u, abort_flag)) return false;
                if (!mbar_wait(&kv_full[r % kRing], static_cast<uint32_t>(r / kRing) & 1u, abort_flag)) return false;
                tc_fence_after();
                issue_s(r % kRing);
                umma_commit(&s_full[t]);
                release(r % kRing, j);
                return true;
            };
            if (ok) ok = scores(0);
            for (int j = 0; j < n_t && ok; ++j) {
                if (j + 1 < n_t && !scores(j + 1)) { ok = false; break; }
                const int r = load_of_v(j, nmax);
                if (!mbar_wait(&p_full[t], static_cast<uint32_t>(j) & 1u, abort_flag)) { ok = false; break; }
                if (!mbar_wait(&kv_full[r % kRing], static_cast<uint32_t>(r / kRing) & 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                issue_pv(r % kRing, j > 0);
                umma_commit(&pv_done[t]);
                release(r % kRing, j);
            }
        }
    } else if (warp >= 4) {
        // ---------------- softmax + output (SPLIT threads per query row) ----------------
        constexpr int COLS = 128 / SPLIT;   // score columns per thread
        constexpr int NCH = COLS / 32;      // 32-column TMEM chunks per thread
        const int t = (warp - 4) / (4 * SPLIT);
        const int half = ((warp - 4) % (4 * SPLIT)) >> 2;   // which column half of the row (always 0 with one thread per row)
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are the ones this warp may touch
        const int coff = half * COLS;
        const int r_in_tile = quarter * 32 + lane;
        const int q_lo = q0 + t * kTileQ;
        const int q_row = q_lo + r_in_tile;
        const int n_t = t == 0 ? n0 : n1;
        const int k_visible = p.causal ? min(p.Skv - 1, q_row + p.causal_off) : p.Skv - 1;  // last key this row may see
        uint8_t* pbuf = smem_p + t * kTileBytes;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t s_tmem = lane_base + t * 128 + coff;
        const uint32_t o_tmem = lane_base + 256 + t * 128 + coff;
        float* slot = xch + t * 128 + r_in_tile;
        volatile uint8_t* fail = xfail + t * 128 + r_in_tile;
        const int bar_id = 1 + t * 4 + quarter;
        const float neg_inf = -INFINITY;
        float m_used = neg_inf;
        float l_sum = 0.f;   // this thread's columns only
        bool ok = true;
        // Combines a per-row value of the two threads of a row (SPLIT = 2): the upper half deposits, the lower half combines
        // and publishes, two named barriers order the three steps. A failed wait on either side is voted through `fail`,
        // so that both warps of the pair leave their loops together and nobody is left behind at a barrier.
        auto pair_combine = [&](float v, bool is_max, bool my_ok) -> float {
            if (SPLIT == 1) return v;
            if (!my_ok) *fail = 1;
            if (half == 1) *slot = v;
            pair_barrier(bar_id, 64);
            float r = v;
            if (half == 0) {
                const float o = *slot;
                r = is_max ? fmaxf(v, o) : v + o;
                *slot = r;
            }
            pair_barrier(bar_id, 64);
            if (half == 1) r = *slot;
            return r;
        };
        for (int j = 0; j < n_t; ++j) {
            bool my_ok = mbar_wait(&s_full[t], static_cast<uint32_t>(j) & 1u, abort_flag);
            my_ok = __all_sync(0xffffffffu, my_ok);
            if (SPLIT == 1 && !my_ok) {
                ok = false;
                break;
            }
            tc_fence_after();
            uint32_t s[NCH][32];
#pragma unroll
            for (int c = 0; c < NCH; ++c) tmem_ld_32x32(s_tmem + c * 32, s[c]);
            tmem_ld_wait();
            // the scores are in registers: the tensor core may write the next block's scores over them right away
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[t]);
            const int k0 = j * kBlockKv;
            // warp-uniform: does any element of this tile x block need the mask?
            const bool need_mask = (k0 + kBlockKv > p.Skv) || (p.causal && k0 + kBlockKv - 1 > q_lo + p.causal_off);
            // Row maximum of the RAW scores (the scale is positive, so it commutes with the maximum); four independent
            // running maxima: with few softmax warps per scheduler there is little else to hide a long dependent chain
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (k0 + coff + c * 32 + i > k_visible) s[c][i] = __float_as_uint(neg_inf);
                    }
                }
            }
            float mxs[4] = {neg_inf, neg_inf, neg_inf, neg_inf};
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
#pragma unroll
                for (int i = 0; i < 32; ++i) mxs[i & 3] = fmaxf(mxs[i & 3], __uint_as_float(s[c][i]));
            }
            const float mx_own = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
            const float mx = pair_combine(mx_own, true, my_ok) * p.scale_log2;  // -inf stays -inf
            if (SPLIT == 2) {
                const bool pair_ok = __all_sync(0xffffffffu, *fail == 0);   // the same rows in both warps: the same answer
                if (!pair_ok) {
                    ok = false;
                    break;
                }
            }
            // The running maximum only moves when some row of the warp outgrew it by more than the threshold: P stays
            // below 2^8 and most blocks need no pass over O. Both threads of a row see the same maxima, hence decide alike.
            bool rescale = false;
            float factor = 1.f;
            if (j == 0) {
                m_used = mx;
            } else {
                rescale = __any_sync(0xffffffffu, mx > m_used + kRescaleThreshold);
                if (rescale) {
                    const float m_new = fmaxf(m_used, mx);
                    factor = (m_used == neg_inf) ? 0.f : fast_exp2(m_used - m_new);
                    m_used = m_new;
                    l_sum *= factor;
                }
            }
            const float base = (m_used == neg_inf) ? 0.f : m_used;
            float parts[4] = {0.f, 0.f, 0.f, 0.f};
            // The two warps of a scheduler (same quarter, one per tile) take turns at the exponentials: the special-function
            // unit serves 4 lanes per cycle, so two warps exponentiating at once both crawl and then both sit in the phases
            // that need no such unit (score load, maximum, P store, barriers). In turns, one warp's other phases hide behind
            // its partner's exponentials. Order: tile 0 block j, tile 1 block j, tile 0 block j + 1, ... as far as both exist.
            if (SPLIT == 1) {
                bool go = true;
                if (t == 0) {
                    if (j > 0 && j - 1 < n1) go = mbar_wait(&turn[quarter * 2 + 0], static_cast<uint32_t>(j - 1) & 1u, abort_flag);
                } else {
                    if (j < n0) go = mbar_wait(&turn[quarter * 2 + 1], static_cast<uint32_t>(j) & 1u, abort_flag);
                }
                go = __all_sync(0xffffffffu, go);
                if (!go) {
                    ok = false;
                    break;
                }
            }
            // exponentials first, packed in place (two probabilities per register): nothing here needs the previous block's
            // P V product, which is still running
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    float e[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        // scale and shift in one FMA: exp2(s * scale * log2(e) - m)
                        e[u] = fast_exp2(fmaf(__uint_as_float(s[c][i + u]), p.scale_log2, -base));
                        parts[u & 3] += e[u];
                    }
                    s[c][i / 2 + 0] = pack2<T>(e[0], e[1]);
                    s[c][i / 2 + 1] = pack2<T>(e[2], e[3]);
                    s[c][i / 2 + 2] = pack2<T>(e[4], e[5]);
                    s[c][i / 2 + 3] = pack2<T>(e[6], e[7]);
                }
            }
            if (SPLIT == 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&turn[quarter * 2 + (t == 0 ? 1 : 0)]);
            }
            // P of the previous block has been consumed and O is at rest once that block's P V product is complete
            if (j > 0) {
                bool done = mbar_wait(&pv_done[t], static_cast<uint32_t>(j - 1) & 1u, abort_flag);
                done = __all_sync(0xffffffffu, done);
                if (SPLIT == 2) {
                    // both warps of a row pair must leave together: vote through the shared flag
                    if (!done) *fail = 1;
                    pair_barrier(bar_id, 64);
                    done = __all_sync(0xffffffffu, *fail == 0);
                }
                if (!done) {
                    ok = false;
                    break;
                }
                tc_fence_after();
            }
            if (rescale) {
#pragma unroll 1
                for (int c = 0; c < NCH; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32(o_tmem + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                    tmem_st_32x32(o_tmem + c * 32, o);
                }
                tmem_st_wait();
            }
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 w;
                    w.x = s[c][i / 2 + 0];
                    w.y = s[c][i / 2 + 1];
                    w.z = s[c][i / 2 + 2];
                    w.w = s[c][i / 2 + 3];
                    // 16-byte chunk `chunk` of the row sits at position chunk ^ (row & 7): the 128-byte swizzle of a
                    // K-major tensor-core operand; columns 0..63 and 64..127 are separate 16 KiB halves
                    const int col = coff + c * 32 + i;
                    const int chunk = (col & 63) >> 3;
                    *reinterpret_cast<uint4*>(pbuf + (col >> 6) * kHalfBytes + r_in_tile * 128 + ((chunk ^ (r_in_tile & 7)) * 16)) = w;
                }
            }
            l_sum += (parts[0] + parts[1]) + (parts[2] + parts[3]);
            fence_proxy_async();  // generic-proxy writes of P -> visible to the tensor core's reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[t]);
        }

        // ---- normalise and store this warp's 32 rows (its column half with two threads per row) ----
        if (ok && q_lo + quarter * 32 < p.Sq) {
            bool my_ok = true;
            if (n_t > 0) {
                my_ok = mbar_wait(&pv_done[t], static_cast<uint32_t>(n_t - 1) & 1u, abort_flag);
                my_ok = __all_sync(0xffffffffu, my_ok);
            }
            const float l_row = pair_combine(l_sum, false, my_ok);
            if (SPLIT == 2) my_ok = __all_sync(0xffffffffu, *fail == 0);
            if (my_ok) {
                tc_fence_after();
                const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
#pragma unroll 1
                for (int c = 0; c < NCH; ++c) {
                    uint32_t o[32];
                    if (n_t > 0) {
                        tmem_ld_32x32(o_tmem + c * 32, o);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = 0u;
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack2<T>(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
                        w.y = pack2<T>(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                        w.z = pack2<T>(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                        w.w = pack2<T>(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                        const int col = coff + c * 32 + i;
                        const int chunk = (col & 63) >> 3;
                        *reinterpret_cast<uint4*>(pbuf + (col >> 6) * kHalfBytes + r_in_tile * 128 + ((chunk ^ (r_in_tile & 7)) * 16)) = w;
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    const int g_begin = SPLIT == 2 ? half : 0, g_end = SPLIT == 2 ? half + 1 : 2;
                    for (int g = g_begin; g < g_end; ++g) {
                        // rows beyond Sq are clipped by the copy engine
                        const int row = q_lo + quarter * 32;
                        tma_store_4d(&map_o, pbuf + g * kHalfBytes + quarter * (32 * 128), g * 64, p.o_hfirst ? h : row, p.o_hfirst ? row : h, b);
                    }
                    tma_store_commit();
                }
                if (p.lse != nullptr && q_row < p.Sq && half == 0) {
                    const float lse = l_row > 0.f ? m_used * 0.6931471805599453f + logf(l_row) : neg_inf;
                    p.lse[static_cast<int64_t>(b) * p.lse_sb + static_cast<int64_t>(h) * p.lse_sh + static_cast<int64_t>(q_row) * p.lse_sq] = lse;
                }
                if (lane == 0) tma_store_wait_all<0>();
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag != 0) {
        // A wait timed out. Give copies and products that are still in flight time to land before shared and tensor
        // memory are released, then report.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0) atomicExch(p.status, 2u);
    }
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, 512);
}


template <typename T, int SPLIT>
cudaError_t launch_prefill_split(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, const AttnParams& p,
                                 int grid, cudaStream_t stream) {
    if (cudaError_t e = tc_ensure_smem_attr(reinterpret_cast<const void*>(attn_prefill_kernel<T, SPLIT>), kAttnSmem); e != cudaSuccess) return e;
    attn_prefill_kernel<T, SPLIT><<<grid, 128 + 256 * SPLIT, kAttnSmem, stream>>>(mq, mk, mv, mo, p);
    return cudaPeekAtLastError();
}

template <typename T>
cudaError_t launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, const AttnParams& p, int grid,
                           cudaStream_t stream) {
    // One thread per row is the default. Two threads per row (B200_ATTN_ROW_SPLIT=2) halve the per-thread work, but measured
    // slower (7B causal prefill 0.62 against 0.38 ms): twenty warps at 96 registers spill, and the two named barriers per block
    // cost more than the shorter chain saves.
    static const bool two_threads = [] {
        const char* e = std::getenv("B200_ATTN_ROW_SPLIT");
        return e != nullptr && e[0] == '2';
    }();
    return two_threads ? launch_prefill_split<T, 2>(mq, mk, mv, mo, p, grid, stream) : launch_prefill_split<T, 1>(mq, mk, mv, mo, p, grid, stream);
}

// [B, S, H, D] view -> 4-D tensor map with a 64-column x box_rows-row box. The driver wants every pitch to be a
// multiple of the one before it, so the head and row dimensions are ordered by pitch; *hfirst tells the kernel which
// coordinate order the map expects.
bool map_of(const TensorView& t, int box_rows, CUtensorMap* map, int* hfirst) {
    const int64_t d = t.shape[3];
    // the pitch of a size-1 dimension never addresses anything; give it the dense value so that it stays a valid multiple
    const int64_t ps = t.shape[1] == 1 ? (t.shape[2] == 1 ? d : t.stride[2] * t.shape[2]) : t.stride[1];
    const int64_t ph = t.shape[2] == 1 ? (t.shape[1] == 1 ? d : t.stride[1] * t.shape[1]) : t.stride[2];
    const bool hf = ph <= ps;
    *hfirst = hf ? 1 : 0;
    const int64_t inner_extent = hf ? ps * t.shape[1] : ph * t.shape[2];
    const int64_t pb = t.shape[0] == 1 ? inner_extent : t.stride[0];
    const int64_t dims[4] = {d, hf ? t.shape[2] : t.shape[1], hf ? t.shape[1] : t.shape[2], t.shape[0]};
    const int64_t pitches[3] = {hf ? ph : ps, hf ? ps : ph, pb};
    return tc_encode_map4(reinterpret_cast<::CUtensorMap_st*>(map), t.dtype, t.data, dims, pitches, hf ? 1 : box_rows, hf ? box_rows : 1);
}

bool tma_viewable(const TensorView& t) {
    if (t.ndim != 4 || t.stride[3] != 1 || !t.aligned(16)) return false;
    for (int d = 0; d < 3; ++d) {
        if (t.shape[d] == 1) continue;
        if (t.stride[d] <= 0 || (t.stride[d] * 2) % 16 != 0 || t.stride[d] * 2 >= (1ll << 40)) return false;
    }
    return true;
}

}  // namespace

// The 512 tensor-memory columns and ~225 KiB of shared memory a CTA takes leave room for one CTA per SM.
diopiError_t attention_prefill_launch(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out, const TensorView* lse,
                                      bool causal, double scale, cudaStream_t stream) {
    AttnParams p = {};
    p.B = static_cast<int>(q.shape[0]);
    p.Sq = static_cast<int>(q.shape[1]);
    p.Hq = static_cast<int>(q.shape[2]);
    p.Skv = static_cast<int>(k.shape[1]);
    p.Hkv = static_cast<int>(k.shape[2]);
    p.q_blocks = (p.Sq + kTilesPerCta * kTileQ - 1) / (kTilesPerCta * kTileQ);
    p.causal = causal ? 1 : 0;
    p.causal_off = p.Skv - p.Sq;
    p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
    const int fmt = q.dtype == diopi_dtype_bfloat16 ? 1 : 0;
    p.idesc_s = make_idesc_f16(fmt, false, kTileQ, kBlockKv);
    p.idesc_pv = make_idesc_f16(fmt, true, kTileQ, kHeadDim);
    if (lse != nullptr) {
        p.lse = static_cast<float*>(lse->data);
        p.lse_sb = lse->stride[0];
        p.lse_sh = lse->stride[1];
        p.lse_sq = lse->stride[2];
    }
    p.status = tc_status_word();
    B200_CHECK(p.status != nullptr, "attention: cannot allocate the status word");
    CUtensorMap mq, mk, mv, mo;
    B200_CHECK(map_of(q, kTileQ, &mq, &p.q_hfirst) && map_of(k, kBlockKv, &mk, &p.k_hfirst) && map_of(v, kBlockKv, &mv, &p.v_hfirst) &&
                   map_of(out, 32, &mo, &p.o_hfirst),
               "attention: cuTensorMapEncodeTiled rejected an operand (pitches must be 16-byte multiples of one another)");
    const int64_t grid = static_cast<int64_t>(p.B) * p.Hq * p.q_blocks;
    B200_CHECK(grid > 0 && grid < 0x7fffffffLL, "attention: grid out of range");
    cudaError_t e = q.dtype == diopi_dtype_bfloat16 ? launch_prefill<__nv_bfloat16>(mq, mk, mv, mo, p, static_cast<int>(grid), stream)
                                                   : launch_prefill<__half>(mq, mk, mv, mo, p, static_cast<int>(grid), stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        B200_FAIL("attention: kernel launch failed: %s", cudaGetErrorString(e));
    }
    return diopiSuccess;
}

bool attention_prefill_applies(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out) {
    if (!(q.dtype == diopi_dtype_bfloat16 || q.dtype == diopi_dtype_float16)) return false;
    if (k.dtype != q.dtype || v.dtype != q.dtype || out.dtype != q.dtype) return false;
    if (!tma_viewable(q) || !tma_viewable(k) || !tma_viewable(v) || !tma_viewable(out)) return false;
    if (q.shape[3] != kHeadDim) return false;
    return true;
}

}  // namespace b200

// ---- decode: one query row per (batch, head) against a long key / value cache ------------------------------------------------
// Bound by reading K and V once from HBM (2 * Skv * 256 bytes per K/V head); the arithmetic is a few flop per byte, so it
// runs on the CUDA cores with every load a full 16-byte vector. This is the fused form of
// dicp/dicp/vendor/AscendGraph/ext_ops.py:89-126 (flash_attention_inference: bmm, / sqrt(d), softmax, bmm per sequence).
//
// A CTA owns one (batch, K/V head, slice of keys) and up to GT query heads of the group that shares that K/V head.
// Eight lanes cover one key row (16 elements = 32 bytes each), so a warp handles four keys per step and the CTA's eight
// warps 32; each lane keeps a running maximum, denominator and a 16-column slice of the output per head, merged across
// lanes (shuffles) and warps (shared memory) at the end. With more than one key slice the partial results go to a
// workspace and a second kernel merges them.
namespace b200 {
namespace {

constexpr int kDecThreads = 256;
constexpr int kDecKeysPerStep = 32;   // 8 warps x 4 keys

struct DecodeParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    int64_t q_sb, q_sh;            // element pitches
    int64_t k_sb, k_ss, k_sh;
    int64_t v_sb, v_ss, v_sh;
    int64_t o_sb, o_sh;
    int Hq, Hkv, group;            // group = Hq / Hkv
    int Skv;
    int splits, keys_per_split;    // keys_per_split is a multiple of kDecKeysPerStep
    float scale_log2;
    float* part;                   // [B * Hq, splits, 130] (m, l, 128 columns) when splits > 1
    float* lse;                    // optional
    int64_t lse_sb, lse_sh;
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& w, float (&f)[8]) {
    // bf16 -> fp32 is a 16-bit shift
    f[0] = __uint_as_float(w.x << 16); f[1] = __uint_as_float(w.x & 0xffff0000u);
    f[2] = __uint_as_float(w.y << 16); f[3] = __uint_as_float(w.y & 0xffff0000u);
    f[4] = __uint_as_float(w.z << 16); f[5] = __uint_as_float(w.z & 0xffff0000u);
    f[6] = __uint_as_float(w.w << 16); f[7] = __uint_as_float(w.w & 0xffff0000u);
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& w, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ uint4 ldg16_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// Merge (m_b, l_b, acc_b) into (m_a, l_a, acc_a): two partial softmax results over disjoint key sets.
template <int N>
__device__ __forceinline__ void merge_partial(float& m_a, float& l_a, float (&acc_a)[N], float m_b, float l_b, const float (&acc_b)[N]) {
    const float m = fmaxf(m_a, m_b);
    const float fa = (m_a == -INFINITY) ? 0.f : fast_exp2(m_a - m);
    const float fb = (m_b == -INFINITY) ? 0.f : fast_exp2(m_b - m);
    l_a = l_a * fa + l_b * fb;
#pragma unroll
    for (int i = 0; i < N; ++i) acc_a[i] = acc_a[i] * fa + acc_b[i] * fb;
    m_a = m;
}

template <typename T, int GT, int U>
__global__ void __launch_bounds__(kDecThreads) attn_decode_kernel(const DecodeParams p) {
    grid_launch_dependents();   // the product that follows may set itself up meanwhile (gemm_tc.cu, launch_splitk)
    __shared__ float red[8][GT][130];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int sub = lane >> 3;   // which of the warp's four keys
    const int col = lane & 7;    // 16-column slice of the row
    const int head_tiles = p.group / GT;
    int idx = blockIdx.x;
    const int ht = idx % head_tiles;
    idx /= head_tiles;
    const int hk = idx % p.Hkv;
    const int b = idx / p.Hkv;
    const int h0 = hk * p.group + ht * GT;
    const int split = blockIdx.y;
    const int key_begin = split * p.keys_per_split;
    const int key_end = min(p.Skv, key_begin + p.keys_per_split);

    float qf[GT][16];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        const T* qrow = static_cast<const T*>(p.q) + static_cast<int64_t>(b) * p.q_sb + static_cast<int64_t>(h0 + g) * p.q_sh + col * 16;
        float lo[8], hi[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(qrow), lo);
        unpack8<T>(*reinterpret_cast<const uint4*>(qrow + 8), hi);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            qf[g][i] = lo[i] * p.scale_log2;
            qf[g][8 + i] = hi[i] * p.scale_log2;
        }
    }
    float m_run[GT], l_run[GT], acc[GT][16];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m_run[g] = -INFINITY;
        l_run[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[g][i] = 0.f;
    }
    const T* kbase = static_cast<const T*>(p.k) + static_cast<int64_t>(b) * p.k_sb + static_cast<int64_t>(hk) * p.k_sh + col * 16;
    const T* vbase = static_cast<const T*>(p.v) + static_cast<int64_t>(b) * p.v_sb + static_cast<int64_t>(hk) * p.v_sh + col * 16;

    // the loop bound is warp-uniform (the shuffles below need the whole warp); lanes past the end are masked
    for (int base0 = key_begin + warp * 4; base0 < key_end; base0 += kDecKeysPerStep * U) {
        const int key0 = base0 + sub;
        uint4 kw[U][2], vw[U][2];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int key = key0 + u * kDecKeysPerStep;
            const int kc = min(key, key_end - 1);  // clamp: rows past the end are loaded from a valid address and masked
            const T* kr = kbase + static_cast<int64_t>(kc) * p.k_ss;
            kw[u][0] = ldg16_stream(kr);
            kw[u][1] = ldg16_stream(kr + 8);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int key = key0 + u * kDecKeysPerStep;
            const int kc = min(key, key_end - 1);
            const T* vr = vbase + static_cast<int64_t>(kc) * p.v_ss;
            vw[u][0] = ldg16_stream(vr);
            vw[u][1] = ldg16_stream(vr + 8);
        }
        float sc[U][GT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float kf[16];
            {
                float lo[8], hi[8];
                unpack8<T>(kw[u][0], lo);
                unpack8<T>(kw[u][1], hi);
#pragma unroll
                for (int i = 0; i < 8; ++i) { kf[i] = lo[i]; kf[8 + i] = hi[i]; }
            }
            const bool valid = key0 + u * kDecKeysPerStep < key_end;
#pragma unroll
            for (int g = 0; g < GT; ++g) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) d = fmaf(qf[g][i], kf[i], d);
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                sc[u][g] = valid ? d : -INFINITY;
            }
        }
        float pr[U][GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            float mx = sc[0][g];
#pragma unroll
            for (int u = 1; u < U; ++u) mx = fmaxf(mx, sc[u][g]);
            const float m_new = fmaxf(m_run[g], mx);
            const float base = (m_new == -INFINITY) ? 0.f : m_new;
            const float factor = (m_run[g] == -INFINITY) ? 0.f : fast_exp2(m_run[g] - base);
            m_run[g] = m_new;
            float add = 0.f;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                pr[u][g] = fast_exp2(sc[u][g] - base);
                add += pr[u][g];
            }
            l_run[g] = l_run[g] * factor + add;
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[g][i] *= factor;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float vf[16];
            {
                float lo[8], hi[8];
                unpack8<T>(vw[u][0], lo);
                unpack8<T>(vw[u][1], hi);
#pragma unroll
                for (int i = 0; i < 8; ++i) { vf[i] = lo[i]; vf[8 + i] = hi[i]; }
            }
#pragma unroll
            for (int g = 0; g < GT; ++g) {
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[g][i] = fmaf(pr[u][g], vf[i], acc[g][i]);
            }
        }
    }

    // ---- merge the four key sub-groups of the warp (lanes 8 and 16 apart hold the same columns) ----
#pragma unroll
    for (int g = 0; g < GT; ++g) {
#pragma unroll
        for (int off = 8; off <= 16; off <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m_run[g], off);
            const float l_o = __shfl_xor_sync(0xffffffffu, l_run[g], off);
            float a_o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) a_o[i] = __shfl_xor_sync(0xffffffffu, acc[g][i], off);
            merge_partial<16>(m_run[g], l_run[g], acc[g], m_o, l_o, a_o);
        }
        if (sub == 0) {
            if (col == 0) {
                red[warp][g][0] = m_run[g];
                red[warp][g][1] = l_run[g];
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) red[warp][g][2 + col * 16 + i] = acc[g][i];
        }
    }
    __syncthreads();
    // ---- merge the eight warps: one thread per (head, column) ----
    for (int item = threadIdx.x; item < GT * 128; item += kDecThreads) {
        const int g = item >> 7;
        const int c = item & 127;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 8; ++w) m = fmaxf(m, red[w][g][0]);
        float l = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float mw = red[w][g][0];
            const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
            l += red[w][g][1] * f;
            a += red[w][g][2 + c] * f;
        }
        const int h = h0 + g;
        if (p.splits == 1) {
            T* orow = static_cast<T*>(p.out) + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(h) * p.o_sh;
            orow[c] = from_f32<T>(l > 0.f ? a / l : 0.f);
            if (c == 0 && p.lse != nullptr) {
                p.lse[static_cast<int64_t>(b) * p.lse_sb + static_cast<int64_t>(h) * p.lse_sh] = l > 0.f ? m * 0.6931471805599453f + logf(l) : -INFINITY;
            }
        } else {
            float* dst = p.part + (static_cast<int64_t>(b * p.Hq + h) * p.splits + split) * 130;
            if (c == 0) {
                dst[0] = m;
                dst[1] = l;
            }
            dst[2 + c] = a;
        }
    }
}

// Merges the key slices of one (batch, head): 128 threads, one per output column.
template <typename T>
__global__ void __launch_bounds__(128) attn_decode_merge_kernel(const DecodeParams p) {
    grid_launch_dependents();   // the product that follows may set itself up meanwhile (gemm_tc.cu, launch_splitk)
    const int bh = blockIdx.x;
    const int b = bh / p.Hq;
    const int h = bh - b * p.Hq;
    const int c = threadIdx.x;
    const float* src = p.part + static_cast<int64_t>(bh) * p.splits * 130;
    float m = -INFINITY;
    for (int s = 0; s < p.splits; ++s) m = fmaxf(m, src[s * 130]);
    float l = 0.f, a = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        const float ms = src[s * 130];
        const float f = (ms == -INFINITY) ? 0.f : fast_exp2(ms - m);
        l += src[s * 130 + 1] * f;
        a += src[s * 130 + 2 + c] * f;
    }
    T* orow = static_cast<T*>(p.out) + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(h) * p.o_sh;
    orow[c] = from_f32<T>(l > 0.f ? a / l : 0.f);
    if (c == 0 && p.lse != nullptr) {
        p.lse[static_cast<int64_t>(b) * p.lse_sb + static_cast<int64_t>(h) * p.lse_sh] = l > 0.f ? m * 0.6931471805599453f + logf(l) : -INFINITY;
    }
}

template <typename T>
void launch_decode(const DecodeParams& p, int gt, int batch, dim3 grid, cudaStream_t stream) {
    switch (gt) {
        case 4: attn_decode_kernel<T, 4, 2><<<grid, kDecThreads, 0, stream>>>(p); break;
        case 2: attn_decode_kernel<T, 2, 4><<<grid, kDecThreads, 0, stream>>>(p); break;
        default: attn_decode_kernel<T, 1, 4><<<grid, kDecThreads, 0, stream>>>(p); break;
    }
    if (p.splits > 1) attn_decode_merge_kernel<T><<<p.Hq * batch, 128, 0, stream>>>(p);
}

bool rows_viewable(const TensorView& t) {
    if (t.ndim != 4 || t.stride[3] != 1 || !t.aligned(16)) return false;
    for (int d = 0; d < 3; ++d) {
        if (t.shape[d] != 1 && (t.stride[d] < 0 || (t.stride[d] * 2) % 16 != 0)) return false;
    }
    return true;
}

}  // namespace

bool attention_decode_applies(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out) {
    if (!(q.dtype == diopi_dtype_bfloat16 || q.dtype == diopi_dtype_float16)) return false;
    if (k.dtype != q.dtype || v.dtype != q.dtype || out.dtype != q.dtype) return false;
    if (q.shape[1] != 1 || q.shape[3] != 128) return false;
    return rows_viewable(q) && rows_viewable(k) && rows_viewable(v) && rows_viewable(out);
}

diopiError_t attention_decode_launch(diopiContextHandle_t ctx, const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out,
                                     const TensorView* lse, double scale, cudaStream_t stream) {
    DecodeParams p = {};
    p.q = q.data; p.k = k.data; p.v = v.data; p.out = out.data;
    p.q_sb = q.stride[0]; p.q_sh = q.stride[2];
    p.k_sb = k.stride[0]; p.k_ss = k.stride[1]; p.k_sh = k.stride[2];
    p.v_sb = v.stride[0]; p.v_ss = v.stride[1]; p.v_sh = v.stride[2];
    p.o_sb = out.stride[0]; p.o_sh = out.stride[2];
    const int B = static_cast<int>(q.shape[0]);
    p.Hq = static_cast<int>(q.shape[2]);
    p.Hkv = static_cast<int>(k.shape[2]);
    p.group = p.Hq / p.Hkv;
    p.Skv = static_cast<int>(k.shape[1]);
    p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
    if (lse != nullptr) {
        p.lse = static_cast<float*>(lse->data);
        p.lse_sb = lse->stride[0];
        p.lse_sh = lse->stride[1];
    }
    const int gt = p.group % 4 == 0 ? 4 : (p.group % 2 == 0 ? 2 : 1);
    const int64_t ctas = static_cast<int64_t>(B) * p.Hkv * (p.group / gt);
    B200_CHECK(ctas > 0 && ctas < 0x7fffffffLL, "attention: grid out of range");
    // enough CTAs for about four per SM, but no slice shorter than 256 keys
    const int sms = sm_count();
    int splits = 1;
    if (ctas < 4 * sms) {
        const int64_t want = (4 * static_cast<int64_t>(sms) + ctas - 1) / ctas;
        const int64_t most = (p.Skv + 255) / 256;
        splits = static_cast<int>(want < most ? want : most);
        if (splits < 1) splits = 1;
        if (splits > 65535) splits = 65535;
    }
    int per = (p.Skv + splits - 1) / splits;
    per = (per + kDecKeysPerStep - 1) / kDecKeysPerStep * kDecKeysPerStep;
    splits = (p.Skv + per - 1) / per;
    p.splits = splits;
    p.keys_per_split = per;
    if (splits > 1) {
        diopiTensorHandle_t ws = nullptr;
        const int64_t bytes = static_cast<int64_t>(B) * p.Hq * splits * 130 * static_cast<int64_t>(sizeof(float));
        B200_CHECK(diopiRequireBuffer(ctx, &ws, bytes, diopi_device) == diopiSuccess && ws != nullptr, "attention: workspace allocation failed");
        void* ptr = nullptr;
        B200_CHECK(diopiGetTensorData(ws, &ptr) == diopiSuccess && ptr != nullptr, "attention: workspace has no data pointer");
        p.part = static_cast<float*>(ptr);
    }
    const dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(splits));
    if (q.dtype == diopi_dtype_bfloat16) launch_decode<__nv_bfloat16>(p, gt, B, grid, stream);
    else launch_decode<__half>(p, gt, B, grid, stream);
    B200_LAUNCH_CHECK("attention decode");
    return diopiSuccess;
}

}  // namespace b200

// q [B, Sq, Hq, D], k / v [B, Skv, Hkv, D], out [B, Sq, Hq, D]; any pitches with a unit innermost one.
extern "C" DIOPI_API diopiError_t diopiMultiHeadAttention(diopiContextHandle_t ctx, diopiTensorHandle_t q, diopiTensorHandle_t k, diopiTensorHandle_t v,
                                                         double dropout_p, bool is_causal, bool return_debug_mask, double scale,
                                                         diopiTensorHandle_t out, diopiTensorHandle_t softmax_lse, diopiGeneratorHandle_t gen,
                                                         diopiTensorHandle_t debug_attn_mask) {
    (void)gen;
    B200_CHECK(dropout_p == 0.0, "diopiMultiHeadAttention: dropout is not supported (inference path), got p=%g", dropout_p);
    B200_CHECK(!return_debug_mask && debug_attn_mask == nullptr, "diopiMultiHeadAttention: the debug mask is not supported");
    B200_VIEW(vq, q);
    B200_VIEW(vk, k);
    B200_VIEW(vv, v);
    B200_VIEW(vo, out);
    B200_CHECK(vq.ndim == 4 && vk.ndim == 4 && vv.ndim == 4 && vo.ndim == 4, "diopiMultiHeadAttention: q, k, v, out must be [batch, seq, heads, dim]");
    B200_CHECK(vq.device == diopi_device && vk.device == diopi_device && vv.device == diopi_device && vo.device == diopi_device,
               "diopiMultiHeadAttention: operands must live on the device");
    for (int d = 0; d < 4; ++d) {
        B200_CHECK(vo.shape[d] == vq.shape[d], "diopiMultiHeadAttention: out must have q's shape");
        B200_CHECK(vk.shape[d] == vv.shape[d], "diopiMultiHeadAttention: k and v must have the same shape");
    }
    B200_CHECK(vk.shape[0] == vq.shape[0] && vk.shape[3] == vq.shape[3], "diopiMultiHeadAttention: k / v batch and head dim must match q");
    B200_CHECK(vk.shape[2] > 0 && vq.shape[2] % vk.shape[2] == 0, "diopiMultiHeadAttention: %lld query heads cannot share %lld key heads",
               static_cast<long long>(vq.shape[2]), static_cast<long long>(vk.shape[2]));
    B200_CHECK(std::isfinite(scale) && scale > 0.0, "diopiMultiHeadAttention: scale must be positive, got %g", scale);
    if (vq.numel == 0) return diopiSuccess;
    B200_CHECK(vk.shape[1] > 0, "diopiMultiHeadAttention: empty key sequence");
    B200_CHECK(vq.shape[1] < (1ll << 30) && vk.shape[1] < (1ll << 30), "diopiMultiHeadAttention: sequence too long");
    b200::TensorView vl;
    const b200::TensorView* lse = nullptr;
    if (softmax_lse != nullptr) {
        if (!b200::make_view(softmax_lse, &vl, "softmax_lse")) return diopiErrorOccurred;
        B200_CHECK(vl.dtype == diopi_dtype_float32 && vl.ndim == 3 && vl.shape[0] == vq.shape[0] && vl.shape[1] == vq.shape[2] &&
                       vl.shape[2] == vq.shape[1],
                   "diopiMultiHeadAttention: softmax_lse must be float32 [batch, heads, seq_q]");
        lse = &vl;
    }
    cudaStream_t stream = b200::stream_of(ctx);
    if (b200::attention_decode_applies(vq, vk, vv, vo)) return b200::attention_decode_launch(ctx, vq, vk, vv, vo, lse, scale, stream);
    B200_CHECK(b200::attention_prefill_applies(vq, vk, vv, vo),
               "diopiMultiHeadAttention: needs bf16 / fp16 operands of one dtype, head dim 128, unit innermost pitch, other pitches "
               "multiples of 8 elements and 16-byte aligned bases");
    return b200::attention_prefill_launch(vq, vk, vv, vo, lse, is_causal, scale, stream);
}
