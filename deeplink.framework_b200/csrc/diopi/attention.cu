// Fused attention for the prefill step: out = softmax(scale * Q K^T + causal mask) V in one kernel, without the
// [heads, Sq, Skv] score tensor ever reaching HBM. This is the fused form of the bmm -> div -> add(mask) -> softmax ->
// bmm sequence of dicp/test/model/llama/model.py:146-150; the reference's own CPU restatement of the fused operator is
// dicp/dicp/vendor/AscendGraph/ext_ops.py:52-86 (prompt_attention_inference: causal, grouped K/V heads).
//
// One CTA per (batch, head, 256 query rows), 384 threads:
//   warp 0       TMA producer: the two 128-row Q tiles once, then K and V blocks of 128 keys through a 3-slot ring
//   warp 1       MMA issuer (one thread): S_t = Q_t K_j^T and O_t += P_t V_j with tcgen05.mma, accumulators in TMEM
//   warp 2       TMEM allocation (512 columns: S_0, S_1, O_0, O_1, 128 fp32 columns each)
//   warps 4..7   softmax of Q tile 0, warps 8..11 of Q tile 1: one thread per query row reads its 128 scores from
//                TMEM, keeps the running maximum and sum, writes P (bf16 / fp16) into swizzled shared memory as the A
//                operand of the second product, and rescales O in TMEM only when the maximum grew by more than 2^8
// The two Q tiles alternate on the tensor core: while one tile's scores are being exponentiated the other tile's
// products run. Causal blocks above the diagonal are skipped; only diagonal blocks pay for the element mask.
// Every wait is bounded (gemm_sm100.cuh); a time-out ends the kernel and is reported through the status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>

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
constexpr int kAttnThreads = 384;
constexpr int kAttnSmem = (kTilesPerCta * 2 + kRing) * kTileBytes + 1024 /*alignment*/ + 256 /*barriers*/;
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

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
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
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

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
            mbar_init(&kv_empty[s], 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], 4);  // one arrival per softmax warp of the tile
            mbar_init(&pv_done[t], 1);
        }
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
            for (int r = 0; r < 2 * nmax; ++r) {
                const int slot = r % kRing;
                const uint32_t phase = static_cast<uint32_t>(r / kRing) & 1u;
                if (!mbar_wait(&kv_empty[slot], phase ^ 1u, abort_flag)) break;
                mbar_arrive_expect_tx(&kv_full[slot], kTileBytes);
                const CUtensorMap* m = (r & 1) ? &map_v : &map_k;
                const int hfirst = (r & 1) ? p.v_hfirst : p.k_hfirst;
                const int row = (r >> 1) * kBlockKv;
                for (int g = 0; g < 2; ++g) {
                    tma_load_4d(smem_kv + slot * kTileBytes + g * kHalfBytes, m, &kv_full[slot], g * 64, hfirst ? hk : row, hfirst ? row : hk, b);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const int nt[2] = {n0, n1};
            // Q is always waited for, also when no block is visible: no copy may still be in flight when the CTA ends
            bool ok = mbar_wait(q_full, 0, abort_flag) && nmax > 0;
            auto issue_s = [&](int t, int slot) {
                const uint32_t qa = smem_u32(smem_q + t * kTileBytes);
                const uint32_t ka = smem_u32(smem_kv + slot * kTileBytes);
#pragma unroll
                for (int k = 0; k < kHeadDim / 16; ++k) {
                    const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
                    umma_f16_ss(tmem_base + t * 128, make_smem_desc_sw128(qa + off, 16, 1024), make_smem_desc_sw128(ka + off, 16, 1024), p.idesc_s,
                                k != 0 ? 1u : 0u);
                }
            };
            auto issue_pv = [&](int t, int slot, bool accumulate) {
                const uint32_t pa = smem_u32(smem_p + t * kTileBytes);
                const uint32_t va = smem_u32(smem_kv + slot * kTileBytes);
#pragma unroll
                for (int k = 0; k < kBlockKv / 16; ++k) {
                    // V is N-contiguous: 16 keys are 16 rows of 128 bytes; the two 64-column halves lie kHalfBytes apart
                    umma_f16_ss(tmem_base + 256 + t * 128, make_smem_desc_sw128(pa + (k >> 2) * kHalfBytes + (k & 3) * 32, 16, 1024),
                                make_smem_desc_sw128(va + k * 2048, kHalfBytes, 1024), p.idesc_pv, (accumulate || k != 0) ? 1u : 0u);
                }
            };
            int r = 0;
            if (ok) {
                ok = mbar_wait(&kv_full[0], 0, abort_flag);
                if (ok) {
                    tc_fence_after();
                    for (int t = 0; t < 2; ++t) {
                        if (nt[t] > 0) {
                            issue_s(t, 0);
                            umma_commit(&s_full[t]);
                        }
                    }
                    umma_commit(&kv_empty[0]);
                    r = 1;
                }
            }
            for (int j = 0; j < nmax && ok; ++j) {
                const int sv = r % kRing;
                if (!mbar_wait(&kv_full[sv], static_cast<uint32_t>(r / kRing) & 1u, abort_flag)) { ok = false; break; }
                ++r;
                const int sk = r % kRing;
                const uint32_t sk_phase = static_cast<uint32_t>(r / kRing) & 1u;
                bool k_ready = false;
                for (int t = 0; t < 2 && ok; ++t) {
                    if (j < nt[t]) {
                        if (!mbar_wait(&p_full[t], static_cast<uint32_t>(j) & 1u, abort_flag)) { ok = false; break; }
                        tc_fence_after();
                        issue_pv(t, sv, j > 0);
                        umma_commit(&pv_done[t]);
                    }
                    if (t == 1) umma_commit(&kv_empty[sv]);  // V_j is free once both tiles' products have read it
                    if (j + 1 < nt[t]) {
                        if (!k_ready) {
                            if (!mbar_wait(&kv_full[sk], sk_phase, abort_flag)) { ok = false; break; }
                            tc_fence_after();
                            k_ready = true;
                        }
                        issue_s(t, sk);
                        umma_commit(&s_full[t]);
                    }
                }
                if (ok && j + 1 < nmax) {
                    umma_commit(&kv_empty[sk]);
                    ++r;
                }
            }
        }
    } else if (warp >= 4) {
        // ---------------- softmax + output (one thread per query row) ----------------
        const int t = (warp - 4) >> 2;
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are the ones this warp may touch
        const int r_in_tile = quarter * 32 + lane;
        const int q_lo = q0 + t * kTileQ;
        const int q_row = q_lo + r_in_tile;
        const int n_t = t == 0 ? n0 : n1;
        const int k_visible = p.causal ? min(p.Skv - 1, q_row + p.causal_off) : p.Skv - 1;  // last key this row may see
        uint8_t* pbuf = smem_p + t * kTileBytes;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t s_tmem = lane_base + t * 128;
        const uint32_t o_tmem = lane_base + 256 + t * 128;
        const float neg_inf = -INFINITY;
        float m_used = neg_inf;
        float l_sum = 0.f;
        bool ok = true;
        for (int j = 0; j < n_t; ++j) {
            ok = mbar_wait(&s_full[t], static_cast<uint32_t>(j) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t s[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_tmem + c * 32, s[c]);
            tmem_ld_wait();
            const int k0 = j * kBlockKv;
            // warp-uniform: does any element of this tile x block need the mask?
            const bool need_mask = (k0 + kBlockKv > p.Skv) || (p.causal && k0 + kBlockKv - 1 > q_lo + p.causal_off);
            float mx = neg_inf;
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float v = __uint_as_float(s[c][i]) * p.scale_log2;
                        if (k0 + c * 32 + i > k_visible) v = neg_inf;
                        s[c][i] = __float_as_uint(v);
                        mx = fmaxf(mx, v);
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float v = __uint_as_float(s[c][i]) * p.scale_log2;
                        s[c][i] = __float_as_uint(v);
                        mx = fmaxf(mx, v);
                    }
                }
            }
            // The running maximum only moves when some row of the warp outgrew it by more than the threshold: P stays
            // below 2^8 and most blocks need no pass over O.
            float factor = 1.f;
            bool rescale = false;
            if (j == 0) {
                m_used = mx;
            } else {
                rescale = __any_sync(0xffffffffu, mx > m_used + kRescaleThreshold);
                if (rescale) {
                    const float m_new = fmaxf(m_used, mx);
                    factor = (m_used == neg_inf) ? 0.f : fast_exp2(m_used - m_new);
                    m_used = m_new;
                }
                // P of the previous block has been consumed and O is at rest
                ok = mbar_wait(&pv_done[t], static_cast<uint32_t>(j - 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (rescale) {
                    l_sum *= factor;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[32];
                        tmem_ld_32x32(o_tmem + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                        tmem_st_32x32(o_tmem + c * 32, o);
                    }
                    tmem_st_wait();
                }
            }
            const float base = (m_used == neg_inf) ? 0.f : m_used;
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    float e[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        e[u] = fast_exp2(__uint_as_float(s[c][i + u]) - base);
                        part += e[u];
                    }
                    uint4 w;
                    w.x = pack2<T>(e[0], e[1]);
                    w.y = pack2<T>(e[2], e[3]);
                    w.z = pack2<T>(e[4], e[5]);
                    w.w = pack2<T>(e[6], e[7]);
                    // 16-byte chunk `chunk` of the row sits at position chunk ^ (row & 7): the 128-byte swizzle of a
                    // K-major tensor-core operand
                    const int chunk = (c & 1) * 4 + (i >> 3);
                    *reinterpret_cast<uint4*>(pbuf + (c >> 1) * kHalfBytes + r_in_tile * 128 + ((chunk ^ (r_in_tile & 7)) * 16)) = w;
                }
            }
            l_sum += part;
            fence_proxy_async();  // generic-proxy writes of P -> visible to the tensor core's reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[t]);
        }

        // ---- normalise and store this warp's 32 rows ----
        if (ok && q_lo + quarter * 32 < p.Sq) {
            if (n_t > 0) {
                ok = mbar_wait(&pv_done[t], static_cast<uint32_t>(n_t - 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                tc_fence_after();
                const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
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
                        const int chunk = (c & 1) * 4 + (i >> 3);
                        *reinterpret_cast<uint4*>(pbuf + (c >> 1) * kHalfBytes + r_in_tile * 128 + ((chunk ^ (r_in_tile & 7)) * 16)) = w;
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    for (int g = 0; g < 2; ++g) {
                        // rows beyond Sq are clipped by the copy engine
                        const int row = q_lo + quarter * 32;
                        tma_store_4d(&map_o, pbuf + g * kHalfBytes + quarter * (32 * 128), g * 64, p.o_hfirst ? h : row, p.o_hfirst ? row : h, b);
                    }
                    tma_store_commit();
                }
                if (p.lse != nullptr && q_row < p.Sq) {
                    const float lse = l_sum > 0.f ? m_used * 0.6931471805599453f + logf(l_sum) : neg_inf;
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


template <typename T>
cudaError_t launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, const AttnParams& p, int grid,
                           cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    attn_prefill_kernel<T><<<grid, kAttnThreads, kAttnSmem, stream>>>(mq, mk, mv, mo, p);
    return cudaPeekAtLastError();
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
    B200_CHECK(b200::attention_prefill_applies(vq, vk, vv, vo),
               "diopiMultiHeadAttention: needs bf16 / fp16 operands of one dtype, head dim 128, unit innermost pitch, other pitches "
               "multiples of 8 elements and 16-byte aligned bases");
    return b200::attention_prefill_launch(vq, vk, vv, vo, lse, is_causal, scale, stream);
}
