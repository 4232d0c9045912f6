// Row-wise memory-bound ops: RMSNorm, LayerNorm, softmax, mean / sum.
//
// Layout: the reduced extent is the dense innermost run of the tensor ("row"). One CTA owns one row; every
// thread keeps its share of the row in registers as 128-bit vectors (up to kMaxVpt per thread), so a row is
// read from HBM exactly once and written exactly once: algorithmic traffic = 2 * row bytes (+ parameters,
// which stay in L2). Reductions are warp shuffles plus one shared-memory hop. Rows longer than
// 1024 threads * kMaxVpt vectors take the strided fallback at the end of this file.
//
// These kernels are bound by how many instructions a row costs as much as by memory (a dozen small CTAs per SM keep enough
// loads in flight; measured: persistent CTAs fed by bulk copies through shared memory, with fewer resident warps, were
// slower). So the arithmetic works on PAIRS of elements: a 32-bit word of two 2-byte elements is widened once to a float2,
// sums / products use the two-wide fp32 instructions of sm_100 (fma / mul / add .f32x2, one issue slot for two results) and
// a pair is narrowed with one cvt.rn.<t>x2.f32 (LayerNorm [16384, 4096] bf16: 0.74 -> 0.87 of the copy bandwidth).
#include "copy.h"
#include "device_utils.cuh"

namespace b200 {
namespace {

constexpr int kMaxVpt = 8;

struct RowCfg {
    int threads;
    int vpt;
};

// Picks the CTA width so that each thread owns about `target` vectors (four: enough bytes in flight per SM with many
// resident CTAs) and never more than kMaxVpt. The softmax keeps its share of the row as fp32 exponentials between its passes;
// with two vectors per thread it stays within 32 registers and the SM holds its full 64 warps (rows of 4096 bf16: 0.83 -> 0.88
// of the copy bandwidth at 16 k rows), while the norms, which re-widen the packed row instead, measured best with four.
bool pick_row_cfg(int64_t nvec, RowCfg* cfg, int target = 4) {
    int64_t threads = (nvec + target - 1) / target;
    threads = ((threads + 31) / 32) * 32;
    if (threads < 32) threads = 32;
    if (threads > 1024) threads = 1024;
    const int64_t vpt = (nvec + threads - 1) / threads;
    if (vpt > kMaxVpt) return false;
    cfg->threads = static_cast<int>(threads);
    cfg->vpt = static_cast<int>(vpt <= 1 ? 1 : (vpt <= 2 ? 2 : (vpt <= 4 ? 4 : 8)));
    return true;
}

template <typename T, int VPT>
__device__ __forceinline__ void load_row(const T* row, int64_t nvec, Vec16<T> (&x)[VPT]) {
    constexpr int V = Vec16<T>::N;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int64_t iv = static_cast<int64_t>(i) * blockDim.x + threadIdx.x;
        if (iv < nvec) x[i] = ld16_stream(row + iv * V);
    }
}

// Pair j of a 16-byte vector as float2, and a vector rebuilt from V/2 float2 results (one narrowing conversion per pair for
// the 2-byte types). The row kernels below do their arithmetic on such pairs with the two-wide fp32 instructions.
template <typename T>
__device__ __forceinline__ float2 vec_pair(const Vec16<T>& v, int j) {
    if constexpr (sizeof(T) == 2) {
        return Pair<T>::widen(word(*reinterpret_cast<const uint4*>(&v), j));
    } else {
        return make_float2(to_f32(v.v[2 * j]), to_f32(v.v[2 * j + 1]));
    }
}
template <typename T>
__device__ __forceinline__ Vec16<T> vec_from_pairs(const float2 (&p)[Vec16<T>::N / 2]) {
    Vec16<T> y;
    if constexpr (sizeof(T) == 2) {
        uint4 raw = make_uint4(Pair<T>::narrow(p[0]), Pair<T>::narrow(p[1]), Pair<T>::narrow(p[2]), Pair<T>::narrow(p[3]));
        *reinterpret_cast<uint4*>(&y) = raw;
    } else {
#pragma unroll
        for (int j = 0; j < Vec16<T>::N / 2; ++j) {
            y.v[2 * j] = from_f32<T>(p[j].x);
            y.v[2 * j + 1] = from_f32<T>(p[j].y);
        }
    }
    return y;
}

// ---- RMSNorm ---------------------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const T* __restrict__ in, T* __restrict__ out, const T* __restrict__ weight,
                                                       const T* __restrict__ bias, void* inv_rms, diopiDtype_t inv_dt, int64_t cols, float eps) {
    grid_launch_dependents();   // the product that follows may set itself up meanwhile (gemm_tc.cu, launch_splitk)
    constexpr int V = Vec16<T>::N;
    __shared__ float red[32];
    const int64_t nvec = cols / V;
    const int64_t r = blockIdx.x;
    const T* row = in + r * cols;
    Vec16<T> x[VPT];
    load_row<T, VPT>(row, nvec, x);
    float ss = 0.f;
    if constexpr (sizeof(T) == 2) {
        // two elements per step: widened pairs, two-wide fused multiply-add
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (static_cast<int64_t>(i) * blockDim.x + threadIdx.x < nvec) {
                const uint4 raw = *reinterpret_cast<const uint4*>(&x[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 v = Pair<T>::widen(word(raw, j));
                    acc = fma2(v, v, acc);
                }
            }
        }
        ss = acc.x + acc.y;
    } else {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (static_cast<int64_t>(i) * blockDim.x + threadIdx.x < nvec) {
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    const float f = to_f32(x[i].v[e]);
                    ss += f * f;
                }
            }
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / static_cast<float>(cols) + eps);
    if (inv_rms != nullptr && threadIdx.x == 0) store_from<float>(inv_rms, inv_dt, r, inv);
    T* orow = out + r * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int64_t iv = static_cast<int64_t>(i) * blockDim.x + threadIdx.x;
        if (iv < nvec) {
            Vec16<T> y;
            if constexpr (sizeof(T) == 2) {
                if (bias == nullptr) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(&x[i]);
                    const float2 inv2 = make_float2(inv, inv);
                    uint32_t o[4];
                    if (weight != nullptr) {
                        const Vec16<T> w = ld16(weight + iv * V);
                        const uint4 wraw = *reinterpret_cast<const uint4*>(&w);
#pragma unroll
                        for (int j = 0; j < 4; ++j) o[j] = Pair<T>::narrow(mul2(mul2(Pair<T>::widen(word(raw, j)), inv2), Pair<T>::widen(word(wraw, j))));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) o[j] = Pair<T>::narrow(mul2(Pair<T>::widen(word(raw, j)), inv2));
                    }
                    st16_stream_raw(orow + iv * V, make_uint4(o[0], o[1], o[2], o[3]));
                    continue;
                }
            }
            if (weight != nullptr) {
                const Vec16<T> w = ld16(weight + iv * V);
#pragma unroll
                for (int e = 0; e < V; ++e) y.v[e] = from_f32<T>(to_f32(x[i].v[e]) * inv * to_f32(w.v[e]));
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) y.v[e] = from_f32<T>(to_f32(x[i].v[e]) * inv);
            }
            if (bias != nullptr) {
                const Vec16<T> b = ld16(bias + iv * V);
#pragma unroll
                for (int e = 0; e < V; ++e) y.v[e] = from_f32<T>(to_f32(y.v[e]) + to_f32(b.v[e]));
            }
            st16_stream(orow + iv * V, y);
        }
    }
}

// ---- LayerNorm ---------------------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(1024) layernorm_kernel(const T* __restrict__ in, T* __restrict__ out, const T* __restrict__ weight,
                                                         const T* __restrict__ bias, void* save_mean, void* save_invstd, diopiDtype_t stat_dt,
                                                         int64_t cols, float eps) {
    constexpr int V = Vec16<T>::N;
    __shared__ float red[32];
    const int64_t nvec = cols / V;
    const int64_t r = blockIdx.x;
    Vec16<T> x[VPT];
    load_row<T, VPT>(in + r * cols, nvec, x);
    // the row is widened to fp32 pairs once and stays in registers for the three passes (sum, squared deviations, output)
    constexpr int P = V / 2;
    float2 f[VPT][P];
    float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const bool live = static_cast<int64_t>(i) * blockDim.x + threadIdx.x < nvec;
#pragma unroll
        for (int j = 0; j < P; ++j) {
            f[i][j] = live ? vec_pair<T>(x[i], j) : make_float2(0.f, 0.f);
            s2 = add2(s2, f[i][j]);
        }
    }
    const float mean = block_sum(s2.x + s2.y, red) / static_cast<float>(cols);
    const float2 mm = make_float2(-mean, -mean);
    float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (static_cast<int64_t>(i) * blockDim.x + threadIdx.x < nvec) {
#pragma unroll
            for (int j = 0; j < P; ++j) {
                f[i][j] = add2(f[i][j], mm);
                q2 = fma2(f[i][j], f[i][j], q2);
            }
        }
    }
    const float var = block_sum(q2.x + q2.y, red) / static_cast<float>(cols);
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
        if (save_mean != nullptr) store_from<float>(save_mean, stat_dt, r, mean);
        if (save_invstd != nullptr) store_from<float>(save_invstd, stat_dt, r, rstd);
    }
    const float2 rs = make_float2(rstd, rstd);
    T* orow = out + r * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int64_t iv = static_cast<int64_t>(i) * blockDim.x + threadIdx.x;
        if (iv < nvec) {
            float2 y[P];
            if (weight != nullptr) {
                const Vec16<T> w = ld16(weight + iv * V);
                if (bias != nullptr) {
                    const Vec16<T> b = ld16(bias + iv * V);
#pragma unroll
                    for (int j = 0; j < P; ++j) y[j] = fma2(mul2(f[i][j], rs), vec_pair<T>(w, j), vec_pair<T>(b, j));
                } else {
#pragma unroll
                    for (int j = 0; j < P; ++j) y[j] = mul2(mul2(f[i][j], rs), vec_pair<T>(w, j));
                }
            } else if (bias != nullptr) {
                const Vec16<T> b = ld16(bias + iv * V);
#pragma unroll
                for (int j = 0; j < P; ++j) y[j] = fma2(f[i][j], rs, vec_pair<T>(b, j));
            } else {
#pragma unroll
                for (int j = 0; j < P; ++j) y[j] = mul2(f[i][j], rs);
            }
            st16_stream(orow + iv * V, vec_from_pairs<T>(y));
        }
    }
}

// ---- softmax over the innermost run ------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(1024) softmax_row_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t cols) {
    constexpr int V = Vec16<T>::N;
    __shared__ float red[32];
    const int64_t nvec = cols / V;
    const int64_t r = blockIdx.x;
    Vec16<T> x[VPT];
    load_row<T, VPT>(in + r * cols, nvec, x);
    constexpr int P = V / 2;
    float2 f[VPT][P];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const bool live = static_cast<int64_t>(i) * blockDim.x + threadIdx.x < nvec;
#pragma unroll
        for (int j = 0; j < P; ++j) {
            f[i][j] = live ? vec_pair<T>(x[i], j) : make_float2(-INFINITY, -INFINITY);
            m = fmaxf(m, fmaxf(f[i][j].x, f[i][j].y));
        }
    }
    m = block_max(m, red);
    // a row of all -inf has no finite maximum: torch yields NaN there, and so does exp(-inf - -inf)
    float2 s2 = make_float2(0.f, 0.f);
    if constexpr (sizeof(T) == 2) {
        // two-byte outputs round to 8 or 11 bits: exp(x - m) as 2^(x * log2(e) - m * log2(e)) with the approximate exponential
        // is far inside that
        constexpr float kLog2e = 1.4426950408889634f;
        const float2 l2 = make_float2(kLog2e, kLog2e), off = make_float2(-m * kLog2e, -m * kLog2e);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const bool live = static_cast<int64_t>(i) * blockDim.x + threadIdx.x < nvec;
#pragma unroll
            for (int j = 0; j < P; ++j) {
                const float2 t = fma2(f[i][j], l2, off);
                f[i][j] = live ? make_float2(exp2f(t.x), exp2f(t.y)) : make_float2(0.f, 0.f);
                s2 = add2(s2, f[i][j]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const bool live = static_cast<int64_t>(i) * blockDim.x + threadIdx.x < nvec;
#pragma unroll
            for (int j = 0; j < P; ++j) {
                f[i][j] = live ? make_float2(expf(f[i][j].x - m), expf(f[i][j].y - m)) : make_float2(0.f, 0.f);
                s2 = add2(s2, f[i][j]);
            }
        }
    }
    const float s = block_sum(s2.x + s2.y, red);
    const float inv = 1.f / s;
    const float2 inv2 = make_float2(inv, inv);
    T* orow = out + r * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int64_t iv = static_cast<int64_t>(i) * blockDim.x + threadIdx.x;
        if (iv < nvec) {
            float2 y[P];
#pragma unroll
            for (int j = 0; j < P; ++j) y[j] = mul2(f[i][j], inv2);
            st16_stream(orow + iv * V, vec_from_pairs<T>(y));
        }
    }
}

// Rows of at most 256 vectors (2048 two-byte or 1024 four-byte elements - the rows of an attention score tensor): one
// WARP per row and eight rows per CTA. A CTA per row would be 32 - 64 threads; at half a million rows the launch rate of
// such tiny CTAs, not memory, bounds the kernel. Lane l owns vectors l, l + 32, ...; reductions are shuffles only.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int64_t cols) {
    constexpr int V = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int nvec = static_cast<int>(cols / V);
    const T* row = in + r * cols;
    Vec16<T> x[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (i * 32 + lane < nvec) x[i] = ld16_stream(row + static_cast<int64_t>(i * 32 + lane) * V);
    }
    float f[VPT][V];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const bool live = i * 32 + lane < nvec;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            f[i][e] = live ? to_f32(x[i].v[e]) : -INFINITY;
            m = fmaxf(m, f[i][e]);
        }
    }
    m = warp_max(m);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
            f[i][e] = (sizeof(T) == 2) ? __expf(f[i][e] - m) : expf(f[i][e] - m);  // exp(-inf) = 0 for the padding lanes
            s += f[i][e];
        }
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
    T* orow = out + r * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (i * 32 + lane < nvec) {
            Vec16<T> y;
#pragma unroll
            for (int e = 0; e < V; ++e) y.v[e] = from_f32<T>(f[i][e] * inv);
            st16_stream(orow + static_cast<int64_t>(i * 32 + lane) * V, y);
        }
    }
}

// Rows of 129 - 256 vectors (the 2048-element rows of a 7B score tensor): TWO warps per row and four rows per CTA. A lane then
// keeps 32 instead of 64 fp32 values between the passes, which takes the kernel from 79 to under 50 registers and the SM from 24 to
// 40 resident warps: these rows are short enough that the time a warp spends exponentiating, with no load in flight, shows. The two
// warps of a row meet twice (maximum, sum) through one shared-memory slot each and a 64-thread named barrier.
template <typename T>
__global__ void __launch_bounds__(256) softmax_warp_pair_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int64_t cols) {
    constexpr int V = Vec16<T>::N;
    constexpr int VPT = 4;
    __shared__ float xch[4][2][2];  // [row of the CTA][maximum / sum][warp of the row]
    const int lane = threadIdx.x & 31;
    const int half = (threadIdx.x >> 5) & 1;
    const int rr = threadIdx.x >> 6;
    const int64_t r = static_cast<int64_t>(blockIdx.x) * 4 + rr;
    const bool row_live = r < rows;
    const int nvec = static_cast<int>(cols / V);
    const T* row = in + (row_live ? r : 0) * cols;
    Vec16<T> x[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int iv = i * 64 + half * 32 + lane;
        if (row_live && iv < nvec) x[i] = ld16_stream(row + static_cast<int64_t>(iv) * V);
    }
    float f[VPT][V];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const bool live = row_live && i * 64 + half * 32 + lane < nvec;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            f[i][e] = live ? to_f32(x[i].v[e]) : -INFINITY;
            m = fmaxf(m, f[i][e]);
        }
    }
    m = warp_max(m);
    if (lane == 0) xch[rr][0][half] = m;
    asm volatile("bar.sync %0, 64;" ::"r"(rr + 1) : "memory");
    m = fmaxf(xch[rr][0][0], xch[rr][0][1]);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
            f[i][e] = (sizeof(T) == 2) ? __expf(f[i][e] - m) : expf(f[i][e] - m);  // exp(-inf) = 0 for the padding lanes
            s += f[i][e];
        }
    }
    s = warp_sum(s);
    if (lane == 0) xch[rr][1][half] = s;
    asm volatile("bar.sync %0, 64;" ::"r"(rr + 1) : "memory");
    s = xch[rr][1][0] + xch[rr][1][1];
    const float inv = 1.f / s;
    T* orow = out + (row_live ? r : 0) * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int iv = i * 64 + half * 32 + lane;
        if (row_live && iv < nvec) {
            Vec16<T> y;
#pragma unroll
            for (int e = 0; e < V; ++e) y.v[e] = from_f32<T>(f[i][e] * inv);
            st16_stream(orow + static_cast<int64_t>(iv) * V, y);
        }
    }
}

// ---- row sum / mean --------------------------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(1024) rowsum_kernel(const T* __restrict__ in, void* out, diopiDtype_t out_dt, int64_t cols, float scale) {
    constexpr int V = Vec16<T>::N;
    __shared__ float red[32];
    const int64_t nvec = cols / V;
    const int64_t r = blockIdx.x;
    Vec16<T> x[VPT];
    load_row<T, VPT>(in + r * cols, nvec, x);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        if (static_cast<int64_t>(i) * blockDim.x + threadIdx.x < nvec) {
#pragma unroll
            for (int e = 0; e < V; ++e) s += to_f32(x[i].v[e]);
        }
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) store_from<float>(out, out_dt, r, s * scale);
}

// ---- strided fallbacks (any dim, any dtype; one warp per output slice) --------------------------------------------------
// The tensor is viewed as [outer, n, inner] with the reduced / normalised extent n in the middle.
template <typename C>
__global__ void softmax_strided_kernel(const void* in, diopiDtype_t in_dt, void* out, diopiDtype_t out_dt, int64_t outer, int64_t n,
                                       int64_t inner) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t s = warp; s < outer * inner; s += nwarps) {
        const int64_t o = s / inner, k = s - o * inner;
        const int64_t base = o * n * inner + k;
        C m = -INFINITY;
        for (int64_t j = lane; j < n; j += 32) {
            const C v = load_as<C>(in, in_dt, base + j * inner);
            m = v > m ? v : m;
        }
        for (int off = 16; off > 0; off >>= 1) {
            const C t = __shfl_xor_sync(0xffffffffu, m, off);
            m = t > m ? t : m;
        }
        C sum = 0;
        for (int64_t j = lane; j < n; j += 32) sum += exp(load_as<C>(in, in_dt, base + j * inner) - m);
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        for (int64_t j = lane; j < n; j += 32) {
            const C v = exp(load_as<C>(in, in_dt, base + j * inner) - m) / sum;
            store_from<C>(out, out_dt, base + j * inner, v);
        }
    }
}

struct ReduceIter {
    int nkeep, nred;
    int64_t keep_shape[kMaxDims], keep_stride[kMaxDims];
    int64_t red_shape[kMaxDims], red_stride[kMaxDims];
    int64_t n_out, n_red;
};

template <typename C>
__global__ void reduce_sum_strided_kernel(const void* in, diopiDtype_t in_dt, void* out, diopiDtype_t out_dt, const ReduceIter it, C scale) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t o = warp; o < it.n_out; o += nwarps) {
        int64_t base = 0, rem = o;
        for (int d = it.nkeep - 1; d >= 0; --d) {
            const int64_t q = rem / it.keep_shape[d];
            base += (rem - q * it.keep_shape[d]) * it.keep_stride[d];
            rem = q;
        }
        C acc = 0;
        for (int64_t j = lane; j < it.n_red; j += 32) {
            int64_t off = base, r = j;
            for (int d = it.nred - 1; d >= 0; --d) {
                const int64_t q = r / it.red_shape[d];
                off += (r - q * it.red_shape[d]) * it.red_stride[d];
                r = q;
            }
            acc += load_as<C>(in, in_dt, off);
        }
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) store_from<C>(out, out_dt, o, acc * scale);
    }
}

#define B200_DISPATCH_VPT(VPT_VALUE, ...)              \
    switch (VPT_VALUE) {                               \
        case 1: { constexpr int VPT = 1; __VA_ARGS__; break; } \
        case 2: { constexpr int VPT = 2; __VA_ARGS__; break; } \
        case 4: { constexpr int VPT = 4; __VA_ARGS__; break; } \
        default: { constexpr int VPT = 8; __VA_ARGS__; break; } \
    }

// Can `v` use the register-resident row kernels for rows of `cols` elements?
bool row_fast_ok(const TensorView& v, int64_t cols, RowCfg* cfg, int target = 4) {
    if (!(v.dtype == diopi_dtype_bfloat16 || v.dtype == diopi_dtype_float16 || v.dtype == diopi_dtype_float32)) return false;
    const int V = 16 / static_cast<int>(v.itemsize);
    if (cols % V != 0 || !v.aligned(16)) return false;
    return pick_row_cfg(cols / V, cfg, target);
}

int64_t shape_product(diopiSize_t s) {
    int64_t p = 1;
    for (int64_t i = 0; i < s.len; ++i) p *= s.data[i];
    return p;
}

bool param_ok(const TensorView* p, const TensorView& x, int64_t cols) {
    return p == nullptr || (p->dtype == x.dtype && p->numel == cols && p->is_contiguous() && p->aligned(16) && p->device == diopi_device);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

diopiError_t diopiRMSNorm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiTensorHandle_t inv_rms, diopiConstTensorHandle_t input,
                          diopiSize_t normalized_shape, diopiConstTensorHandle_t weight, diopiConstTensorHandle_t bias, double eps) {
    B200_VIEW(vo, out);
    B200_VIEW(vx_raw, input);
    TensorView vw, vb, vinv;
    if (weight && !make_view(weight, &vw, "weight")) return diopiErrorOccurred;
    if (bias && !make_view(bias, &vb, "bias")) return diopiErrorOccurred;
    if (inv_rms && !make_view(inv_rms, &vinv, "inv_rms")) return diopiErrorOccurred;
    B200_CHECK(normalized_shape.len >= 1 && normalized_shape.len <= vx_raw.ndim, "diopiRMSNorm: bad normalized_shape rank");
    for (int64_t i = 0; i < normalized_shape.len; ++i) {
        B200_CHECK(normalized_shape.data[i] == vx_raw.shape[vx_raw.ndim - normalized_shape.len + i], "diopiRMSNorm: normalized_shape mismatches the input");
    }
    const int64_t cols = shape_product(normalized_shape);
    B200_CHECK(vo.numel == vx_raw.numel && vo.dtype == vx_raw.dtype, "diopiRMSNorm: output must match the input shape and dtype");
    B200_CHECK(vo.is_contiguous(), "diopiRMSNorm: output must be contiguous");
    if (vo.numel == 0) return diopiSuccess;
    const int64_t rows = vx_raw.numel / cols;
    if (inv_rms) B200_CHECK(vinv.numel == rows && vinv.is_contiguous(), "diopiRMSNorm: inv_rms must be dense with one entry per row");
    TensorView vx;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    RowCfg cfg;
    B200_CHECK(row_fast_ok(vx, cols, &cfg) && vo.aligned(16),
               "diopiRMSNorm: rows of %lld %s elements are outside the supported range (16-byte multiple, at most %d vectors)", (long long)cols,
               dtype_name(vx.dtype), 1024 * kMaxVpt);
    B200_CHECK(param_ok(weight ? &vw : nullptr, vx, cols) && param_ok(bias ? &vb : nullptr, vx, cols),
               "diopiRMSNorm: weight/bias must be dense device tensors of the input dtype with normalized_shape elements");
    cudaStream_t stream = stream_of(ctx);
    const unsigned grid = static_cast<unsigned>(rows);
    B200_CHECK(rows <= 0x7fffffffLL, "diopiRMSNorm: too many rows");
#define LAUNCH_RMS(T)                                                                                                                   \
    B200_DISPATCH_VPT(cfg.vpt, (rmsnorm_kernel<T, VPT><<<grid, cfg.threads, 0, stream>>>(                                                 \
                                   static_cast<const T*>(vx.data), static_cast<T*>(vo.data), weight ? static_cast<const T*>(vw.data) : nullptr, \
                                   bias ? static_cast<const T*>(vb.data) : nullptr, inv_rms ? vinv.data : nullptr,                        \
                                   inv_rms ? vinv.dtype : diopi_dtype_float32, cols, static_cast<float>(eps))))
    if (vx.dtype == diopi_dtype_bfloat16) { LAUNCH_RMS(bf16); }
    else if (vx.dtype == diopi_dtype_float16) { LAUNCH_RMS(fp16); }
    else { LAUNCH_RMS(float); }
#undef LAUNCH_RMS
    B200_LAUNCH_CHECK("diopiRMSNorm");
    return diopiSuccess;
}

diopiError_t diopiLayerNorm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiTensorHandle_t save_mean, diopiTensorHandle_t save_invstd,
                            diopiConstTensorHandle_t input, diopiConstTensorHandle_t weight, diopiConstTensorHandle_t bias,
                            diopiSize_t normalized_shape, double eps) {
    B200_VIEW(vo, out);
    B200_VIEW(vx_raw, input);
    TensorView vw, vb, vm, vs;
    if (weight && !make_view(weight, &vw, "weight")) return diopiErrorOccurred;
    if (bias && !make_view(bias, &vb, "bias")) return diopiErrorOccurred;
    if (save_mean && !make_view(save_mean, &vm, "save_mean")) return diopiErrorOccurred;
    if (save_invstd && !make_view(save_invstd, &vs, "save_invstd")) return diopiErrorOccurred;
    B200_CHECK(normalized_shape.len >= 1 && normalized_shape.len <= vx_raw.ndim, "diopiLayerNorm: bad normalized_shape rank");
    for (int64_t i = 0; i < normalized_shape.len; ++i) {
        B200_CHECK(normalized_shape.data[i] == vx_raw.shape[vx_raw.ndim - normalized_shape.len + i], "diopiLayerNorm: normalized_shape mismatches the input");
    }
    const int64_t cols = shape_product(normalized_shape);
    B200_CHECK(vo.numel == vx_raw.numel && vo.dtype == vx_raw.dtype, "diopiLayerNorm: output must match the input shape and dtype");
    B200_CHECK(vo.is_contiguous(), "diopiLayerNorm: output must be contiguous");
    if (vo.numel == 0) return diopiSuccess;
    const int64_t rows = vx_raw.numel / cols;
    if (save_mean) B200_CHECK(vm.numel == rows && vm.is_contiguous(), "diopiLayerNorm: save_mean must be dense with one entry per row");
    if (save_invstd) B200_CHECK(vs.numel == rows && vs.is_contiguous(), "diopiLayerNorm: save_invstd must be dense with one entry per row");
    if (save_mean && save_invstd) B200_CHECK(vm.dtype == vs.dtype, "diopiLayerNorm: save_mean / save_invstd dtypes differ");
    TensorView vx;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    RowCfg cfg;
    B200_CHECK(row_fast_ok(vx, cols, &cfg) && vo.aligned(16),
               "diopiLayerNorm: rows of %lld %s elements are outside the supported range (16-byte multiple, at most %d vectors)", (long long)cols,
               dtype_name(vx.dtype), 1024 * kMaxVpt);
    B200_CHECK(param_ok(weight ? &vw : nullptr, vx, cols) && param_ok(bias ? &vb : nullptr, vx, cols),
               "diopiLayerNorm: weight/bias must be dense device tensors of the input dtype with normalized_shape elements");
    cudaStream_t stream = stream_of(ctx);
    B200_CHECK(rows <= 0x7fffffffLL, "diopiLayerNorm: too many rows");
    const unsigned grid = static_cast<unsigned>(rows);
    const diopiDtype_t stat_dt = save_mean ? vm.dtype : (save_invstd ? vs.dtype : diopi_dtype_float32);
#define LAUNCH_LN(T)                                                                                                                    \
    B200_DISPATCH_VPT(cfg.vpt, (layernorm_kernel<T, VPT><<<grid, cfg.threads, 0, stream>>>(                                               \
                                   static_cast<const T*>(vx.data), static_cast<T*>(vo.data), weight ? static_cast<const T*>(vw.data) : nullptr, \
                                   bias ? static_cast<const T*>(vb.data) : nullptr, save_mean ? vm.data : nullptr,                        \
                                   save_invstd ? vs.data : nullptr, stat_dt, cols, static_cast<float>(eps))))
    if (vx.dtype == diopi_dtype_bfloat16) { LAUNCH_LN(bf16); }
    else if (vx.dtype == diopi_dtype_float16) { LAUNCH_LN(fp16); }
    else { LAUNCH_LN(float); }
#undef LAUNCH_LN
    B200_LAUNCH_CHECK("diopiLayerNorm");
    return diopiSuccess;
}

diopiError_t diopiSoftmax(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, int64_t dim) {
    B200_VIEW(vo, out);
    B200_VIEW(vx_raw, input);
    B200_CHECK(vo.numel == vx_raw.numel, "diopiSoftmax: output must match the input shape");
    B200_CHECK(vo.is_contiguous(), "diopiSoftmax: output must be contiguous");
    B200_CHECK(is_floating(vx_raw.dtype) && is_floating(vo.dtype), "diopiSoftmax: floating dtypes only");
    if (vo.numel == 0) return diopiSuccess;
    const int nd = vx_raw.ndim == 0 ? 1 : vx_raw.ndim;
    if (dim < 0) dim += nd;
    B200_CHECK(dim >= 0 && dim < nd, "diopiSoftmax: dim out of range");
    TensorView vx;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    int64_t outer = 1, inner = 1;
    const int64_t n = vx.ndim == 0 ? 1 : vx.shape[dim];
    for (int d = 0; d < dim; ++d) outer *= vx.shape[d];
    for (int d = static_cast<int>(dim) + 1; d < vx.ndim; ++d) inner *= vx.shape[d];
    cudaStream_t stream = stream_of(ctx);
    RowCfg cfg;
    if (inner == 1 && vo.dtype == vx.dtype && row_fast_ok(vx, n, &cfg, 2) && vo.aligned(16) && outer <= 0x7fffffffLL) {
        const unsigned grid = static_cast<unsigned>(outer);
        const int64_t nvec = n * vx.itemsize / 16;
        if (nvec <= 256 && outer >= 1024) {
            // many short rows: a warp per row
            if (nvec > 128 && vx.itemsize == 2) {
                // two warps per row (score tensor of the 7B layer, [256, 2048, 2048]: 0.75 -> 0.67 ms, 0.98 of the copy bandwidth)
                const unsigned pgrid = static_cast<unsigned>((outer + 3) / 4);
                if (vx.dtype == diopi_dtype_bfloat16) softmax_warp_pair_kernel<bf16><<<pgrid, 256, 0, stream>>>(static_cast<const bf16*>(vx.data), static_cast<bf16*>(vo.data), outer, n);
                else softmax_warp_pair_kernel<fp16><<<pgrid, 256, 0, stream>>>(static_cast<const fp16*>(vx.data), static_cast<fp16*>(vo.data), outer, n);
                B200_LAUNCH_CHECK("diopiSoftmax");
                return diopiSuccess;
            }
            const unsigned wgrid = static_cast<unsigned>((outer + 7) / 8);
            const int wvpt = nvec <= 32 ? 1 : (nvec <= 64 ? 2 : (nvec <= 128 ? 4 : 8));
#define LAUNCH_SMW(T) \
    B200_DISPATCH_VPT(wvpt, (softmax_warp_kernel<T, VPT><<<wgrid, 256, 0, stream>>>(static_cast<const T*>(vx.data), static_cast<T*>(vo.data), outer, n)))
            if (vx.dtype == diopi_dtype_bfloat16) { LAUNCH_SMW(bf16); }
            else if (vx.dtype == diopi_dtype_float16) { LAUNCH_SMW(fp16); }
            else { LAUNCH_SMW(float); }
#undef LAUNCH_SMW
            B200_LAUNCH_CHECK("diopiSoftmax");
            return diopiSuccess;
        }
#define LAUNCH_SM(T) \
    B200_DISPATCH_VPT(cfg.vpt, (softmax_row_kernel<T, VPT><<<grid, cfg.threads, 0, stream>>>(static_cast<const T*>(vx.data), static_cast<T*>(vo.data), n)))
        if (vx.dtype == diopi_dtype_bfloat16) { LAUNCH_SM(bf16); }
        else if (vx.dtype == diopi_dtype_float16) { LAUNCH_SM(fp16); }
        else { LAUNCH_SM(float); }
#undef LAUNCH_SM
    } else {
        const int64_t slices = outer * inner;
        int64_t blocks = (slices * 32 + 255) / 256;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
        if (blocks > cap) blocks = cap;
        if (vo.dtype == diopi_dtype_float64) {
            softmax_strided_kernel<double><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(vx.data, vx.dtype, vo.data, vo.dtype, outer, n, inner);
        } else {
            softmax_strided_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(vx.data, vx.dtype, vo.data, vo.dtype, outer, n, inner);
        }
    }
    B200_LAUNCH_CHECK("diopiSoftmax");
    return diopiSuccess;
}

static diopiError_t reduce_sum_impl(diopiContextHandle_t ctx, const char* name, diopiTensorHandle_t out, diopiConstTensorHandle_t input,
                                    diopiSize_t dim, bool mean) {
    B200_VIEW(vo, out);
    B200_VIEW(vx, input);
    B200_CHECK(vo.is_contiguous(), "%s: output must be contiguous", name);
    B200_CHECK(vx.device == diopi_device && vo.device == diopi_device, "%s: operands must be device tensors", name);
    bool reduced[kMaxDims] = {false};
    if (dim.len == 0 || dim.data == nullptr) {
        for (int d = 0; d < vx.ndim; ++d) reduced[d] = true;
    } else {
        for (int64_t i = 0; i < dim.len; ++i) {
            int64_t d = dim.data[i];
            if (d < 0) d += vx.ndim;
            B200_CHECK(d >= 0 && d < (vx.ndim == 0 ? 1 : vx.ndim), "%s: dim out of range", name);
            if (vx.ndim > 0) reduced[d] = true;
        }
    }
    ReduceIter it;
    it.nkeep = it.nred = 0;
    it.n_out = it.n_red = 1;
    for (int d = 0; d < vx.ndim; ++d) {
        if (reduced[d]) {
            it.red_shape[it.nred] = vx.shape[d];
            it.red_stride[it.nred++] = vx.stride[d];
            it.n_red *= vx.shape[d];
        } else {
            it.keep_shape[it.nkeep] = vx.shape[d];
            it.keep_stride[it.nkeep++] = vx.stride[d];
            it.n_out *= vx.shape[d];
        }
    }
    B200_CHECK(vo.numel == it.n_out, "%s: output has %lld elements, expected %lld", name, (long long)vo.numel, (long long)it.n_out);
    if (vo.numel == 0) return diopiSuccess;
    cudaStream_t stream = stream_of(ctx);
    if (it.n_red == 0) return diopiZeroInp(ctx, out);
    const double scale = mean ? 1.0 / static_cast<double>(it.n_red) : 1.0;

    // fast path: the reduced dims are the dense tail of a dense tensor
    bool tail = vx.is_contiguous();
    for (int d = 0, seen = 0; d < vx.ndim && tail; ++d) {
        if (reduced[d]) seen = 1;
        else if (seen && vx.shape[d] != 1) tail = false;
    }
    RowCfg cfg;
    if (tail && row_fast_ok(vx, it.n_red, &cfg) && it.n_out <= 0x7fffffffLL) {
        const unsigned grid = static_cast<unsigned>(it.n_out);
#define LAUNCH_RS(T) \
    B200_DISPATCH_VPT(cfg.vpt, (rowsum_kernel<T, VPT><<<grid, cfg.threads, 0, stream>>>(static_cast<const T*>(vx.data), vo.data, vo.dtype, it.n_red, static_cast<float>(scale))))
        if (vx.dtype == diopi_dtype_bfloat16) { LAUNCH_RS(bf16); }
        else if (vx.dtype == diopi_dtype_float16) { LAUNCH_RS(fp16); }
        else { LAUNCH_RS(float); }
#undef LAUNCH_RS
    } else {
        int64_t blocks = (it.n_out * 32 + 255) / 256;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
        if (blocks > cap) blocks = cap;
        if (vo.dtype == diopi_dtype_float64) {
            reduce_sum_strided_kernel<double><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(vx.data, vx.dtype, vo.data, vo.dtype, it, scale);
        } else if (is_floating(vo.dtype)) {
            reduce_sum_strided_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(vx.data, vx.dtype, vo.data, vo.dtype, it, static_cast<float>(scale));
        } else {
            B200_CHECK(!mean, "%s: mean needs a floating output", name);
            reduce_sum_strided_kernel<int64_t><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(vx.data, vx.dtype, vo.data, vo.dtype, it, (int64_t)1);
        }
    }
    B200_LAUNCH_CHECK(name);
    return diopiSuccess;
}

diopiError_t diopiMean(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiSize_t dim) {
    return reduce_sum_impl(ctx, "diopiMean", out, input, dim, true);
}
diopiError_t diopiSum(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiSize_t dim) {
    return reduce_sum_impl(ctx, "diopiSum", out, input, dim, false);
}

}  // extern "C"
