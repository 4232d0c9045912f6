// Element-wise engine.
//
// Two kernel families serve every unary / binary / ternary op of the library:
//   * ew_vec_kernel   - all operands share one 2- or 4-byte float dtype, the output is dense, every
//                       input is either dense or a dense block that repeats along the leading
//                       dimensions ("modulo broadcast": a [S,S] mask added to [B,H,S,S] scores, an [H]
//                       weight applied to [T,H] rows). 128-bit loads/stores, 4 independent vectors
//                       in flight per thread, streaming cache hints. This is the HBM-roofline path.
//   * ew_generic_kernel - anything else: arbitrary strides, broadcasting by zero strides, mixed
//                       dtypes (converted per element), integer and fp64 arithmetic.
// The op is a functor template over the compute type C (float, double or int64_t).
#pragma once

#include "common.h"
#include "device_utils.cuh"

namespace b200 {

struct ScalarArgs {
    double f[2] = {0.0, 0.0};
    int64_t i[2] = {0, 0};
};

inline void scalar_to_args(const diopiScalar_t* s, ScalarArgs* a, int slot) {
    if (s == nullptr) {
        a->f[slot] = 1.0;
        a->i[slot] = 1;
    } else if (s->stype == diopi_dtype_float64 || s->stype == diopi_dtype_float32) {
        a->f[slot] = s->fval;
        a->i[slot] = static_cast<int64_t>(s->fval);
    } else {
        a->i[slot] = s->ival;
        a->f[slot] = static_cast<double>(s->ival);
    }
}

template <typename C> __host__ __device__ inline C pick_scalar(const ScalarArgs& a, int slot) { return static_cast<C>(a.f[slot]); }
template <> __host__ __device__ inline int64_t pick_scalar<int64_t>(const ScalarArgs& a, int slot) { return a.i[slot]; }

template <int NARGS>
struct EwIter {
    int ndim;
    int64_t numel;
    int64_t shape[kMaxDims];
    int64_t stride[NARGS][kMaxDims];  // elements; operand 0 is the output
    void* ptr[NARGS];
    diopiDtype_t dtype[NARGS];
};

// Broadcast `in` against `out` (right-aligned). Returns false when shapes are incompatible.
inline bool broadcast_strides(const TensorView& out, const TensorView& in, int64_t* strides) {
    const int off = out.ndim - in.ndim;
    if (off < 0) return false;
    for (int d = 0; d < out.ndim; ++d) {
        if (d < off) {
            strides[d] = 0;
        } else {
            const int64_t s = in.shape[d - off];
            if (s == out.shape[d]) {
                strides[d] = (s == 1) ? 0 : in.stride[d - off];
            } else if (s == 1) {
                strides[d] = 0;
            } else {
                return false;
            }
        }
    }
    return true;
}

template <int NARGS>
inline bool build_iter(const TensorView& out, const TensorView* const* ins, EwIter<NARGS>* it) {
    int64_t shape[kMaxDims];
    int64_t st[NARGS][kMaxDims];
    const int nd = out.ndim;
    for (int d = 0; d < nd; ++d) {
        shape[d] = out.shape[d];
        st[0][d] = (out.shape[d] == 1) ? 0 : out.stride[d];
    }
    for (int a = 1; a < NARGS; ++a) {
        if (!broadcast_strides(out, *ins[a - 1], st[a])) return false;
    }
    // Coalesce neighbouring dimensions that every operand walks contiguously.
    int w = -1;
    for (int d = 0; d < nd; ++d) {
        if (shape[d] == 1) continue;
        if (w >= 0) {
            bool merge = true;
            for (int a = 0; a < NARGS; ++a) merge = merge && (st[a][w] == st[a][d] * shape[d]);
            if (merge) {
                it->shape[w] *= shape[d];
                for (int a = 0; a < NARGS; ++a) {
                    it->stride[a][w] = st[a][d];
                    st[a][w] = st[a][d];
                }
                continue;
            }
        }
        ++w;
        it->shape[w] = shape[d];
        for (int a = 0; a < NARGS; ++a) {
            it->stride[a][w] = st[a][d];
            st[a][w] = st[a][d];
        }
    }
    it->ndim = w + 1;
    it->numel = out.numel;
    it->ptr[0] = out.data;
    it->dtype[0] = out.dtype;
    for (int a = 1; a < NARGS; ++a) {
        it->ptr[a] = ins[a - 1]->data;
        it->dtype[a] = ins[a - 1]->dtype;
    }
    return true;
}

// ---- general kernel -------------------------------------------------------------------------------
template <typename C, int NIN, typename Op>
__global__ void __launch_bounds__(256) ew_generic_kernel(const EwIter<NIN + 1> it, const Op op) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < it.numel; i += step) {
        int64_t off[NIN + 1];
#pragma unroll
        for (int a = 0; a <= NIN; ++a) off[a] = 0;
        int64_t rem = i;
        for (int d = it.ndim - 1; d >= 0; --d) {
            const int64_t q = rem / it.shape[d];
            const int64_t c = rem - q * it.shape[d];
            rem = q;
#pragma unroll
            for (int a = 0; a <= NIN; ++a) off[a] += c * it.stride[a][d];
        }
        C in[NIN > 0 ? NIN : 1];
#pragma unroll
        for (int a = 0; a < NIN; ++a) in[a] = load_as<C>(it.ptr[a + 1], it.dtype[a + 1], off[a + 1]);
        C r;
        if constexpr (NIN == 0) r = op();
        else if constexpr (NIN == 1) r = op(in[0]);
        else if constexpr (NIN == 2) r = op(in[0], in[1]);
        else r = op(in[0], in[1], in[2]);
        store_from<C>(it.ptr[0], it.dtype[0], off[0], r);
    }
}

// ---- vector kernel -----------------------------------------------------------------------------------
// period[a]: number of 16-byte vectors after which input a repeats (0 = same length as the output).
struct VecPeriods {
    int64_t period[3];
    int narrow;  // every vector index fits 32 bits: the repeat index is then a 32-bit remainder (a 64-bit one costs ~10x more)
};

// One CTA = one tile of 256 threads x 4 vectors (16 KiB per operand); all loads of a thread are issued before the first
// use. BCAST = false: every input is as long as the output (no index arithmetic beyond the tile offset).
template <typename T, int NIN, bool BCAST, typename Op>
__global__ void __launch_bounds__(256, 4) ew_vec_kernel(T* out, const T* a0, const T* a1, const T* a2, int64_t numel, const VecPeriods per,
                                                        const Op op) {
    constexpr int V = Vec16<T>::N;
    constexpr int UNROLL = 4;
    const int64_t nvec = numel / V;
    const T* ins[3] = {a0, a1, a2};
    const int64_t base = static_cast<int64_t>(blockIdx.x) * (256 * UNROLL) + threadIdx.x;
    // A repeating input is indexed by (vector index mod period). One remainder per thread and input; the other three
    // vectors of the thread sit 256 vectors further on each, so their index follows by addition and a conditional wrap.
    int64_t rep[NIN > 0 ? NIN : 1];
    if constexpr (BCAST) {
#pragma unroll
        for (int a = 0; a < NIN; ++a) {
            rep[a] = 0;
            if (per.period[a] != 0) {
                rep[a] = per.narrow ? static_cast<int64_t>(static_cast<uint32_t>(base) % static_cast<uint32_t>(per.period[a])) : base % per.period[a];
            }
        }
    }
    Vec16<T> x[NIN > 0 ? NIN : 1][UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int64_t iv = base + u * 256;
        if (iv < nvec) {
#pragma unroll
            for (int a = 0; a < NIN; ++a) {
                if (!BCAST || per.period[a] == 0) {
                    x[a][u] = ld16_stream(ins[a] + iv * V);
                } else {
                    x[a][u] = ld16(ins[a] + rep[a] * V);
                }
            }
        }
        if constexpr (BCAST) {
#pragma unroll
            for (int a = 0; a < NIN; ++a) {
                if (per.period[a] != 0) {
                    rep[a] += 256;
                    if (per.period[a] >= 256) {
                        if (rep[a] >= per.period[a]) rep[a] -= per.period[a];
                    } else {
                        rep[a] %= per.period[a];  // short rows (fewer than 256 vectors): rare, small
                    }
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int64_t iv = base + u * 256;
        if (iv < nvec) {
            Vec16<T> r;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                float y;
                if constexpr (NIN == 0) y = op();
                else if constexpr (NIN == 1) y = op(to_f32(x[0][u].v[e]));
                else if constexpr (NIN == 2) y = op(to_f32(x[0][u].v[e]), to_f32(x[1][u].v[e]));
                else y = op(to_f32(x[0][u].v[e]), to_f32(x[1][u].v[e]), to_f32(x[2][u].v[e]));
                r.v[e] = from_f32<T>(y);
            }
            st16_stream(out + iv * V, r);
        }
    }
    // ragged tail (numel not a multiple of the vector width): one thread per element
    if (blockIdx.x == 0) {
        for (int64_t i = nvec * V + threadIdx.x; i < numel; i += blockDim.x) {
            float in[3] = {0.f, 0.f, 0.f};
#pragma unroll
            for (int a = 0; a < NIN; ++a) {
                const int64_t j = (!BCAST || per.period[a] == 0) ? i : i % (per.period[a] * V);
                in[a] = to_f32(ins[a][j]);
            }
            float y;
            if constexpr (NIN == 0) y = op();
            else if constexpr (NIN == 1) y = op(in[0]);
            else if constexpr (NIN == 2) y = op(in[0], in[1]);
            else y = op(in[0], in[1], in[2]);
            out[i] = from_f32<T>(y);
        }
    }
}

// Binary op whose input `REP` is a dense block that repeats along the leading dimensions (a [S, S] mask added to
// [B*H, S, S] scores). A CTA owns one 1024-vector tile of the block, keeps it in registers and streams the matching tile of
// every repetition through it, so the repeating operand is read once in total instead of once per repetition (and the L2
// carries only the streaming operand). gridDim.y splits the repetitions.
template <typename T, int REP, typename Op>
__global__ void __launch_bounds__(256, 4) ew_repeat_kernel(T* out, const T* dense, const T* block, int64_t period, int64_t reps, const Op op) {
    constexpr int V = Vec16<T>::N;
    constexpr int UNROLL = 4;
    const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * (256 * UNROLL) + threadIdx.x;
    Vec16<T> blk[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int64_t iv = tile0 + u * 256;
        if (iv < period) blk[u] = ld16(block + iv * V);
    }
    const int64_t per_y = (reps + gridDim.y - 1) / gridDim.y;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * per_y;
    const int64_t r1 = r0 + per_y < reps ? r0 + per_y : reps;
    for (int64_t r = r0; r < r1; ++r) {
        const int64_t base = r * period;
        Vec16<T> x[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t iv = tile0 + u * 256;
            if (iv < period) x[u] = ld16_stream(dense + (base + iv) * V);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t iv = tile0 + u * 256;
            if (iv < period) {
                Vec16<T> y;
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    const float a = to_f32(x[u].v[e]), b = to_f32(blk[u].v[e]);
                    y.v[e] = from_f32<T>(REP == 1 ? op(a, b) : op(b, a));
                }
                st16_stream(out + (base + iv) * V, y);
            }
        }
    }
}

// The same operation with one CTA per (tile of the block, repetition) and the block's vectors read through L2 (an 8 MB mask
// stays there): no loop, so every CTA has all its loads in flight at once like the plain vector kernel, and the grid's second
// dimension is the repetition, so no index needs a remainder. Preferred; the looping form above serves more than 65535
// repetitions.
template <typename T, int REP, typename Op>
__global__ void __launch_bounds__(256, 4) ew_repeat_tile_kernel(T* out, const T* dense, const T* block, int64_t period, const Op op) {
    constexpr int V = Vec16<T>::N;
    constexpr int UNROLL = 4;
    const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * (256 * UNROLL) + threadIdx.x;
    const int64_t base = static_cast<int64_t>(blockIdx.y) * period;
    Vec16<T> x[UNROLL], blk[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int64_t iv = tile0 + u * 256;
        if (iv < period) {
            x[u] = ld16_stream(dense + (base + iv) * V);
            blk[u] = ld16(block + iv * V);
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int64_t iv = tile0 + u * 256;
        if (iv < period) {
            Vec16<T> y;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float a = to_f32(x[u].v[e]), b = to_f32(blk[u].v[e]);
                y.v[e] = from_f32<T>(REP == 1 ? op(a, b) : op(b, a));
            }
            st16_stream(out + (base + iv) * V, y);
        }
    }
}

// ---- row kernel --------------------------------------------------------------------------------------------------------
// Operands of one 2- or 4-byte float dtype whose innermost run is dense (or, for an input, broadcast) while the outer
// dimensions have arbitrary pitches: transposed views ([B, S, h, D] read as [B, h, S, D]), slices, tables broadcast over
// batch and heads, outputs that keep the input's permutation. One thread moves 16-byte vectors; the outer index of a
// vector is decomposed with 32-bit divisions. This is what keeps an op-by-op rotary embedding on views near the
// bandwidth of the dense path instead of the element-at-a-time general kernel.
template <typename T, int NIN, typename Op>
__global__ void __launch_bounds__(256) ew_rows_kernel(const EwIter<NIN + 1> it, const uint32_t nvec, const uint32_t vec_per_row, const Op op) {
    constexpr int V = Vec16<T>::N;
    constexpr int UNROLL = 4;
    const int last = it.ndim - 1;
    const uint32_t base = blockIdx.x * (256u * UNROLL) + threadIdx.x;
    int64_t off[UNROLL][NIN + 1];
    bool live[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const uint32_t iv = base + u * 256u;
        live[u] = iv < nvec;
        uint32_t r = iv / vec_per_row;
        const uint32_t col = iv - r * vec_per_row;
#pragma unroll
        for (int a = 0; a <= NIN; ++a) off[u][a] = it.stride[a][last] != 0 ? static_cast<int64_t>(col) * V : 0;
        for (int d = last - 1; d >= 0; --d) {
            const uint32_t sh = static_cast<uint32_t>(it.shape[d]);
            const uint32_t q = r / sh;
            const uint32_t c = r - q * sh;
            r = q;
#pragma unroll
            for (int a = 0; a <= NIN; ++a) off[u][a] += static_cast<int64_t>(c) * it.stride[a][d];
        }
    }
    Vec16<T> x[NIN > 0 ? NIN : 1][UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        if (!live[u]) continue;
#pragma unroll
        for (int a = 0; a < NIN; ++a) {
            const T* p = static_cast<const T*>(it.ptr[a + 1]) + off[u][a + 1];
            if (it.stride[a + 1][last] != 0) {
                x[a][u] = ld16(p);
            } else {
                const T s = *p;  // one value for the whole row
#pragma unroll
                for (int e = 0; e < V; ++e) x[a][u].v[e] = s;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        if (!live[u]) continue;
        Vec16<T> y;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            float f;
            if constexpr (NIN == 0) f = op();
            else if constexpr (NIN == 1) f = op(to_f32(x[0][u].v[e]));
            else if constexpr (NIN == 2) f = op(to_f32(x[0][u].v[e]), to_f32(x[1][u].v[e]));
            else f = op(to_f32(x[0][u].v[e]), to_f32(x[1][u].v[e]), to_f32(x[2][u].v[e]));
            y.v[e] = from_f32<T>(f);
        }
        st16(static_cast<T*>(it.ptr[0]) + off[u][0], y);
    }
}

// Eligibility of the row kernel for an iterator built by build_iter: one float dtype everywhere, the output's innermost
// pitch 1, every input's innermost pitch 1 or 0, whole 16-byte vectors per row, 16-byte aligned vector addresses.
template <int NARGS>
inline bool rows_eligible(const EwIter<NARGS>& it, int64_t itemsize) {
    if (it.ndim < 1) return false;
    const int last = it.ndim - 1;
    const int64_t V = 16 / itemsize;
    if (it.stride[0][last] != 1 || it.shape[last] % V != 0) return false;
    if (it.numel / V >= 0xffffffffLL) return false;
    for (int a = 0; a < NARGS; ++a) {
        if (it.dtype[a] != it.dtype[0]) return false;
        const int64_t inner = it.stride[a][last];
        if (inner != 1 && inner != 0) return false;
        if (inner == 1) {
            if (reinterpret_cast<uintptr_t>(it.ptr[a]) % 16 != 0) return false;
            for (int d = 0; d < last; ++d) {
                if (it.stride[a][d] % V != 0) return false;
            }
        }
        for (int d = 0; d < last; ++d) {
            if (it.shape[d] >= 0x7fffffffLL) return false;
        }
    }
    return true;
}

template <typename T, int NIN, typename Op>
void launch_vec(const TensorView& out, const void* const* p, const VecPeriods& per, const Op& op, cudaStream_t stream) {
    constexpr int V = Vec16<T>::N;
    const int64_t nvec = out.numel / V;
    if constexpr (NIN == 2) {
        // exactly one repeating input, at least one full tile long, whole vectors only
        const int rep = (per.period[0] != 0 && per.period[1] == 0) ? 0 : ((per.period[1] != 0 && per.period[0] == 0) ? 1 : -1);
        if (rep >= 0 && per.period[rep] >= 1024 && out.numel % V == 0 && nvec % per.period[rep] == 0) {
            const int64_t period = per.period[rep], reps = nvec / period;
            const int64_t tiles = (period + 1023) / 1024;
            int64_t ysplit = (static_cast<int64_t>(sm_count()) * 8 + tiles - 1) / tiles;  // about eight CTAs per SM in total
            if (ysplit > reps) ysplit = reps;
            if (ysplit > 65535) ysplit = 65535;
            if (ysplit < 1) ysplit = 1;
            // one CTA per (tile, repetition) wherever the repetitions fit the grid's second dimension: mask add on the 2 GiB score
            // tensor 0.75 -> 0.62 ms (1.07 of the copy bandwidth) against the looping form below
            if (tiles <= 0x7fffffffLL && reps <= 65535) {
                dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(reps));
                T* o = static_cast<T*>(out.data);
                if (rep == 1) ew_repeat_tile_kernel<T, 1, Op><<<grid, 256, 0, stream>>>(o, static_cast<const T*>(p[0]), static_cast<const T*>(p[1]), period, op);
                else ew_repeat_tile_kernel<T, 0, Op><<<grid, 256, 0, stream>>>(o, static_cast<const T*>(p[1]), static_cast<const T*>(p[0]), period, op);
                return;
            }
            if (tiles <= 0x7fffffffLL) {
                dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(ysplit));
                T* o = static_cast<T*>(out.data);
                if (rep == 1) ew_repeat_kernel<T, 1, Op><<<grid, 256, 0, stream>>>(o, static_cast<const T*>(p[0]), static_cast<const T*>(p[1]), period, reps, op);
                else ew_repeat_kernel<T, 0, Op><<<grid, 256, 0, stream>>>(o, static_cast<const T*>(p[1]), static_cast<const T*>(p[0]), period, reps, op);
                return;
            }
        }
    }
    int64_t blocks = (nvec + 1023) / 1024;
    if (blocks < 1) blocks = 1;
    const unsigned grid = static_cast<unsigned>(blocks);
    const bool bcast = per.period[0] != 0 || per.period[1] != 0 || per.period[2] != 0;
    T* o = static_cast<T*>(out.data);
    const T* a0 = static_cast<const T*>(p[0]);
    const T* a1 = static_cast<const T*>(p[1]);
    const T* a2 = static_cast<const T*>(p[2]);
    if (bcast) ew_vec_kernel<T, NIN, true, Op><<<grid, 256, 0, stream>>>(o, a0, a1, a2, out.numel, per, op);
    else ew_vec_kernel<T, NIN, false, Op><<<grid, 256, 0, stream>>>(o, a0, a1, a2, out.numel, per, op);
}

// Does `in` qualify for the vector kernel against the dense output `out`? Fills the repeat period.
inline bool vec_operand_ok(const TensorView& out, const TensorView& in, int vec_elems, int64_t* period) {
    if (in.dtype != out.dtype || in.device != diopi_device) return false;
    if (!in.aligned(16) || !in.is_contiguous()) return false;
    if (in.numel == out.numel) {
        // same element count and dense: identical linear order only if shapes match after dropping 1s
        int i = 0, o = 0;
        while (true) {
            while (i < in.ndim && in.shape[i] == 1) ++i;
            while (o < out.ndim && out.shape[o] == 1) ++o;
            if (i == in.ndim || o == out.ndim) break;
            if (in.shape[i] != out.shape[o]) return false;
            ++i; ++o;
        }
        if (i != in.ndim || o != out.ndim) return false;
        *period = 0;
        return true;
    }
    // modulo broadcast: in's shape (leading 1s dropped) must equal the trailing dims of out
    int lead = 0;
    while (lead < in.ndim && in.shape[lead] == 1) ++lead;
    const int nd = in.ndim - lead;
    if (nd == 0 || nd > out.ndim) return false;
    for (int d = 0; d < nd; ++d) {
        if (in.shape[lead + d] != out.shape[out.ndim - nd + d]) return false;
    }
    if (in.numel % vec_elems != 0) return false;
    *period = in.numel / vec_elems;
    return true;
}

inline int ew_grid(int64_t work_items, int threads) {
    int64_t blocks = (work_items + threads - 1) / threads;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

// An op may name a cheaper functor for tensors stored in 16 bits (fast exponential / reciprocal whose error is far below
// the 8- or 11-bit output): specialise HalfOp<Op>. The default is the op itself.
template <template <typename> class OpT>
struct HalfOp {
    template <typename C>
    using type = OpT<C>;
};

// OpT<C> must be constructible from (const ScalarArgs&).
template <template <typename> class OpT, int NIN>
diopiError_t launch_elementwise(diopiContextHandle_t ctx, const char* name, const TensorView& out, const TensorView* const* ins,
                                const ScalarArgs& sargs, bool allow_vec = true) {
    if (out.numel == 0) return diopiSuccess;
    B200_CHECK(out.device == diopi_device, "%s: output must be a device tensor", name);
    for (int a = 0; a < NIN; ++a) {
        B200_CHECK(ins[a]->device == diopi_device, "%s: input %d is a host tensor with %lld elements; only 0-dim host scalars are accepted",
                   name, a, (long long)ins[a]->numel);
    }
    cudaStream_t stream = stream_of(ctx);

    // --- vector path ---
    const bool vec_dtype = out.dtype == diopi_dtype_bfloat16 || out.dtype == diopi_dtype_float16 || out.dtype == diopi_dtype_float32;
    if (allow_vec && vec_dtype && out.is_contiguous() && out.aligned(16)) {
        const int vec_elems = 16 / static_cast<int>(out.itemsize);
        VecPeriods per{{0, 0, 0}, 0};
        bool ok = true;
        for (int a = 0; a < NIN && ok; ++a) ok = vec_operand_ok(out, *ins[a], vec_elems, &per.period[a]);
        if (ok) {
            const int64_t nvec = out.numel / vec_elems;
            per.narrow = nvec < 0xffffffffLL ? 1 : 0;
            B200_CHECK((nvec + 1023) / 1024 <= 0x7fffffffLL, "%s: tensor too large", name);
            const void* p[3] = {nullptr, nullptr, nullptr};
            for (int a = 0; a < NIN; ++a) p[a] = ins[a]->data;
            using HOp = typename HalfOp<OpT>::template type<float>;
            if (out.dtype == diopi_dtype_bfloat16) launch_vec<bf16, NIN, HOp>(out, p, per, HOp(sargs), stream);
            else if (out.dtype == diopi_dtype_float16) launch_vec<fp16, NIN, HOp>(out, p, per, HOp(sargs), stream);
            else launch_vec<float, NIN, OpT<float>>(out, p, per, OpT<float>(sargs), stream);
            B200_LAUNCH_CHECK(name);
            return diopiSuccess;
        }
    }

    // --- general path ---
    EwIter<NIN + 1> it;
    B200_CHECK(build_iter<NIN + 1>(out, ins, &it), "%s: operand shapes cannot be broadcast to the output shape", name);
    if (allow_vec && vec_dtype && rows_eligible<NIN + 1>(it, out.itemsize)) {
        const int64_t V = 16 / out.itemsize;
        const uint32_t nvec = static_cast<uint32_t>(it.numel / V);
        const uint32_t vpr = static_cast<uint32_t>(it.shape[it.ndim - 1] / V);
        const unsigned grid = (nvec + 1023u) / 1024u;
        using HOp = typename HalfOp<OpT>::template type<float>;
        if (out.dtype == diopi_dtype_bfloat16) ew_rows_kernel<bf16, NIN, HOp><<<grid, 256, 0, stream>>>(it, nvec, vpr, HOp(sargs));
        else if (out.dtype == diopi_dtype_float16) ew_rows_kernel<fp16, NIN, HOp><<<grid, 256, 0, stream>>>(it, nvec, vpr, HOp(sargs));
        else ew_rows_kernel<float, NIN, OpT<float>><<<grid, 256, 0, stream>>>(it, nvec, vpr, OpT<float>(sargs));
        B200_LAUNCH_CHECK(name);
        return diopiSuccess;
    }
    const int threads = 256;
    const int grid = ew_grid(out.numel, threads);
    if (out.dtype == diopi_dtype_float64) {
        ew_generic_kernel<double, NIN, OpT<double>><<<grid, threads, 0, stream>>>(it, OpT<double>(sargs));
    } else if (is_floating(out.dtype)) {
        ew_generic_kernel<float, NIN, OpT<float>><<<grid, threads, 0, stream>>>(it, OpT<float>(sargs));
    } else if (is_integral(out.dtype, true)) {
        // bool outputs of float inputs (e.g. where/masked ops) still compute in the input domain
        bool float_in = false;
        for (int a = 0; a < NIN; ++a) float_in = float_in || is_floating(ins[a]->dtype);
        if (float_in) ew_generic_kernel<float, NIN, OpT<float>><<<grid, threads, 0, stream>>>(it, OpT<float>(sargs));
        else ew_generic_kernel<int64_t, NIN, OpT<int64_t>><<<grid, threads, 0, stream>>>(it, OpT<int64_t>(sargs));
    } else {
        B200_FAIL("%s: output dtype %s not supported", name, dtype_name(out.dtype));
    }
    B200_LAUNCH_CHECK(name);
    return diopiSuccess;
}

}  // namespace b200
