// Operators of a token-sampling loop: argmax, sort, top-k, cumulative sum, gather, multinomial, tensor indexing.
// Reference call sites: dipu/scripts/autogen_diopi_wrapper/diopi_functions.yaml:816-828 (topk), 1143-1175 (sort),
// 1199-1211 (multinomial), 1516-1519 (argmax), 1908-1912 (cumsum), 1923-1924 (gather), 2349-2382 (index, index_put_).
// Sizes are those of a logits matrix ([sequences, vocabulary], 32 k - 128 k columns): the kernels are one CTA per row
// and bound by latency / L2 traffic rather than HBM; results follow torch CPU semantics (ties resolved towards the lower
// index, NaN ordered above every number, stable ordering of equal keys).
//
// Every tensor is viewed as [outer, n, inner] with the operated dimension in the middle; inputs that are not dense are
// first made dense through the copy service.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cmath>
#include <vector>

#include "copy.h"
#include "device_utils.cuh"

namespace b200 {
namespace {

struct Slices {
    int64_t outer = 1, n = 1, inner = 1;
};

Slices slices_of(const TensorView& v, int64_t dim) {
    Slices s;
    if (v.ndim == 0) return s;
    s.n = v.shape[dim];
    for (int d = 0; d < dim; ++d) s.outer *= v.shape[d];
    for (int d = static_cast<int>(dim) + 1; d < v.ndim; ++d) s.inner *= v.shape[d];
    return s;
}

bool wrap_dim(int64_t* dim, int ndim) {
    const int64_t nd = ndim == 0 ? 1 : ndim;
    if (*dim < -nd || *dim >= nd) return false;
    if (*dim < 0) *dim += nd;
    return true;
}

// Order-preserving map of a value onto uint32: a < b  <=>  key(a) < key(b); NaN above everything (torch's sort order).
__device__ __forceinline__ uint32_t ordered_key_f32(float f) {
    if (f != f) return 0xffffffffu;
    const uint32_t u = (f == 0.f) ? 0u : __float_as_uint(f);  // -0.0 and +0.0 compare equal, so they share a key
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t load_key(const void* p, diopiDtype_t dt, int64_t i) {
    switch (dt) {
        case diopi_dtype_float32: return ordered_key_f32(static_cast<const float*>(p)[i]);
        case diopi_dtype_bfloat16: return ordered_key_f32(__bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]));
        case diopi_dtype_float16: return ordered_key_f32(__half2float(static_cast<const __half*>(p)[i]));
        case diopi_dtype_int32: return static_cast<uint32_t>(static_cast<const int32_t*>(p)[i]) ^ 0x80000000u;
        case diopi_dtype_int16: return static_cast<uint32_t>(static_cast<int32_t>(static_cast<const int16_t*>(p)[i])) ^ 0x80000000u;
        case diopi_dtype_int8: return static_cast<uint32_t>(static_cast<int32_t>(static_cast<const int8_t*>(p)[i])) ^ 0x80000000u;
        case diopi_dtype_uint8: case diopi_dtype_bool: return static_cast<const uint8_t*>(p)[i];
        default: return 0;
    }
}
// The value itself goes back out untouched (copied from the input element), so no inverse map is needed for storing.
bool key32_dtype(diopiDtype_t dt) {
    switch (dt) {
        case diopi_dtype_float32: case diopi_dtype_bfloat16: case diopi_dtype_float16: case diopi_dtype_int32: case diopi_dtype_int16:
        case diopi_dtype_int8: case diopi_dtype_uint8: case diopi_dtype_bool:
            return true;
        default:
            return false;
    }
}

__device__ __forceinline__ void copy_element(void* dst, int64_t di, const void* src, int64_t si, int itemsize) {
    switch (itemsize) {
        case 1: static_cast<uint8_t*>(dst)[di] = static_cast<const uint8_t*>(src)[si]; break;
        case 2: static_cast<uint16_t*>(dst)[di] = static_cast<const uint16_t*>(src)[si]; break;
        case 4: static_cast<uint32_t*>(dst)[di] = static_cast<const uint32_t*>(src)[si]; break;
        default: static_cast<uint64_t*>(dst)[di] = static_cast<const uint64_t*>(src)[si]; break;
    }
}

// ---- argmax ---------------------------------------------------------------------------------------------------------------
// One CTA per slice. The composite (key, ~index) makes "largest value, lowest index" a plain 64-bit maximum.
__global__ void __launch_bounds__(256) argmax_kernel(const void* in, diopiDtype_t dt, int64_t* out, Slices s) {
    __shared__ unsigned long long red[8];
    const int64_t slice = blockIdx.x;
    const int64_t o = slice / s.inner, k = slice - o * s.inner;
    const int64_t base = o * s.n * s.inner + k;
    unsigned long long best = 0;
    for (int64_t j = threadIdx.x; j < s.n; j += blockDim.x) {
        const unsigned long long c = (static_cast<unsigned long long>(load_key(in, dt, base + j * s.inner)) << 32) |
                                     static_cast<uint32_t>(~static_cast<uint32_t>(j));
        best = c > best ? c : best;
    }
    for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, off);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = red[w] > best ? red[w] : best;
        out[slice] = static_cast<int64_t>(~static_cast<uint32_t>(best & 0xffffffffu));
    }
}

// ---- cumulative sum ---------------------------------------------------------------------------------------------------------
// One CTA per slice; every thread owns a contiguous run, the run totals are scanned across the block, and the sequence is
// repeated for slices longer than one pass. C: accumulation type (float for 2- and 4-byte floats, double, int64).
template <typename C>
__global__ void __launch_bounds__(256) cumsum_kernel(const void* in, diopiDtype_t in_dt, void* out, diopiDtype_t out_dt, Slices s) {
    __shared__ C warp_tot[8];
    __shared__ C carry_s;
    const int64_t slice = blockIdx.x;
    const int64_t o = slice / s.inner, k = slice - o * s.inner;
    const int64_t base = o * s.n * s.inner + k;
    constexpr int RUN = 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry_s = C(0);
    __syncthreads();
    for (int64_t start = 0; start < s.n; start += 256 * RUN) {
        const int64_t j0 = start + static_cast<int64_t>(threadIdx.x) * RUN;
        C v[RUN];
        C run = C(0);
#pragma unroll
        for (int i = 0; i < RUN; ++i) {
            v[i] = (j0 + i < s.n) ? load_as<C>(in, in_dt, base + (j0 + i) * s.inner) : C(0);
            run += v[i];
            v[i] = run;  // inclusive within the run
        }
        // exclusive scan of the run totals across the block
        C incl = run;
        for (int off = 1; off < 32; off <<= 1) {
            const C t = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += t;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        C before = carry_s;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        before += incl - run;
#pragma unroll
        for (int i = 0; i < RUN; ++i) {
            if (j0 + i < s.n) store_from<C>(out, out_dt, base + (j0 + i) * s.inner, before + v[i]);
        }
        __syncthreads();
        if (threadIdx.x == 255) carry_s = before + run;
        __syncthreads();
    }
}

// ---- gather --------------------------------------------------------------------------------------------------------------------
// out[o, j, k] = self[o', index[o, j, k], k'] with the index tensor's own (possibly smaller) extents outside `dim`.
struct GatherIter {
    int ndim, dim;
    int64_t numel;
    int64_t idx_shape[kMaxDims];
    int64_t self_stride[kMaxDims];
    int64_t self_dim_size;
};

__global__ void __launch_bounds__(256) gather_kernel(const void* self, int itemsize, const int64_t* index, void* out, const GatherIter it) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < it.numel; i += step) {
        int64_t rem = i, off = 0;
        const int64_t ix = index[i];
        for (int d = it.ndim - 1; d >= 0; --d) {
            const int64_t q = rem / it.idx_shape[d];
            const int64_t c = rem - q * it.idx_shape[d];
            rem = q;
            off += (d == it.dim ? ix : c) * it.self_stride[d];
        }
        if (ix < 0 || ix >= it.self_dim_size) continue;  // torch raises here; on the device the element is left untouched
        copy_element(out, i, self, off, itemsize);
    }
}


// ---- sort / top-k -------------------------------------------------------------------------------------------------------------
// One CTA per slice sorts 64-bit composites (order-preserving key << 32 | position): equal keys keep their original order
// (the position breaks the tie), which is torch's stable order, and "descending" only flips the key bits. Slices of up to
// 4096 elements run a bitonic network in shared memory; longer ones the radix sort below; a small k of a long slice the
// radix selection. The first n_out sorted elements are written out (n_out = n for sort, k for top-k).
constexpr int kSortThreads = 1024;
constexpr int64_t kSortSmemElems = 4096;   // longer slices take the radix sort

struct SortArgs {
    const void* in;
    diopiDtype_t dt;
    int itemsize;
    void* values;        // may be nullptr
    int64_t* indices;    // may be nullptr
    Slices s;
    int64_t n_pad, n_out;
    uint32_t flip;       // 0xffffffff for descending
};

// One compare-exchange stage of the network over `count` elements of `buf` whose first element has global position `origin`
// (the direction of a pair depends on its global position and the size of the bitonic sequences being merged).
__device__ __forceinline__ void bitonic_stage(unsigned long long* buf, int64_t count, int64_t origin, int64_t size, int64_t stride) {
    const int64_t mask = stride - 1;
    for (int64_t t = threadIdx.x; t < (count >> 1); t += kSortThreads) {
        const int64_t i = ((t & ~mask) << 1) | (t & mask);
        const int64_t p = i + stride;
        const bool up = ((origin + i) & size) == 0;
        const unsigned long long x = buf[i], y = buf[p];
        if ((x > y) == up) {
            buf[i] = y;
            buf[p] = x;
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kSortThreads) sort_kernel(const SortArgs a) {
    __shared__ unsigned long long buf[kSortSmemElems];
    const int64_t slice = blockIdx.x;
    const int64_t o = slice / a.s.inner, k = slice - o * a.s.inner;
    const int64_t base = o * a.s.n * a.s.inner + k;
    for (int64_t j = threadIdx.x; j < a.n_pad; j += kSortThreads) {
        unsigned long long c = ~0ull;  // padding sorts to the end
        if (j < a.s.n) c = (static_cast<unsigned long long>(load_key(a.in, a.dt, base + j * a.s.inner) ^ a.flip) << 32) | static_cast<uint32_t>(j);
        buf[j] = c;
    }
    __syncthreads();
    for (int64_t size = 2; size <= a.n_pad; size <<= 1) {
        for (int64_t stride = size >> 1; stride > 0; stride >>= 1) bitonic_stage(buf, a.n_pad, 0, size, stride);
    }
    // output slice geometry: the operated dimension has n_out elements
    const int64_t obase = o * a.n_out * a.s.inner + k;
    for (int64_t r = threadIdx.x; r < a.n_out; r += kSortThreads) {
        const int64_t j = static_cast<int64_t>(buf[r] & 0xffffffffull);
        if (a.values != nullptr) copy_element(a.values, obase + r * a.s.inner, a.in, base + j * a.s.inner, a.itemsize);
        if (a.indices != nullptr) a.indices[obase + r * a.s.inner] = j;
    }
}

// ---- radix sort of long slices ------------------------------------------------------------------------------------------------
// Least-significant-digit radix sort, 8 bits per pass, one 1024-thread CTA per slice: four stable counting passes over
// (key, position) records that ping-pong between two workspace buffers (they stay in L2). Stability makes equal keys keep
// their original order, so the result is the same as the bitonic network's, at a fraction of its ~120 stages.
// A pass: histogram of the digit -> exclusive scan -> chunks of 1024 records in order, where a record's slot is
// (digit base) + (records of that digit in earlier chunks) + (in earlier warps of the chunk) + (in earlier lanes of the warp).
__global__ void __launch_bounds__(kSortThreads) radix_sort_kernel(const SortArgs a, unsigned long long* buf0, unsigned long long* buf1) {
    __shared__ unsigned int hist[256];          // digit base, then running base while the chunks are placed
    __shared__ unsigned short warp_cnt[32][256];  // per chunk: records of each digit in each warp
    const int64_t slice = blockIdx.x;
    const int64_t o = slice / a.s.inner, k = slice - o * a.s.inner;
    const int64_t base = o * a.s.n * a.s.inner + k;
    const int64_t n = a.s.n;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned long long* src = buf0 + slice * n;
    unsigned long long* dst = buf1 + slice * n;
    for (int64_t j = threadIdx.x; j < n; j += kSortThreads) {
        src[j] = (static_cast<unsigned long long>(load_key(a.in, a.dt, base + j * a.s.inner) ^ a.flip) << 32) | static_cast<uint32_t>(j);
    }
    __syncthreads();
    for (int shift = 32; shift < 64; shift += 8) {
        if (threadIdx.x < 256) hist[threadIdx.x] = 0;
        __syncthreads();
        for (int64_t j = threadIdx.x; j < n; j += kSortThreads) atomicAdd(&hist[(src[j] >> shift) & 255u], 1u);
        __syncthreads();
        if (warp == 0) {
            // exclusive scan of 256 counters by one warp: 8 per lane
            unsigned int v[8], sum = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = hist[lane * 8 + i];
                sum += v[i];
            }
            unsigned int incl = sum;
            for (int off = 1; off < 32; off <<= 1) {
                const unsigned int t = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += t;
            }
            unsigned int run = incl - sum;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                hist[lane * 8 + i] = run;
                run += v[i];
            }
        }
        __syncthreads();
        for (int64_t start = 0; start < n; start += kSortThreads) {
            for (int i = threadIdx.x; i < 32 * 256; i += kSortThreads) (&warp_cnt[0][0])[i] = 0;
            __syncthreads();
            const int64_t j = start + threadIdx.x;
            const bool live = j < n;
            unsigned long long rec = 0;
            unsigned int digit = 0x100u + lane;  // idle lanes: a value no live lane has, different per lane
            if (live) {
                rec = src[j];
                digit = static_cast<unsigned int>(rec >> shift) & 255u;
            }
            const unsigned int peers = __match_any_sync(0xffffffffu, digit);
            const unsigned int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
            if (live && rank_in_warp == 0) warp_cnt[warp][digit] = static_cast<unsigned short>(__popc(peers));
            __syncthreads();
            // per digit: the counts of the 32 warps become exclusive offsets inside the chunk; the chunk total stays in a register
            unsigned int chunk_total = 0;
            if (threadIdx.x < 256) {
                for (int w = 0; w < 32; ++w) {
                    const unsigned int c = warp_cnt[w][threadIdx.x];
                    warp_cnt[w][threadIdx.x] = static_cast<unsigned short>(chunk_total);
                    chunk_total += c;
                }
            }
            __syncthreads();
            if (live) dst[hist[digit] + warp_cnt[warp][digit] + rank_in_warp] = rec;
            __syncthreads();
            if (threadIdx.x < 256) hist[threadIdx.x] += chunk_total;   // the base moves past this chunk
            // (the next iteration's first barrier orders this update before anyone reads hist again)
        }
        __syncthreads();
        unsigned long long* t = src;
        src = dst;
        dst = t;
    }
    // four passes: the sorted records are back in buf0's half that `src` now names
    const int64_t obase = o * a.n_out * a.s.inner + k;
    for (int64_t r = threadIdx.x; r < a.n_out; r += kSortThreads) {
        const int64_t j = static_cast<int64_t>(src[r] & 0xffffffffull);
        if (a.values != nullptr) copy_element(a.values, obase + r * a.s.inner, a.in, base + j * a.s.inner, a.itemsize);
        if (a.indices != nullptr) a.indices[obase + r * a.s.inner] = j;
    }
}

// ---- top-k by radix selection -----------------------------------------------------------------------------------------------
// For k up to 2048 a full sort is wasted work: four passes over the slice with a 256-bin histogram each pin down the
// k-th key (most significant byte first), one more pass collects the k winners (everything beyond the threshold key plus, in
// position order, as many elements equal to it as are still needed), and only those are sorted. One CTA per slice; the
// slice is read five times (from L2 after the first pass) instead of going through ~120 network stages.
constexpr int kSelectMaxK = 2048;

__global__ void __launch_bounds__(kSortThreads) topk_select_kernel(const SortArgs a) {
    __shared__ unsigned int hist[256];
    __shared__ unsigned int sel_prefix, sel_remaining, n_taken, warp_cnt[32], tie_base;
    __shared__ unsigned long long cand[kSelectMaxK];
    const int64_t slice = blockIdx.x;
    const int64_t o = slice / a.s.inner, k = slice - o * a.s.inner;
    const int64_t base = o * a.s.n * a.s.inner + k;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        sel_prefix = 0;
        sel_remaining = static_cast<unsigned int>(a.n_out);
        n_taken = 0;
        tie_base = 0;
    }
    // with the flip applied the wanted elements are the n_out SMALLEST keys
    uint32_t mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (threadIdx.x < 256) hist[threadIdx.x] = 0;
        __syncthreads();
        const uint32_t prefix = sel_prefix;
        for (int64_t j = threadIdx.x; j < a.s.n; j += kSortThreads) {
            const uint32_t key = load_key(a.in, a.dt, base + j * a.s.inner) ^ a.flip;
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int rem = sel_remaining, cum = 0;
            int bkt = 0;
            for (; bkt < 256; ++bkt) {
                if (cum + hist[bkt] >= rem) break;
                cum += hist[bkt];
            }
            sel_prefix = prefix | (static_cast<uint32_t>(bkt) << shift);
            sel_remaining = rem - cum;   // still needed among the elements of the chosen bucket
        }
        mask |= 255u << shift;
        __syncthreads();
    }
    const uint32_t threshold = sel_prefix;     // the n_out-th smallest key
    const unsigned int need_ties = sel_remaining;  // how many elements EQUAL to it belong to the result (>= 1)
    // collect: keys below the threshold in any order, ties in position order
    for (int64_t start = 0; start < a.s.n; start += kSortThreads) {
        const int64_t j = start + threadIdx.x;
        uint32_t key = 0xffffffffu;
        bool below = false, tie = false;
        if (j < a.s.n) {
            key = load_key(a.in, a.dt, base + j * a.s.inner) ^ a.flip;
            below = key < threshold;
            tie = key == threshold;
        }
        if (below) {
            const unsigned int pos = atomicAdd(&n_taken, 1u);
            cand[pos] = (static_cast<unsigned long long>(key) << 32) | static_cast<uint32_t>(j);
        }
        const unsigned int ballot = __ballot_sync(0xffffffffu, tie);
        if (lane == 0) warp_cnt[warp] = __popc(ballot);
        __syncthreads();
        unsigned int before = tie_base;
        for (int w = 0; w < warp; ++w) before += warp_cnt[w];
        const unsigned int rank = before + __popc(ballot & ((1u << lane) - 1u));
        if (tie && rank < need_ties) {
            const unsigned int pos = atomicAdd(&n_taken, 1u);
            cand[pos] = (static_cast<unsigned long long>(key) << 32) | static_cast<uint32_t>(j);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int tot = 0;
            for (int w = 0; w < kSortThreads / 32; ++w) tot += warp_cnt[w];
            tie_base += tot;
        }
        __syncthreads();
    }
    // exactly n_out candidates; pad to a power of two and sort them
    int64_t n_pad = 2;
    while (n_pad < a.n_out) n_pad <<= 1;
    for (int64_t j = a.n_out + threadIdx.x; j < n_pad; j += kSortThreads) cand[j] = ~0ull;
    __syncthreads();
    for (int64_t size = 2; size <= n_pad; size <<= 1) {
        for (int64_t stride = size >> 1; stride > 0; stride >>= 1) bitonic_stage(cand, n_pad, 0, size, stride);
    }
    const int64_t obase = o * a.n_out * a.s.inner + k;
    for (int64_t r = threadIdx.x; r < a.n_out; r += kSortThreads) {
        const int64_t j = static_cast<int64_t>(cand[r] & 0xffffffffull);
        if (a.values != nullptr) copy_element(a.values, obase + r * a.s.inner, a.in, base + j * a.s.inner, a.itemsize);
        if (a.indices != nullptr) a.indices[obase + r * a.s.inner] = j;
    }
}

diopiError_t launch_sort(diopiContextHandle_t ctx, const char* name, const TensorView& x, int64_t dim, bool descending, int64_t n_out,
                         const TensorView* values, const TensorView* indices, cudaStream_t stream) {
    B200_CHECK(key32_dtype(x.dtype), "%s: dtype %s is not supported (floats up to 32 bits, integers up to 32 bits, bool)", name, dtype_name(x.dtype));
    const Slices s = slices_of(x, dim);
    if (s.outer * s.inner == 0 || n_out == 0) return diopiSuccess;
    B200_CHECK(s.n < (1ll << 31), "%s: dimension too long", name);
    B200_CHECK(s.outer * s.inner <= 0x7fffffffLL, "%s: too many slices", name);
    int64_t n_pad = 1;
    while (n_pad < s.n) n_pad <<= 1;
    if (n_pad < 2) n_pad = 2;
    SortArgs a;
    a.in = x.data;
    a.dt = x.dtype;
    a.itemsize = static_cast<int>(x.itemsize);
    a.values = values != nullptr ? values->data : nullptr;
    a.indices = indices != nullptr ? static_cast<int64_t*>(indices->data) : nullptr;
    a.s = s;
    a.n_pad = n_pad;
    a.n_out = n_out;
    a.flip = descending ? 0xffffffffu : 0u;
    if (n_out < s.n && n_out <= kSelectMaxK && s.n > 4096) {
        // a small part of a long slice is wanted (top-k, draws without replacement): select, then sort only the winners
        topk_select_kernel<<<static_cast<unsigned>(s.outer * s.inner), kSortThreads, 0, stream>>>(a);
        B200_LAUNCH_CHECK(name);
        return diopiSuccess;
    }
    if (s.n > 4096) {
        // long slices: radix sort on two workspace buffers of (key, position) records
        diopiTensorHandle_t ws = nullptr;
        const int64_t bytes = 2 * s.outer * s.inner * s.n * static_cast<int64_t>(sizeof(unsigned long long));
        B200_CHECK(diopiRequireBuffer(ctx, &ws, bytes, diopi_device) == diopiSuccess && ws != nullptr, "%s: workspace allocation failed", name);
        void* ptr = nullptr;
        B200_CHECK(diopiGetTensorData(ws, &ptr) == diopiSuccess && ptr != nullptr, "%s: workspace has no data pointer", name);
        unsigned long long* b0 = static_cast<unsigned long long*>(ptr);
        radix_sort_kernel<<<static_cast<unsigned>(s.outer * s.inner), kSortThreads, 0, stream>>>(a, b0, b0 + s.outer * s.inner * s.n);
        B200_LAUNCH_CHECK(name);
        return diopiSuccess;
    }
    sort_kernel<<<static_cast<unsigned>(s.outer * s.inner), kSortThreads, 0, stream>>>(a);
    B200_LAUNCH_CHECK(name);
    return diopiSuccess;
}

// ---- multinomial ---------------------------------------------------------------------------------------------------------------
// Counter-based generator (Philox 4x32, 10 rounds, Salmon et al. 2011): the key is the generator's seed, the counter is
// (stream index, generator offset), so a draw depends only on (seed, offset, row, sample) and not on the launch geometry.
struct Philox {
    uint32_t key[2];
    __device__ Philox(uint64_t seed) {
        key[0] = static_cast<uint32_t>(seed);
        key[1] = static_cast<uint32_t>(seed >> 32);
    }
    __device__ uint4 operator()(uint64_t index, uint64_t offset) const {
        uint32_t c0 = static_cast<uint32_t>(index), c1 = static_cast<uint32_t>(index >> 32), c2 = static_cast<uint32_t>(offset),
                 c3 = static_cast<uint32_t>(offset >> 32);
        uint32_t k0 = key[0], k1 = key[1];
#pragma unroll
        for (int r = 0; r < 10; ++r) {
            const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
            const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
            c0 = hi1 ^ c1 ^ k0;
            c1 = lo1;
            c2 = hi0 ^ c3 ^ k1;
            c3 = lo0;
            k0 += 0x9E3779B9u;
            k1 += 0xBB67AE85u;
        }
        return make_uint4(c0, c1, c2, c3);
    }
};
// [0, 1) with 24 random bits: never 1, so u * total stays below total
__device__ __forceinline__ float uniform24(uint32_t r) { return static_cast<float>(r >> 8) * (1.0f / 16777216.0f); }

// Draws with replacement from each row's (unnormalised) weights by inverting the cumulative sum: one CTA per row keeps the
// per-thread run totals and their block-wide prefix, then every sample is located by the thread whose run contains it.
__global__ void __launch_bounds__(256) multinomial_kernel(const void* probs, diopiDtype_t dt, int64_t n, int64_t num_samples, int64_t* out,
                                                          uint64_t seed, uint64_t offset) {
    __shared__ float prefix[257];
    __shared__ float runs[256];
    const int64_t row = blockIdx.x;
    const int64_t base = row * n;
    const int64_t len = (n + 255) / 256;
    const int64_t j0 = static_cast<int64_t>(threadIdx.x) * len;
    const int64_t j1 = j0 + len < n ? j0 + len : n;
    float run = 0.f;
    for (int64_t j = j0; j < j1; ++j) run += fmaxf(load_as<float>(probs, dt, base + j), 0.f);
    runs[threadIdx.x] = run;
    __syncthreads();
    // One thread adds the 256 run totals in order: prefix[t + 1] = prefix[t] + run[t] exactly, so the boundaries never
    // decrease, a run without positive weight owns the EMPTY interval, and the intervals tile [0, total) - none of which a
    // tree-shaped scan guarantees in floating point (a masked-out run could own a one-ulp interval and return a token of
    // weight zero).
    if (threadIdx.x == 0) {
        float c = 0.f;
        for (int t = 0; t < 256; ++t) {
            prefix[t] = c;
            c += runs[t];
        }
        prefix[256] = c;
    }
    __syncthreads();
    const float total = prefix[256];
    const Philox gen(seed);
    for (int64_t sidx = 0; sidx < num_samples; ++sidx) {
        const uint4 r = gen(static_cast<uint64_t>(row * num_samples + sidx), offset);
        float x = uniform24(r.x) * total;
        if (!(x < total)) x = 0.f;  // only when total is 0, inf or NaN: degenerate rows yield index of the first weight
        // the owner: x in [prefix[t], prefix[t+1]), non-empty only for a run that holds positive weight
        if (x >= prefix[threadIdx.x] && x < prefix[threadIdx.x + 1]) {
            float c = prefix[threadIdx.x];
            int64_t pick = -1, last_pos = -1;
            for (int64_t j = j0; j < j1; ++j) {
                const float w = fmaxf(load_as<float>(probs, dt, base + j), 0.f);
                if (w > 0.f) last_pos = j;
                c += w;
                if (x < c) {
                    pick = j;
                    break;
                }
            }
            if (pick < 0) pick = last_pos >= 0 ? last_pos : j0;  // rounding at the end of the run: its last positive weight
            out[row * num_samples + sidx] = pick;
        } else if (total <= 0.f && threadIdx.x == 0) {
            out[row * num_samples + sidx] = 0;
        }
    }
}

// Without replacement: the num_samples smallest of e_j / w_j with e_j ~ Exp(1) are a draw without replacement (exponential
// race); the keys are written here and ordered by the sort kernel.
__global__ void __launch_bounds__(256) race_keys_kernel(const void* probs, diopiDtype_t dt, int64_t total, float* keys, uint64_t seed,
                                                        uint64_t offset) {
    const Philox gen(seed);
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
        const float w = load_as<float>(probs, dt, i);
        const uint4 r = gen(static_cast<uint64_t>(i), offset);
        const float u = 1.0f - uniform24(r.x);  // (0, 1]
        keys[i] = w > 0.f ? -__logf(u) / w : INFINITY;
    }
}

// ---- tensor indexing -------------------------------------------------------------------------------------------------------------
// self[e_0, ..., e_{k-1}] where every e_d is an int64 index tensor, a boolean mask (which stands for as many index tensors as it
// has dimensions: the coordinates of its true elements, in row-major order) or "all of this dimension" (NULL; also every
// dimension after the last entry). The index tensors broadcast to one shape S. As in torch, S takes the place of the indexed
// dimensions when they are adjacent, and goes first when they are not. Negative indices wrap; out-of-range ones are skipped.
struct IndexIter {
    int nidx, ns, nout;                  // index tensors, dimensions of S, dimensions of the result
    int64_t numel;                       // elements of the result
    int64_t s_shape[kMaxDims];
    int64_t idx_stride[kMaxDims][kMaxDims];  // [index tensor][dimension of S], 0 where broadcast
    const int64_t* idx_ptr[kMaxDims];
    int64_t self_idx_stride[kMaxDims], self_idx_size[kMaxDims];
    int64_t out_shape[kMaxDims];
    int64_t out_self_stride[kMaxDims];   // kept dimensions: the stride in self
    int out_s_dim[kMaxDims];             // dimensions of S: which one; -1 for a kept dimension
};

__device__ __forceinline__ bool index_offset(const IndexIter& it, int64_t i, int64_t* self_off) {
    int64_t coord[kMaxDims];
    int64_t off = 0, rem = i;
    for (int d = it.nout - 1; d >= 0; --d) {
        const int64_t q = rem / it.out_shape[d];
        const int64_t c = rem - q * it.out_shape[d];
        rem = q;
        if (it.out_s_dim[d] >= 0) coord[it.out_s_dim[d]] = c;
        else off += c * it.out_self_stride[d];
    }
    for (int t = 0; t < it.nidx; ++t) {
        int64_t io = 0;
        for (int d = 0; d < it.ns; ++d) io += coord[d] * it.idx_stride[t][d];
        int64_t ix = it.idx_ptr[t][io];
        if (ix < 0) ix += it.self_idx_size[t];
        if (ix < 0 || ix >= it.self_idx_size[t]) return false;
        off += ix * it.self_idx_stride[t];
    }
    *self_off = off;
    return true;
}

// Coordinates of the true elements of a mask, in row-major order: coords[d * capacity + n] is coordinate d of the n-th true
// element; *count receives their number. One CTA walks the mask in chunks of its width with a block-wide scan per chunk
// (index masks are small; the order of the result is what matters).
struct MaskDesc {
    const uint8_t* data;
    int ndim;
    int64_t numel;
    int64_t shape[kMaxDims], stride[kMaxDims];
};
__global__ void __launch_bounds__(1024) mask_nonzero_kernel(const MaskDesc m, int64_t* coords, int64_t capacity, int64_t* count) {
    __shared__ int warp_tot[32];
    __shared__ int64_t base;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int64_t c0 = 0; c0 < m.numel; c0 += blockDim.x) {
        const int64_t i = c0 + threadIdx.x;
        int64_t cd[kMaxDims];
        int flag = 0;
        if (i < m.numel) {
            int64_t off = 0, rem = i;
            for (int d = m.ndim - 1; d >= 0; --d) {
                const int64_t q = rem / m.shape[d];
                cd[d] = rem - q * m.shape[d];
                off += cd[d] * m.stride[d];
                rem = q;
            }
            flag = m.data[off] != 0 ? 1 : 0;
        }
        int incl = flag;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) {
            if (w < warp) before += warp_tot[w];
            total += warp_tot[w];
        }
        if (flag) {
            const int64_t n = base + before + incl - 1;
            for (int d = 0; d < m.ndim; ++d) coords[d * capacity + n] = cd[d];
        }
        __syncthreads();
        if (threadIdx.x == 0) base += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) *count = base;
}

__global__ void __launch_bounds__(256) index_get_kernel(const void* self, int itemsize, void* out, const IndexIter it) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < it.numel; i += step) {
        int64_t off;
        if (index_offset(it, i, &off)) copy_element(out, i, self, off, itemsize);
    }
}

template <typename T>
__device__ __forceinline__ void atomic_add_as(T* p, T v) { atomicAdd(p, v); }
template <>
__device__ __forceinline__ void atomic_add_as<int64_t>(int64_t* p, int64_t v) {
    atomicAdd(reinterpret_cast<unsigned long long*>(p), static_cast<unsigned long long>(v));
}

// values: element i of the broadcast value tensor sits at offset sum(coord * val_stride) - passed as a dense tensor here.
template <typename T, bool ACC>
__global__ void __launch_bounds__(256) index_put_kernel(T* self, const T* values, const IndexIter it) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < it.numel; i += step) {
        int64_t off;
        if (!index_offset(it, i, &off)) continue;
        if constexpr (ACC) atomic_add_as<T>(self + off, values[i]);
        else self[off] = values[i];
    }
}

// Fills an IndexIter from the index handles (NULL = the whole dimension, boolean masks are turned into the coordinates of
// their true elements first - this reads their count back and therefore synchronises the stream). Returns false with the error
// string set when the indices do not fit the tensor.
bool build_index_iter(diopiContextHandle_t ctx, const char* name, const TensorView& self, diopiConstTensorHandle_t* indices, int64_t nums,
                      IndexIter* it) {
    if (nums < 0 || nums > kMaxDims) {
        set_last_error("%s: %lld index entries", name, static_cast<long long>(nums));
        return false;
    }
    // one entry per dimension of self: an int64 index tensor (as a view) or nothing
    TensorView entry[kMaxDims];
    bool has[kMaxDims] = {false};
    int dim = 0;
    cudaStream_t stream = stream_of(ctx);
    for (int64_t t = 0; t < nums; ++t) {
        if (indices[t] == nullptr) {
            if (dim >= self.ndim) {
                set_last_error("%s: too many indices for a %d-dimensional tensor", name, self.ndim);
                return false;
            }
            ++dim;
            continue;
        }
        TensorView v;
        if (!make_view(indices[t], &v, "index")) return false;
        if (v.device != diopi_device) {
            set_last_error("%s: index tensors must be device tensors", name);
            return false;
        }
        if (v.dtype == diopi_dtype_int64) {
            if (dim >= self.ndim) {
                set_last_error("%s: too many indices for a %d-dimensional tensor", name, self.ndim);
                return false;
            }
            entry[dim] = v;
            has[dim++] = true;
            continue;
        }
        if (v.dtype != diopi_dtype_bool && v.dtype != diopi_dtype_uint8) {
            set_last_error("%s: index tensors must be int64 tensors or boolean masks (got %s)", name, dtype_name(v.dtype));
            return false;
        }
        // a mask of m dimensions indexes m dimensions of self with the coordinates of its true elements
        const int m = v.ndim == 0 ? 1 : v.ndim;
        if (dim + m > self.ndim) {
            set_last_error("%s: too many indices for a %d-dimensional tensor", name, self.ndim);
            return false;
        }
        for (int d = 0; d < v.ndim; ++d) {
            if (v.shape[d] != self.shape[dim + d]) {
                set_last_error("%s: the mask's shape does not match the indexed dimensions", name);
                return false;
            }
        }
        int64_t count = 0;
        int64_t* coords = nullptr;
        const int64_t capacity = v.numel > 0 ? v.numel : 1;
        if (v.numel > 0) {
            diopiTensorHandle_t ws = nullptr;
            void* wsp = nullptr;
            if (diopiRequireBuffer(ctx, &ws, (static_cast<int64_t>(m) * capacity + 1) * 8, diopi_device) != diopiSuccess || ws == nullptr ||
                diopiGetTensorData(ws, &wsp) != diopiSuccess || wsp == nullptr) {
                set_last_error("%s: workspace allocation for a mask failed", name);
                return false;
            }
            coords = static_cast<int64_t*>(wsp);
            MaskDesc md;
            md.data = static_cast<const uint8_t*>(v.data);
            md.ndim = v.ndim;
            md.numel = v.numel;
            for (int d = 0; d < v.ndim; ++d) { md.shape[d] = v.shape[d]; md.stride[d] = v.stride[d]; }
            mask_nonzero_kernel<<<1, 1024, 0, stream>>>(md, coords, capacity, coords + static_cast<int64_t>(m) * capacity);
            if (cudaMemcpyAsync(&count, coords + static_cast<int64_t>(m) * capacity, 8, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
                cudaStreamSynchronize(stream) != cudaSuccess) {
                (void)cudaGetLastError();
                set_last_error("%s: reading a mask's element count failed", name);
                return false;
            }
        }
        for (int d = 0; d < m; ++d) {
            TensorView c;
            c.data = coords != nullptr ? static_cast<void*>(coords + static_cast<int64_t>(d) * capacity) : nullptr;
            c.dtype = diopi_dtype_int64;
            c.device = diopi_device;
            c.itemsize = 8;
            c.ndim = 1;
            c.shape[0] = count;
            c.stride[0] = 1;
            c.numel = count;
            c.defined = true;
            entry[dim] = c;
            has[dim++] = true;
        }
    }
    // broadcast shape S of the index tensors
    int ns = 0, nidx = 0, first = -1, last = -1;
    for (int d = 0; d < self.ndim; ++d) {
        if (!has[d]) continue;
        ns = entry[d].ndim > ns ? entry[d].ndim : ns;
        if (first < 0) first = d;
        last = d;
        ++nidx;
    }
    it->nidx = nidx;
    it->ns = ns;
    for (int d = 0; d < ns; ++d) it->s_shape[d] = 1;
    for (int d0 = 0; d0 < self.ndim; ++d0) {
        if (!has[d0]) continue;
        const TensorView& v = entry[d0];
        for (int d = 0; d < v.ndim; ++d) {
            const int sd = ns - v.ndim + d;
            if (v.shape[d] != 1) {
                if (it->s_shape[sd] != 1 && it->s_shape[sd] != v.shape[d]) {
                    set_last_error("%s: index tensors cannot be broadcast together", name);
                    return false;
                }
                it->s_shape[sd] = v.shape[d];
            }
        }
    }
    int t = 0;
    bool adjacent = true;
    for (int d = 0; d < self.ndim; ++d) {
        if (!has[d]) {
            if (first >= 0 && d > first && d < last) adjacent = false;
            continue;
        }
        const TensorView& v = entry[d];
        for (int k = 0; k < ns; ++k) it->idx_stride[t][k] = 0;
        for (int k = 0; k < v.ndim; ++k) it->idx_stride[t][ns - v.ndim + k] = v.shape[k] == 1 ? 0 : v.stride[k];
        it->idx_ptr[t] = static_cast<const int64_t*>(v.data);
        it->self_idx_stride[t] = self.stride[d];
        it->self_idx_size[t] = self.shape[d];
        ++t;
    }
    // result dimensions: kept dimensions before the indexed ones, S, kept dimensions after - or S first when the indexed
    // dimensions are not adjacent
    int nout = 0;
    auto put_kept = [&](int d) {
        it->out_shape[nout] = self.shape[d];
        it->out_self_stride[nout] = self.stride[d];
        it->out_s_dim[nout++] = -1;
    };
    auto put_s = [&]() {
        for (int k = 0; k < ns; ++k) {
            it->out_shape[nout] = it->s_shape[k];
            it->out_self_stride[nout] = 0;
            it->out_s_dim[nout++] = k;
        }
    };
    const int kept = self.ndim - nidx;
    if (kept + ns > kMaxDims) {
        set_last_error("%s: the result has too many dimensions", name);
        return false;
    }
    if (nidx == 0) {
        for (int d = 0; d < self.ndim; ++d) put_kept(d);
    } else if (adjacent) {
        for (int d = 0; d < first; ++d) put_kept(d);
        put_s();
        for (int d = last + 1; d < self.ndim; ++d) put_kept(d);
    } else {
        put_s();
        for (int d = 0; d < self.ndim; ++d) {
            if (!has[d]) put_kept(d);
        }
    }
    it->nout = nout;
    it->numel = 1;
    for (int d = 0; d < nout; ++d) it->numel *= it->out_shape[d];
    return true;
}

bool shape_matches_except(const TensorView& a, const TensorView& b, int64_t dim, int64_t b_dim_size) {
    if (a.ndim != b.ndim) return false;
    for (int d = 0; d < a.ndim; ++d) {
        const int64_t want = d == dim ? b_dim_size : a.shape[d];
        if (b.shape[d] != want) return false;
    }
    return true;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

diopiError_t diopiArgmax(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, const int64_t* dim, bool keepdim) {
    (void)keepdim;  // the host has shaped `out`; only its element count matters here
    B200_VIEW(vo, out);
    B200_VIEW(vx_raw, input);
    B200_CHECK(vo.dtype == diopi_dtype_int64 && vo.is_contiguous(), "diopiArgmax: out must be a dense int64 tensor");
    B200_CHECK(key32_dtype(vx_raw.dtype), "diopiArgmax: dtype %s is not supported", dtype_name(vx_raw.dtype));
    B200_CHECK(vx_raw.numel > 0, "diopiArgmax: empty input");
    TensorView vx;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    Slices s;
    if (dim == nullptr) {
        s.n = vx.numel;  // the flattened tensor is one slice
    } else {
        int64_t d = *dim;
        B200_CHECK(wrap_dim(&d, vx.ndim), "diopiArgmax: dim %lld out of range", static_cast<long long>(*dim));
        s = slices_of(vx, d);
    }
    B200_CHECK(vo.numel == s.outer * s.inner, "diopiArgmax: out has %lld elements, expected %lld", static_cast<long long>(vo.numel),
               static_cast<long long>(s.outer * s.inner));
    B200_CHECK(s.n < (1ll << 32) && s.outer * s.inner <= 0x7fffffffLL, "diopiArgmax: tensor too large");
    argmax_kernel<<<static_cast<unsigned>(s.outer * s.inner), 256, 0, stream_of(ctx)>>>(vx.data, vx.dtype, static_cast<int64_t*>(vo.data), s);
    B200_LAUNCH_CHECK("diopiArgmax");
    return diopiSuccess;
}

diopiError_t diopiCumsum(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, int64_t dim) {
    B200_VIEW(vo, out);
    B200_VIEW(vx_raw, input);
    B200_CHECK(vo.numel == vx_raw.numel && vo.is_contiguous(), "diopiCumsum: out must be dense and of the input's size");
    if (vo.numel == 0) return diopiSuccess;
    B200_CHECK(wrap_dim(&dim, vx_raw.ndim), "diopiCumsum: dim out of range");
    TensorView vx;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    const Slices s = slices_of(vx, dim);
    B200_CHECK(s.outer * s.inner <= 0x7fffffffLL, "diopiCumsum: too many slices");
    const unsigned grid = static_cast<unsigned>(s.outer * s.inner);
    cudaStream_t stream = stream_of(ctx);
    if (vo.dtype == diopi_dtype_float64) cumsum_kernel<double><<<grid, 256, 0, stream>>>(vx.data, vx.dtype, vo.data, vo.dtype, s);
    else if (is_floating(vo.dtype)) cumsum_kernel<float><<<grid, 256, 0, stream>>>(vx.data, vx.dtype, vo.data, vo.dtype, s);
    else if (is_integral(vo.dtype, true)) cumsum_kernel<int64_t><<<grid, 256, 0, stream>>>(vx.data, vx.dtype, vo.data, vo.dtype, s);
    else B200_FAIL("diopiCumsum: output dtype %s not supported", dtype_name(vo.dtype));
    B200_LAUNCH_CHECK("diopiCumsum");
    return diopiSuccess;
}

diopiError_t diopiGather(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, int64_t dim, diopiConstTensorHandle_t index) {
    B200_VIEW(vo, out);
    B200_VIEW(vx, input);
    B200_VIEW(vi_raw, index);
    B200_CHECK(vi_raw.dtype == diopi_dtype_int64, "diopiGather: index must be int64");
    B200_CHECK(vo.dtype == vx.dtype && vo.is_contiguous() && vo.numel == vi_raw.numel, "diopiGather: out must be dense, of the input's dtype and the index's size");
    if (vo.numel == 0) return diopiSuccess;
    B200_CHECK(wrap_dim(&dim, vx.ndim), "diopiGather: dim out of range");
    B200_CHECK(vi_raw.ndim == vx.ndim || (vx.ndim == 0 && vi_raw.ndim <= 1), "diopiGather: index must have the input's number of dimensions");
    TensorView vi;
    if (make_contiguous(ctx, vi_raw, &vi) != diopiSuccess) return diopiErrorOccurred;
    GatherIter it;
    it.ndim = vx.ndim;
    it.dim = static_cast<int>(dim);
    it.numel = vi.numel;
    it.self_dim_size = vx.ndim == 0 ? 1 : vx.shape[dim];
    for (int d = 0; d < vx.ndim; ++d) {
        B200_CHECK(d == dim || vi.shape[d] <= vx.shape[d], "diopiGather: index extent %d exceeds the input's", d);
        it.idx_shape[d] = vi.shape[d];
        it.self_stride[d] = vx.stride[d];
    }
    const int grid = static_cast<int>(std::min<int64_t>((vi.numel + 255) / 256, static_cast<int64_t>(sm_count()) * 32));
    gather_kernel<<<grid, 256, 0, stream_of(ctx)>>>(vx.data, static_cast<int>(vx.itemsize), static_cast<const int64_t*>(vi.data), vo.data, it);
    B200_LAUNCH_CHECK("diopiGather");
    return diopiSuccess;
}

diopiError_t diopiSort(diopiContextHandle_t ctx, diopiTensorHandle_t values, diopiTensorHandle_t indices, diopiConstTensorHandle_t input, int64_t dim,
                       bool descending, const bool* stable) {
    (void)stable;  // the order is always the stable one
    B200_VIEW(vv, values);
    B200_VIEW(vi, indices);
    B200_VIEW(vx_raw, input);
    B200_CHECK(wrap_dim(&dim, vx_raw.ndim), "diopiSort: dim out of range");
    B200_CHECK(vv.dtype == vx_raw.dtype && vv.is_contiguous() && vv.numel == vx_raw.numel, "diopiSort: values must be dense with the input's dtype and size");
    B200_CHECK(vi.dtype == diopi_dtype_int64 && vi.is_contiguous() && vi.numel == vx_raw.numel, "diopiSort: indices must be dense int64 of the input's size");
    if (vx_raw.numel == 0) return diopiSuccess;
    TensorView vx;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    const int64_t n = vx.ndim == 0 ? 1 : vx.shape[dim];
    return launch_sort(ctx, "diopiSort", vx, dim, descending, n, &vv, &vi, stream_of(ctx));
}

diopiError_t diopiTopk(diopiContextHandle_t ctx, diopiTensorHandle_t values, diopiTensorHandle_t indices, diopiConstTensorHandle_t input, int64_t k,
                       int64_t dim, bool largest, bool sorted) {
    (void)sorted;  // the result is always in sorted order, which satisfies both settings
    B200_VIEW(vv, values);
    B200_VIEW(vi, indices);
    B200_VIEW(vx_raw, input);
    B200_CHECK(wrap_dim(&dim, vx_raw.ndim), "diopiTopk: dim out of range");
    const int64_t n = vx_raw.ndim == 0 ? 1 : vx_raw.shape[dim];
    B200_CHECK(k >= 0 && k <= n, "diopiTopk: k = %lld is outside [0, %lld]", static_cast<long long>(k), static_cast<long long>(n));
    B200_CHECK(vv.dtype == vx_raw.dtype && vv.is_contiguous() && vi.dtype == diopi_dtype_int64 && vi.is_contiguous(),
               "diopiTopk: values (input dtype) and indices (int64) must be dense");
    B200_CHECK(vx_raw.ndim == 0 || (shape_matches_except(vx_raw, vv, dim, k) && shape_matches_except(vx_raw, vi, dim, k)),
               "diopiTopk: values / indices must have the input's shape with k along dim");
    if (vx_raw.numel == 0 || k == 0) return diopiSuccess;
    TensorView vx;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    return launch_sort(ctx, "diopiTopk", vx, dim, largest, k, &vv, &vi, stream_of(ctx));
}


diopiError_t diopiMultinomial(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, int64_t num_samples, bool replacement,
                              diopiGeneratorHandle_t generator) {
    B200_VIEW(vo, out);
    B200_VIEW(vx_raw, input);
    B200_CHECK(vx_raw.ndim == 1 || vx_raw.ndim == 2, "diopiMultinomial: weights must be a vector or a matrix");
    B200_CHECK(is_floating(vx_raw.dtype) && vx_raw.dtype != diopi_dtype_float64, "diopiMultinomial: weights must be float16 / bfloat16 / float32");
    const int64_t rows = vx_raw.ndim == 2 ? vx_raw.shape[0] : 1;
    const int64_t n = vx_raw.shape[vx_raw.ndim - 1];
    B200_CHECK(num_samples > 0 && n > 0, "diopiMultinomial: needs at least one category and one sample");
    B200_CHECK(replacement || num_samples <= n, "diopiMultinomial: cannot draw %lld samples without replacement from %lld categories",
               static_cast<long long>(num_samples), static_cast<long long>(n));
    B200_CHECK(vo.dtype == diopi_dtype_int64 && vo.is_contiguous() && vo.numel == rows * num_samples,
               "diopiMultinomial: out must be dense int64 with rows x num_samples elements");
    if (rows == 0) return diopiSuccess;
    B200_CHECK(rows <= 0x7fffffffLL, "diopiMultinomial: too many rows");
    TensorView vx;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    // Generator state: the host's generator when given (its offset advances by the draws consumed, in multiples of 4),
    // else a library-wide default stream.
    static std::atomic<uint64_t> default_offset{0};
    uint64_t seed = 67280421310721ull, offset = 0;
    if (generator != nullptr) {
        B200_CHECK(diopiGeneratorGetSeedAndOffset(generator, &seed, &offset) == diopiSuccess, "diopiMultinomial: cannot read the generator");
    } else {
        offset = default_offset.load();
    }
    const uint64_t draws = static_cast<uint64_t>(replacement || num_samples == 1 ? rows * num_samples : rows * n);
    const uint64_t advance = (draws + 3) / 4 * 4;
    if (generator != nullptr) {
        B200_CHECK(diopiGeneratorSetSeedAndOffset(generator, seed, offset + advance) == diopiSuccess, "diopiMultinomial: cannot advance the generator");
    } else {
        default_offset.fetch_add(advance);
    }
    cudaStream_t stream = stream_of(ctx);
    if (replacement || num_samples == 1) {
        multinomial_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(vx.data, vx.dtype, n, num_samples, static_cast<int64_t*>(vo.data), seed, offset);
        B200_LAUNCH_CHECK("diopiMultinomial");
        return diopiSuccess;
    }
    diopiTensorHandle_t ws = nullptr;
    B200_CHECK(diopiRequireBuffer(ctx, &ws, rows * n * static_cast<int64_t>(sizeof(float)), diopi_device) == diopiSuccess && ws != nullptr,
               "diopiMultinomial: workspace allocation failed");
    void* keys = nullptr;
    B200_CHECK(diopiGetTensorData(ws, &keys) == diopiSuccess && keys != nullptr, "diopiMultinomial: workspace has no data pointer");
    const int grid = static_cast<int>(std::min<int64_t>((rows * n + 255) / 256, static_cast<int64_t>(sm_count()) * 32));
    race_keys_kernel<<<grid, 256, 0, stream>>>(vx.data, vx.dtype, rows * n, static_cast<float*>(keys), seed, offset);
    B200_LAUNCH_CHECK("diopiMultinomial");
    TensorView kv;
    kv.data = keys;
    kv.dtype = diopi_dtype_float32;
    kv.ndim = 2;
    kv.shape[0] = rows;
    kv.shape[1] = n;
    kv.stride[0] = n;
    kv.stride[1] = 1;
    kv.numel = rows * n;
    kv.itemsize = 4;
    kv.defined = true;
    return launch_sort(ctx, "diopiMultinomial", kv, 1, /*descending=*/false, num_samples, nullptr, &vo, stream);
}

diopiError_t diopiIndex(diopiContextHandle_t ctx, diopiTensorHandle_t* out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t* indices, int64_t nums) {
    B200_CHECK(out != nullptr && indices != nullptr, "diopiIndex: null argument");
    B200_VIEW(vx, input);
    IndexIter it;
    if (!build_index_iter(ctx, "diopiIndex", vx, indices, nums, &it)) return diopiErrorOccurred;
    int64_t shape[kMaxDims];
    const int nd = it.nout;
    for (int d = 0; d < nd; ++d) shape[d] = it.out_shape[d];
    diopiSize_t size;
    size.data = shape;
    size.len = nd;
    // the library allocates the result (`&out_ptr` in the reference's wrapper): it belongs to the host afterwards
    B200_CHECK(diopiRequireTensor(ctx, out, &size, nullptr, vx.dtype, diopi_device) == diopiSuccess && *out != nullptr, "diopiIndex: cannot allocate the result");
    if (it.numel == 0) return diopiSuccess;
    B200_VIEW(vo, *out);
    const int grid = static_cast<int>(std::min<int64_t>((it.numel + 255) / 256, static_cast<int64_t>(sm_count()) * 32));
    index_get_kernel<<<grid, 256, 0, stream_of(ctx)>>>(vx.data, static_cast<int>(vx.itemsize), vo.data, it);
    B200_LAUNCH_CHECK("diopiIndex");
    return diopiSuccess;
}

diopiError_t diopiIndexPutInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, diopiConstTensorHandle_t values, diopiConstTensorHandle_t* indices,
                              int64_t nums, bool accumulate) {
    B200_CHECK(indices != nullptr, "diopiIndexPutInp: null argument");
    B200_VIEW(vx, input);
    B200_VIEW(vv_raw, values);
    B200_CHECK(vv_raw.dtype == vx.dtype, "diopiIndexPutInp: values must have the tensor's dtype");
    IndexIter it;
    if (!build_index_iter(ctx, "diopiIndexPutInp", vx, indices, nums, &it)) return diopiErrorOccurred;
    if (it.numel == 0) return diopiSuccess;
    // values broadcast to S + rest, materialised dense (a scalar or a row is the common case and tiny)
    TensorView target;
    target.dtype = vx.dtype;
    target.itemsize = vx.itemsize;
    target.device = diopi_device;
    target.ndim = it.nout;
    for (int d = 0; d < it.nout; ++d) target.shape[d] = it.out_shape[d];
    int64_t st = 1;
    for (int d = target.ndim - 1; d >= 0; --d) {
        target.stride[d] = st;
        st *= target.shape[d];
    }
    target.numel = it.numel;
    target.defined = true;
    diopiTensorHandle_t ws = nullptr;
    B200_CHECK(diopiRequireBuffer(ctx, &ws, it.numel * vx.itemsize, diopi_device) == diopiSuccess && ws != nullptr, "diopiIndexPutInp: workspace allocation failed");
    B200_CHECK(diopiGetTensorData(ws, &target.data) == diopiSuccess && target.data != nullptr, "diopiIndexPutInp: workspace has no data pointer");
    if (copy_impl(ctx, vv_raw, target) != diopiSuccess) return diopiErrorOccurred;
    const int grid = static_cast<int>(std::min<int64_t>((it.numel + 255) / 256, static_cast<int64_t>(sm_count()) * 32));
    cudaStream_t stream = stream_of(ctx);
#define B200_PUT(T)                                                                                                             \
    do {                                                                                                                        \
        if (accumulate) index_put_kernel<T, true><<<grid, 256, 0, stream>>>(static_cast<T*>(vx.data), static_cast<const T*>(target.data), it); \
        else index_put_kernel<T, false><<<grid, 256, 0, stream>>>(static_cast<T*>(vx.data), static_cast<const T*>(target.data), it);           \
    } while (0)
    switch (vx.dtype) {
        case diopi_dtype_float32: B200_PUT(float); break;
        case diopi_dtype_bfloat16: B200_PUT(__nv_bfloat16); break;
        case diopi_dtype_float16: B200_PUT(__half); break;
        case diopi_dtype_int32: B200_PUT(int); break;
        case diopi_dtype_int64: B200_PUT(int64_t); break;
        default:
            B200_CHECK(!accumulate, "diopiIndexPutInp: accumulate is supported for float32 / float16 / bfloat16 / int32 / int64 only");
            if (vx.itemsize == 1) index_put_kernel<uint8_t, false><<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(vx.data), static_cast<const uint8_t*>(target.data), it);
            else if (vx.itemsize == 2) index_put_kernel<uint16_t, false><<<grid, 256, 0, stream>>>(static_cast<uint16_t*>(vx.data), static_cast<const uint16_t*>(target.data), it);
            else if (vx.itemsize == 8) index_put_kernel<double, false><<<grid, 256, 0, stream>>>(static_cast<double*>(vx.data), static_cast<const double*>(target.data), it);
            else B200_FAIL("diopiIndexPutInp: dtype %s not supported", dtype_name(vx.dtype));
    }
#undef B200_PUT
    B200_LAUNCH_CHECK("diopiIndexPutInp");
    return diopiSuccess;
}

}  // extern "C"
