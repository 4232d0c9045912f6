// diopiCopyInp and friends: dtype cast, layout change (transpose materialisation, KV append), broadcast
// expansion, peer copies; plus the index-driven movers (index_select / embedding, cat, triu, arange).
//
// Path selection for a copy, fastest first:
//   1. same dtype, both dense in the same order       -> cudaMemcpyAsync (device copy engine / SM copy)
//   2. dense cast between bf16 / fp16 / fp32          -> cast_vec_kernel, 128-bit accesses on the narrow side
//   3. same dtype, innermost run dense on both sides  -> strided copy of 16-byte (or 8/4/2-byte) words
//   4. everything else                                -> the general element-wise kernel (convert per element)
#include "copy.h"

#include "elementwise.cuh"

namespace b200 {
namespace {

template <typename C>
struct OpCopy {
    explicit OpCopy(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C a) const { return a; }
};

// ---- 2. dense cast --------------------------------------------------------------------------------------
template <typename S, typename D>
__global__ void __launch_bounds__(256) cast_vec_kernel(const S* __restrict__ src, D* __restrict__ dst, int64_t numel) {
    // One "group" = the elements of ONE 16-byte store, so that a warp's store instruction covers 512 contiguous bytes
    // (full sectors); the matching load is 8, 16 or 32 bytes per thread, contiguous across the warp as well. Widening
    // casts move fewer bytes per group and keep more groups in flight.
    constexpr int G = 16 / sizeof(D);
    constexpr int IN_BYTES = G * sizeof(S);
    constexpr int UNROLL = IN_BYTES < 16 ? 8 : 4;
    const int64_t ngroup = numel / G;
    const int64_t tile = static_cast<int64_t>(blockDim.x) * UNROLL;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < ngroup; base += static_cast<int64_t>(gridDim.x) * tile) {
        alignas(16) S in[UNROLL][G];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t g = base + u * blockDim.x + threadIdx.x;
            if (g < ngroup) {
                if constexpr (IN_BYTES == 8) {
                    *reinterpret_cast<uint2*>(&in[u][0]) = __ldcs(reinterpret_cast<const uint2*>(src + g * G));
                } else if constexpr (IN_BYTES == 4) {
                    *reinterpret_cast<uint32_t*>(&in[u][0]) = __ldcs(reinterpret_cast<const uint32_t*>(src + g * G));
                } else {
                    const uint4* p = reinterpret_cast<const uint4*>(src + g * G);
                    uint4* q = reinterpret_cast<uint4*>(&in[u][0]);
#pragma unroll
                    for (int w = 0; w < IN_BYTES / 16; ++w) q[w] = __ldcs(p + w);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t g = base + u * blockDim.x + threadIdx.x;
            if (g < ngroup) {
                alignas(16) D o[G];
#pragma unroll
                for (int e = 0; e < G; ++e) o[e] = from_f32<D>(to_f32(in[u][e]));
                __stcs(reinterpret_cast<uint4*>(dst + g * G), *reinterpret_cast<const uint4*>(&o[0]));
            }
        }
    }
    if (blockIdx.x == 0) {
        for (int64_t i = ngroup * G + threadIdx.x; i < numel; i += blockDim.x) dst[i] = from_f32<D>(to_f32(src[i]));
    }
}

template <typename S, typename D>
void launch_cast(const void* src, void* dst, int64_t numel, cudaStream_t stream) {
    constexpr int G = 16 / sizeof(D);
    constexpr int UNROLL = G * sizeof(S) < 16 ? 8 : 4;
    const int64_t ngroup = numel / G;
    const int grid = ew_grid((ngroup + UNROLL - 1) / UNROLL + 1, 256);
    cast_vec_kernel<S, D><<<grid, 256, 0, stream>>>(static_cast<const S*>(src), static_cast<D*>(dst), numel);
}

// ---- 3. strided copy of fixed-size words ---------------------------------------------------------------------
struct WordIter {
    int ndim;            // outer dims (the dense inner run is not counted)
    int64_t nrows;       // product of the outer dims
    int64_t row_words;   // words per inner run
    int64_t shape[kMaxDims];
    int64_t sstride[kMaxDims];  // in words
    int64_t dstride[kMaxDims];
};

// The tensor is a set of dense inner runs ("rows") of row_words words each, placed by the outer strides. A group of
// GROUP lanes walks one row. Each group keeps ROWS consecutive rows in flight; the outer index is decomposed once per
// group (in 32-bit arithmetic when the row count allows) and the following rows are reached by stepping the last outer
// dimension, with a full decomposition only where a row crosses into the next slice.
template <typename I>
__device__ __forceinline__ void decompose_row(const WordIter& it, I row, int64_t* s, int64_t* d, I* c_last) {
    I rem = row;
    int64_t so = 0, dof = 0;
    I c = 0;
    for (int k = it.ndim - 1; k >= 0; --k) {
        const I sh = static_cast<I>(it.shape[k]);
        const I q = rem / sh;
        c = rem - q * sh;
        if (k == it.ndim - 1) *c_last = c;
        rem = q;
        so += static_cast<int64_t>(c) * it.sstride[k];
        dof += static_cast<int64_t>(c) * it.dstride[k];
    }
    *s = so;
    *d = dof;
}

template <typename W, int GROUP, int ROWS, typename I>
__global__ void __launch_bounds__(256) strided_word_copy_kernel(const W* __restrict__ src, W* __restrict__ dst, const WordIter it) {
    const int lane = threadIdx.x % GROUP;
    const int64_t group = (static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x) / GROUP;
    const int64_t row0 = group * ROWS;
    if (row0 >= it.nrows) return;
    int64_t so[ROWS], d_o[ROWS];
    I c_last = 0;
    decompose_row<I>(it, static_cast<I>(row0), &so[0], &d_o[0], &c_last);
    const int last = it.ndim - 1;
    const int64_t room = last >= 0 ? it.shape[last] - static_cast<int64_t>(c_last) : 1;  // rows left in this slice, this one included
#pragma unroll
    for (int r = 1; r < ROWS; ++r) {
        if (r < room) {
            so[r] = so[0] + r * it.sstride[last];
            d_o[r] = d_o[0] + r * it.dstride[last];
        } else if (row0 + r < it.nrows) {
            I dummy;
            decompose_row<I>(it, static_cast<I>(row0 + r), &so[r], &d_o[r], &dummy);
        } else {
            so[r] = so[0];
            d_o[r] = d_o[0];
        }
    }
    for (int64_t w = lane; w < it.row_words; w += GROUP) {
        W val[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (row0 + r < it.nrows) val[r] = src[so[r] + w];
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (row0 + r < it.nrows) dst[d_o[r] + w] = val[r];
        }
    }
}

template <typename W, int GROUP>
void launch_word_copy_g(const W* s, W* d, const WordIter& wi, cudaStream_t stream) {
    // rows that one pass of the group covers: more rows in flight per thread; long rows: fewer (the inner loop iterates)
    const bool short_rows = wi.row_words <= GROUP;
    const int rows = short_rows ? 8 : 4;
    const int64_t groups = (wi.nrows + rows - 1) / rows;
    const int64_t threads = groups * GROUP;
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    const bool small = wi.nrows < 0x7fffffffLL;
    if (short_rows) {
        if (small) strided_word_copy_kernel<W, GROUP, 8, uint32_t><<<grid, 256, 0, stream>>>(s, d, wi);
        else strided_word_copy_kernel<W, GROUP, 8, int64_t><<<grid, 256, 0, stream>>>(s, d, wi);
    } else {
        if (small) strided_word_copy_kernel<W, GROUP, 4, uint32_t><<<grid, 256, 0, stream>>>(s, d, wi);
        else strided_word_copy_kernel<W, GROUP, 4, int64_t><<<grid, 256, 0, stream>>>(s, d, wi);
    }
}

// Rows whose two innermost outer dimensions are swapped between source and destination (a [.., S, H, row] ->
// [.., H, S, row] transpose materialisation): walking the rows in destination order reads 256-byte pieces that lie a
// whole source slice apart, and walking them in source order writes such pieces. Here a CTA takes a tile of TA x TB rows
// (TA along the dimension that is dense in the source, TB along the one that is dense in the destination), so that both
// sides see runs of several KiB; every word still goes straight from its source to its destination address.
template <typename W, int GROUP>
__global__ void __launch_bounds__(256) tiled_row_copy_kernel(const W* __restrict__ src, W* __restrict__ dst, const WordIter it, const int tiles_a,
                                                            const int tiles_b) {
    constexpr int TA = 8, TB = 16, NG = 256 / GROUP, PER = TA * TB / NG;
    const int lane = threadIdx.x % GROUP;
    const int g = threadIdx.x / GROUP;
    const int da = it.ndim - 2, db = it.ndim - 1;
    unsigned tile = blockIdx.x;
    const unsigned ta = tile % tiles_a;
    tile /= tiles_a;
    const unsigned tb = tile % tiles_b;
    unsigned rem = tile / tiles_b;
    int64_t so = 0, dof = 0;
    for (int k = it.ndim - 3; k >= 0; --k) {
        const unsigned sh = static_cast<unsigned>(it.shape[k]);
        const unsigned q = rem / sh;
        const unsigned c = rem - q * sh;
        rem = q;
        so += static_cast<int64_t>(c) * it.sstride[k];
        dof += static_cast<int64_t>(c) * it.dstride[k];
    }
    const int A = static_cast<int>(it.shape[da]), B = static_cast<int>(it.shape[db]);
    int64_t s_off[PER], d_off[PER];
    bool ok[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int id = g + NG * i;          // row of the tile: a runs fastest
        const int a = ta * TA + id % TA;
        const int b = tb * TB + id / TA;
        ok[i] = a < A && b < B;
        s_off[i] = so + static_cast<int64_t>(a) * it.sstride[da] + static_cast<int64_t>(b) * it.sstride[db];
        d_off[i] = dof + static_cast<int64_t>(a) * it.dstride[da] + static_cast<int64_t>(b) * it.dstride[db];
    }
    for (int64_t w = lane; w < it.row_words; w += GROUP) {
        W val[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if (ok[i]) val[i] = src[s_off[i] + w];
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if (ok[i]) dst[d_off[i] + w] = val[i];
        }
    }
}

// True when the tiled kernel was launched.
template <typename W>
bool try_tiled_row_copy(const W* s, W* d, const WordIter& wi, cudaStream_t stream) {
    if (wi.ndim < 2 || wi.row_words < 4 || wi.row_words > 64) return false;
    const int da = wi.ndim - 2, db = wi.ndim - 1;
    // destination order has db innermost; the source has da innermost: a swap
    if (!(wi.sstride[da] < wi.sstride[db] && wi.dstride[db] < wi.dstride[da])) return false;
    if (wi.shape[da] < 8 || wi.shape[db] < 16 || wi.shape[da] > 0x3fffffff || wi.shape[db] > 0x3fffffff) return false;
    const int64_t tiles_a = (wi.shape[da] + 7) / 8, tiles_b = (wi.shape[db] + 15) / 16;
    int64_t outer = 1;
    for (int k = 0; k < wi.ndim - 2; ++k) outer *= wi.shape[k];
    const int64_t tiles = outer * tiles_a * tiles_b;
    if (tiles <= 0 || tiles > 0x7fffffffLL) return false;
    const unsigned grid = static_cast<unsigned>(tiles);
    if (wi.row_words <= 16) tiled_row_copy_kernel<W, 16><<<grid, 256, 0, stream>>>(s, d, wi, static_cast<int>(tiles_a), static_cast<int>(tiles_b));
    else tiled_row_copy_kernel<W, 32><<<grid, 256, 0, stream>>>(s, d, wi, static_cast<int>(tiles_a), static_cast<int>(tiles_b));
    return true;
}

template <typename W>
void launch_word_copy(const void* src, void* dst, const WordIter& wi, cudaStream_t stream) {
    int group = 32;
    while (group > 1 && group / 2 >= wi.row_words) group >>= 1;
    const W* s = static_cast<const W*>(src);
    W* d = static_cast<W*>(dst);
    if (sizeof(W) == 16 && try_tiled_row_copy<W>(s, d, wi, stream)) return;
    switch (group) {
        case 32: launch_word_copy_g<W, 32>(s, d, wi, stream); break;
        case 16: launch_word_copy_g<W, 16>(s, d, wi, stream); break;
        case 8: launch_word_copy_g<W, 8>(s, d, wi, stream); break;
        case 4: launch_word_copy_g<W, 4>(s, d, wi, stream); break;
        case 2: launch_word_copy_g<W, 2>(s, d, wi, stream); break;
        default: launch_word_copy_g<W, 1>(s, d, wi, stream); break;
    }
}

// Same-order test: both dense and equal shapes after dropping size-1 dims.
bool same_dense_order(const TensorView& a, const TensorView& b) {
    if (!a.is_contiguous() || !b.is_contiguous() || a.numel != b.numel) return false;
    return true;  // dense + equal element count + (checked by caller) broadcast-compatible shapes
}

bool shapes_equal_mod1(const TensorView& a, const TensorView& b) {
    int i = 0, o = 0;
    while (true) {
        while (i < a.ndim && a.shape[i] == 1) ++i;
        while (o < b.ndim && b.shape[o] == 1) ++o;
        if (i == a.ndim || o == b.ndim) break;
        if (a.shape[i] != b.shape[o]) return false;
        ++i; ++o;
    }
    return i == a.ndim && o == b.ndim;
}

bool try_word_copy(const TensorView& src, const TensorView& dst, cudaStream_t stream) {
    if (src.dtype != dst.dtype) return false;
    EwIter<2> it;
    const TensorView* ins[1] = {&src};
    if (!build_iter<2>(dst, ins, &it)) return false;
    if (it.ndim == 0) return false;
    const int last = it.ndim - 1;
    if (it.stride[0][last] != 1 || it.stride[1][last] != 1) return false;
    const int64_t es = dst.itemsize;
    const int64_t run_bytes = it.shape[last] * es;
    // widest word that divides the inner run, every outer stride and both base addresses
    int word = 16;
    for (; word > es; word >>= 1) {
        bool ok = (run_bytes % word == 0) && src.aligned(word) && dst.aligned(word);
        for (int d = 0; d < last && ok; ++d) {
            ok = ((it.stride[0][d] * es) % word == 0) && ((it.stride[1][d] * es) % word == 0);
        }
        if (ok) break;
    }
    if (word < es) word = static_cast<int>(es);
    const int64_t epw = word / es;
    WordIter wi;
    wi.ndim = last;
    wi.row_words = it.shape[last] / epw;
    wi.nrows = 1;
    for (int d = 0; d < last; ++d) {
        wi.shape[d] = it.shape[d];
        wi.dstride[d] = it.stride[0][d] / epw;
        wi.sstride[d] = it.stride[1][d] / epw;
        wi.nrows *= it.shape[d];
    }
    // Few long rows (an expand of whole [S, D] planes, say) would leave most of the GPU idle: cut the inner run into
    // pieces of at most 512 words by adding an outer dimension that walks the pieces.
    if (wi.row_words > 512 && wi.ndim < kMaxDims) {
        int64_t pieces = 1;
        while (wi.row_words / pieces > 512 && (wi.row_words / pieces) % 2 == 0) pieces *= 2;
        if (pieces > 1) {
            const int64_t piece_words = wi.row_words / pieces;
            wi.shape[wi.ndim] = pieces;
            wi.sstride[wi.ndim] = piece_words;
            wi.dstride[wi.ndim] = piece_words;
            ++wi.ndim;
            wi.nrows *= pieces;
            wi.row_words = piece_words;
        }
    }
    if ((wi.nrows + 3) / 4 * 32 / 256 + 1 > 0x7fffffffLL) return false;
    switch (word) {
        case 16: launch_word_copy<uint4>(src.data, dst.data, wi, stream); break;
        case 8: launch_word_copy<uint2>(src.data, dst.data, wi, stream); break;
        case 4: launch_word_copy<uint32_t>(src.data, dst.data, wi, stream); break;
        case 2: launch_word_copy<uint16_t>(src.data, dst.data, wi, stream); break;
        default: launch_word_copy<uint8_t>(src.data, dst.data, wi, stream); break;
    }
    return true;
}

}  // namespace

diopiError_t copy_impl(diopiContextHandle_t ctx, const TensorView& src, const TensorView& dst) {
    if (dst.numel == 0) return diopiSuccess;
    cudaStream_t stream = stream_of(ctx);
    const bool dense_same = same_dense_order(src, dst) && shapes_equal_mod1(src, dst);

    // host <-> device: only plain byte moves are done here (DIPU relays anything else through a device tensor,
    // reference dipu/torch_dipu/csrc_dipu/aten/ops/DIPUCopy.hpp:495-527)
    if (src.device == diopi_host || dst.device == diopi_host) {
        B200_CHECK(dense_same && src.dtype == dst.dtype,
                   "diopiCopyInp: a host tensor takes part in a copy that is not a dense same-dtype byte move");
        B200_CUDA(cudaMemcpyAsync(dst.data, src.data, static_cast<size_t>(dst.numel * dst.itemsize), cudaMemcpyDefault, stream));
        return diopiSuccess;
    }
    if (src.data == dst.data && dense_same && src.dtype == dst.dtype) return diopiSuccess;

    if (dense_same && src.dtype == dst.dtype) {
        B200_CUDA(cudaMemcpyAsync(dst.data, src.data, static_cast<size_t>(dst.numel * dst.itemsize), cudaMemcpyDeviceToDevice, stream));
        return diopiSuccess;
    }
    if (dense_same && src.aligned(16) && dst.aligned(16)) {
        const diopiDtype_t s = src.dtype, d = dst.dtype;
        bool done = true;
        if (s == diopi_dtype_bfloat16 && d == diopi_dtype_float32) launch_cast<bf16, float>(src.data, dst.data, dst.numel, stream);
        else if (s == diopi_dtype_float32 && d == diopi_dtype_bfloat16) launch_cast<float, bf16>(src.data, dst.data, dst.numel, stream);
        else if (s == diopi_dtype_float16 && d == diopi_dtype_float32) launch_cast<fp16, float>(src.data, dst.data, dst.numel, stream);
        else if (s == diopi_dtype_float32 && d == diopi_dtype_float16) launch_cast<float, fp16>(src.data, dst.data, dst.numel, stream);
        else if (s == diopi_dtype_bfloat16 && d == diopi_dtype_float16) launch_cast<bf16, fp16>(src.data, dst.data, dst.numel, stream);
        else if (s == diopi_dtype_float16 && d == diopi_dtype_bfloat16) launch_cast<fp16, bf16>(src.data, dst.data, dst.numel, stream);
        else done = false;
        if (done) {
            B200_LAUNCH_CHECK("diopiCopyInp(cast)");
            return diopiSuccess;
        }
    }
    if (try_word_copy(src, dst, stream)) {
        B200_LAUNCH_CHECK("diopiCopyInp(strided)");
        return diopiSuccess;
    }
    const TensorView* ins[1] = {&src};
    return launch_elementwise<OpCopy, 1>(ctx, "diopiCopyInp", dst, ins, ScalarArgs(), /*allow_vec=*/false);
}

diopiError_t make_contiguous(diopiContextHandle_t ctx, const TensorView& v, TensorView* out) {
    if (v.is_contiguous()) {
        *out = v;
        return diopiSuccess;
    }
    diopiTensorHandle_t tmp = nullptr;
    diopiSize_t size{v.shape, v.ndim};
    B200_CHECK(diopiRequireTensor(ctx, &tmp, &size, nullptr, v.dtype, diopi_device) == diopiSuccess && tmp != nullptr,
               "workspace allocation of %lld bytes failed", (long long)(v.numel * v.itemsize));
    if (!make_view(tmp, out, "workspace")) return diopiErrorOccurred;
    return copy_impl(ctx, v, *out);
}

namespace {

// ---- gather of rows (index_select / embedding) ------------------------------------------------------------
// input viewed as [outer, dim_size, inner words], output as [outer, n_index, inner words].
template <typename W, typename I>
__global__ void __launch_bounds__(256) gather_rows_kernel(const W* __restrict__ in, W* __restrict__ out, const I* __restrict__ index,
                                                          int64_t outer, int64_t dim_size, int64_t n_index, int64_t inner, int64_t total) {
    constexpr int UNROLL = 4;
    const int64_t tile = static_cast<int64_t>(blockDim.x) * UNROLL;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < total; base += static_cast<int64_t>(gridDim.x) * tile) {
        W val[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t i = base + u * blockDim.x + threadIdx.x;
            if (i < total) {
                const int64_t row = i / inner;
                const int64_t k = i - row * inner;
                const int64_t o = row / n_index;
                const int64_t j = row - o * n_index;
                int64_t r = static_cast<int64_t>(index[j]);
                if (r < 0) r += dim_size;
                if (r >= 0 && r < dim_size) {
                    val[u] = in[(o * dim_size + r) * inner + k];
                } else {
                    // out-of-range index: defined result (zeros) instead of a wild read
                    W z;
                    memset(&z, 0, sizeof(W));
                    val[u] = z;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t i = base + u * blockDim.x + threadIdx.x;
            if (i < total) out[i] = val[u];
        }
    }
}

template <typename W>
void launch_gather(const void* in, void* out, const TensorView& index, int64_t outer, int64_t dim_size, int64_t n_index, int64_t inner_words,
                   cudaStream_t stream) {
    const int64_t total = outer * n_index * inner_words;
    const int grid = ew_grid((total + 3) / 4 + 1, 256);
    if (index.dtype == diopi_dtype_int64) {
        gather_rows_kernel<W, int64_t><<<grid, 256, 0, stream>>>(static_cast<const W*>(in), static_cast<W*>(out),
                                                                  static_cast<const int64_t*>(index.data), outer, dim_size, n_index, inner_words, total);
    } else {
        gather_rows_kernel<W, int32_t><<<grid, 256, 0, stream>>>(static_cast<const W*>(in), static_cast<W*>(out),
                                                                  static_cast<const int32_t*>(index.data), outer, dim_size, n_index, inner_words, total);
    }
}

diopiError_t gather_rows(diopiContextHandle_t ctx, const char* name, const TensorView& vout, const TensorView& vin_raw, int64_t dim,
                         const TensorView& vidx_raw) {
    B200_CHECK(vidx_raw.dtype == diopi_dtype_int64 || vidx_raw.dtype == diopi_dtype_int32, "%s: index dtype must be int32 or int64, got %s", name,
               dtype_name(vidx_raw.dtype));
    B200_CHECK(vin_raw.dtype == vout.dtype, "%s: input and output dtypes differ (%s vs %s)", name, dtype_name(vin_raw.dtype), dtype_name(vout.dtype));
    B200_CHECK(vout.is_contiguous(), "%s: output must be contiguous", name);
    B200_CHECK(vidx_raw.device == diopi_device && vin_raw.device == diopi_device, "%s: operands must be device tensors", name);
    if (vout.numel == 0) return diopiSuccess;
    TensorView vin, vidx;
    if (make_contiguous(ctx, vin_raw, &vin) != diopiSuccess) return diopiErrorOccurred;
    if (make_contiguous(ctx, vidx_raw, &vidx) != diopiSuccess) return diopiErrorOccurred;
    const int nd = vin.ndim == 0 ? 1 : vin.ndim;
    if (dim < 0) dim += nd;
    B200_CHECK(dim >= 0 && dim < nd, "%s: dim %lld out of range for rank %d", name, (long long)dim, vin.ndim);
    int64_t outer = 1, inner = 1;
    const int64_t dim_size = vin.ndim == 0 ? 1 : vin.shape[dim];
    for (int d = 0; d < dim; ++d) outer *= vin.shape[d];
    for (int d = static_cast<int>(dim) + 1; d < vin.ndim; ++d) inner *= vin.shape[d];
    const int64_t n_index = vidx.numel;
    B200_CHECK(vout.numel == outer * n_index * inner, "%s: output has %lld elements, expected %lld", name, (long long)vout.numel,
               (long long)(outer * n_index * inner));
    const int64_t inner_bytes = inner * vin.itemsize;
    cudaStream_t stream = stream_of(ctx);
    int word = 16;
    while (word > 1 && !(inner_bytes % word == 0 && vin.aligned(word) && vout.aligned(word))) word >>= 1;
    const int64_t iw = inner_bytes / word;
    switch (word) {
        case 16: launch_gather<uint4>(vin.data, vout.data, vidx, outer, dim_size, n_index, iw, stream); break;
        case 8: launch_gather<uint2>(vin.data, vout.data, vidx, outer, dim_size, n_index, iw, stream); break;
        case 4: launch_gather<uint32_t>(vin.data, vout.data, vidx, outer, dim_size, n_index, iw, stream); break;
        case 2: launch_gather<uint16_t>(vin.data, vout.data, vidx, outer, dim_size, n_index, iw, stream); break;
        default: launch_gather<uint8_t>(vin.data, vout.data, vidx, outer, dim_size, n_index, iw, stream); break;
    }
    B200_LAUNCH_CHECK(name);
    return diopiSuccess;
}

// ---- triu -------------------------------------------------------------------------------------------------------
template <typename W>
__global__ void triu_kernel(const W* __restrict__ in, W* __restrict__ out, int64_t rows, int64_t cols, int64_t total, int64_t diagonal) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t c = i % cols;
        const int64_t r = (i / cols) % rows;
        W z;
        memset(&z, 0, sizeof(W));
        out[i] = (c - r >= diagonal) ? in[i] : z;
    }
}

template <typename C>
__global__ void arange_kernel(void* out, diopiDtype_t dt, int64_t n, C start, C step) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        store_from<C>(out, dt, i, start + static_cast<C>(i) * step);
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

diopiError_t diopiCopyInp(diopiContextHandle_t ctx, diopiConstTensorHandle_t src, diopiTensorHandle_t dest) {
    B200_VIEW(vs, src);
    B200_VIEW(vd, dest);
    // expand_as semantics: src must broadcast to dest
    int64_t tmp[kMaxDims];
    B200_CHECK(broadcast_strides(vd, vs, tmp), "diopiCopyInp: source shape cannot be broadcast to the destination shape");
    return copy_impl(ctx, vs, vd);
}

diopiError_t diopiCastDtype(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) {
    return diopiCopyInp(ctx, input, out);
}

diopiError_t diopiIndexSelect(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, int64_t dim,
                              diopiConstTensorHandle_t index) {
    B200_VIEW(vo, out);
    B200_VIEW(vi, input);
    B200_VIEW(vx, index);
    B200_CHECK(vx.ndim <= 1, "diopiIndexSelect: index must be 0-d or 1-d");
    return gather_rows(ctx, "diopiIndexSelect", vo, vi, dim, vx);
}

diopiError_t diopiEmbedding(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t weight, diopiConstTensorHandle_t indices,
                            int64_t, bool, bool) {
    B200_VIEW(vo, out);
    B200_VIEW(vw, weight);
    B200_VIEW(vx, indices);
    B200_CHECK(vw.ndim == 2, "diopiEmbedding: weight must be 2-d");
    return gather_rows(ctx, "diopiEmbedding", vo, vw, 0, vx);
}

diopiError_t diopiCat(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t* tensors, int64_t num_inputs, int64_t dim) {
    B200_VIEW(vo, out);
    B200_CHECK(tensors != nullptr && num_inputs > 0, "diopiCat: no inputs");
    if (dim < 0) dim += vo.ndim;
    B200_CHECK(dim >= 0 && dim < vo.ndim, "diopiCat: dim out of range");
    int64_t offset = 0;
    for (int64_t t = 0; t < num_inputs; ++t) {
        B200_VIEW(vi, tensors[t]);
        if (vi.numel == 0 && vi.ndim == 1) continue;  // legacy empty tensor is skipped by cat
        B200_CHECK(vi.ndim == vo.ndim, "diopiCat: input %lld has rank %d, output rank %d", (long long)t, vi.ndim, vo.ndim);
        for (int d = 0; d < vo.ndim; ++d) {
            if (d != dim) B200_CHECK(vi.shape[d] == vo.shape[d], "diopiCat: input %lld mismatches the output in dim %d", (long long)t, d);
        }
        B200_CHECK(offset + vi.shape[dim] <= vo.shape[dim], "diopiCat: inputs exceed the output extent");
        TensorView slice = vo;
        slice.shape[dim] = vi.shape[dim];
        slice.numel = vi.numel;
        slice.data = static_cast<char*>(vo.data) + offset * vo.stride[dim] * vo.itemsize;
        if (copy_impl(ctx, vi, slice) != diopiSuccess) return diopiErrorOccurred;
        offset += vi.shape[dim];
    }
    B200_CHECK(offset == vo.shape[dim], "diopiCat: inputs cover %lld of %lld entries along dim", (long long)offset, (long long)vo.shape[dim]);
    return diopiSuccess;
}

diopiError_t diopiTriu(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, int64_t diagonal) {
    B200_VIEW(vo, out);
    B200_VIEW(vi_raw, input);
    B200_CHECK(vo.ndim >= 2 && vo.numel == vi_raw.numel && vo.dtype == vi_raw.dtype, "diopiTriu: needs rank >= 2 and matching input/output");
    B200_CHECK(vo.is_contiguous(), "diopiTriu: output must be contiguous");
    if (vo.numel == 0) return diopiSuccess;
    TensorView vi;
    if (make_contiguous(ctx, vi_raw, &vi) != diopiSuccess) return diopiErrorOccurred;
    const int64_t rows = vo.shape[vo.ndim - 2], cols = vo.shape[vo.ndim - 1];
    const int grid = ew_grid(vo.numel, 256);
    cudaStream_t stream = stream_of(ctx);
    switch (vo.itemsize) {
        case 1: triu_kernel<uint8_t><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(vi.data), static_cast<uint8_t*>(vo.data), rows, cols, vo.numel, diagonal); break;
        case 2: triu_kernel<uint16_t><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(vi.data), static_cast<uint16_t*>(vo.data), rows, cols, vo.numel, diagonal); break;
        case 4: triu_kernel<uint32_t><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(vi.data), static_cast<uint32_t*>(vo.data), rows, cols, vo.numel, diagonal); break;
        case 8: triu_kernel<uint2><<<grid, 256, 0, stream>>>(static_cast<const uint2*>(vi.data), static_cast<uint2*>(vo.data), rows, cols, vo.numel, diagonal); break;
        default: B200_FAIL("diopiTriu: element size %lld not supported", (long long)vo.itemsize);
    }
    B200_LAUNCH_CHECK("diopiTriu");
    return diopiSuccess;
}
diopiError_t diopiTriuInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, int64_t diagonal) { return diopiTriu(ctx, input, input, diagonal); }

diopiError_t diopiArange(diopiContextHandle_t ctx, diopiTensorHandle_t out, const diopiScalar_t* start, const diopiScalar_t* end,
                         const diopiScalar_t* step) {
    B200_VIEW(vo, out);
    (void)end;
    B200_CHECK(start && step, "diopiArange: start/step is NULL");
    B200_CHECK(vo.is_contiguous(), "diopiArange: output must be contiguous");
    if (vo.numel == 0) return diopiSuccess;
    ScalarArgs sa;
    scalar_to_args(start, &sa, 0);
    scalar_to_args(step, &sa, 1);
    const int grid = ew_grid(vo.numel, 256);
    cudaStream_t stream = stream_of(ctx);
    if (vo.dtype == diopi_dtype_float64) arange_kernel<double><<<grid, 256, 0, stream>>>(vo.data, vo.dtype, vo.numel, sa.f[0], sa.f[1]);
    else if (is_floating(vo.dtype)) arange_kernel<float><<<grid, 256, 0, stream>>>(vo.data, vo.dtype, vo.numel, (float)sa.f[0], (float)sa.f[1]);
    else arange_kernel<int64_t><<<grid, 256, 0, stream>>>(vo.data, vo.dtype, vo.numel, sa.i[0], sa.i[1]);
    B200_LAUNCH_CHECK("diopiArange");
    return diopiSuccess;
}

}  // extern "C"
