// diopiRotaryEmbedding: rotate feature pairs of q/k by position-dependent angles.
//
// x is viewed as [tokens, heads, dim]; cos/sin as [table_rows, table_cols] with table_cols = dim/2 (one angle per
// pair) or dim (full-width tables). Token t uses table row t % table_rows, so a [seq, dim/2] table broadcasts over
// the batch and a [batch*seq, ...] table is used row for row. One thread owns 8 pairs: it reads two 16-byte
// vectors of x (the two partners), the matching angles, and writes two vectors. Algorithmic traffic:
// 2 * bytes(x) + table rows touched.
//
// Arithmetic follows the reference's CPU restatements: half-split pairs (i, i + dim/2)
// (dicp/dicp/vendor/AscendGraph/ext_ops.py:24-33) and interleaved pairs (2i, 2i+1), i.e. complex multiplication
// (dicp/test/model/llama/model.py:58-69). Products and sums are formed in fp32 and rounded once.
#include <cstdlib>

#include "copy.h"
#include "device_utils.cuh"
#include "gemm.h"
#include "row_pipe.cuh"

namespace b200 {
namespace {

template <typename TC>
__device__ __forceinline__ void load_angles8(const TC* p, float (&a)[8]) {
    if constexpr (sizeof(TC) == 4) {
        const float4 lo = *reinterpret_cast<const float4*>(p);
        const float4 hi = *reinterpret_cast<const float4*>(p + 4);
        a[0] = lo.x; a[1] = lo.y; a[2] = lo.z; a[3] = lo.w;
        a[4] = hi.x; a[5] = hi.y; a[6] = hi.z; a[7] = hi.w;
    } else {
        const Vec16<TC> v = ld16(p);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = to_f32(v.v[e]);
    }
}

// Half-split layout, 2-byte element types, dim/2 a multiple of 8.
template <typename T, typename TC>
__global__ void __launch_bounds__(256) rope_half_kernel(const T* x, T* out, const TC* __restrict__ cos_t,
                                                        const TC* __restrict__ sin_t, int64_t tokens, int heads, int dim, int64_t table_rows,
                                                        int table_cols, float sin_sign) {
    const int half = dim / 2;
    const int chunks = half / 8;
    // A block covers 256 / chunks (token, head) rows; the thread's chunk and row come from threadIdx with 32-bit arithmetic
    // and one division per loop trip remains (64-bit index arithmetic per thread costs as much as the rotation itself).
    const int rows_per_block = 256 / chunks;
    const int local_row = static_cast<int>(threadIdx.x) / chunks;
    const int c = static_cast<int>(threadIdx.x) - local_row * chunks;
    const int64_t total_rows = tokens * heads;
    const bool narrow = total_rows < 0x7fffffffLL;
    for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_block; row0 < total_rows; row0 += static_cast<int64_t>(gridDim.x) * rows_per_block) {
        const int64_t th = row0 + local_row;  // token * heads + head
        if (local_row >= rows_per_block || th >= total_rows) continue;
        int64_t row;
        if (narrow && table_rows < 0x7fffffffLL) {
            const uint32_t t = static_cast<uint32_t>(th) / static_cast<uint32_t>(heads);
            row = t % static_cast<uint32_t>(table_rows);
        } else {
            row = (th / heads) % table_rows;
        }
        const T* px = x + th * dim + c * 8;
        const Vec16<T> x0 = ld16_stream(px);
        const Vec16<T> x1 = ld16_stream(px + half);
        float c0[8], s0[8], c1[8], s1[8];
        load_angles8<TC>(cos_t + row * table_cols + c * 8, c0);
        load_angles8<TC>(sin_t + row * table_cols + c * 8, s0);
        if (table_cols == dim) {
            load_angles8<TC>(cos_t + row * table_cols + half + c * 8, c1);
            load_angles8<TC>(sin_t + row * table_cols + half + c * 8, s1);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { c1[e] = c0[e]; s1[e] = s0[e]; }
        }
        // pairs of elements: widened words, two-wide fp32 arithmetic, one narrowing conversion per pair
        const uint4 ra = *reinterpret_cast<const uint4*>(&x0), rb = *reinterpret_cast<const uint4*>(&x1);
        uint32_t o0[4], o1[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 va = Pair<T>::widen(word(ra, j)), vb = Pair<T>::widen(word(rb, j));
            const float2 cc0 = make_float2(c0[2 * j], c0[2 * j + 1]), ns0 = make_float2(-sin_sign * s0[2 * j], -sin_sign * s0[2 * j + 1]);
            const float2 cc1 = make_float2(c1[2 * j], c1[2 * j + 1]), ss1 = make_float2(sin_sign * s1[2 * j], sin_sign * s1[2 * j + 1]);
            o0[j] = Pair<T>::narrow(fma2(vb, ns0, mul2(va, cc0)));   // a * cos - b * sin
            o1[j] = Pair<T>::narrow(fma2(va, ss1, mul2(vb, cc1)));   // b * cos + a * sin
        }
        T* po = out + th * dim + c * 8;
        st16_stream_raw(po, make_uint4(o0[0], o0[1], o0[2], o0[3]));
        st16_stream_raw(po + half, make_uint4(o1[0], o1[1], o1[2], o1[3]));
    }
}

// Half-split layout with [rows, dim/2] tables, pipelined (row_pipe.cuh): a "row" of a warp's ring is one token, heads * dim
// elements. Lane l rotates the 8 pairs of items l, l + 32, ... where item = (head, chunk of 8 pairs); 32 is a multiple of the
// chunks per head, so a lane's chunk is the same for all its items: it reads the 8 + 8 angles of that chunk once per token,
// and reads them for its NEXT token before it rotates the current one (the table row comes from L2; its latency would
// otherwise sit in every iteration).
template <typename T, typename TC>
__global__ void __launch_bounds__(512) rope_wpipe_kernel(const T* x, T* out, const TC* __restrict__ cos_t, const TC* __restrict__ sin_t, int64_t tokens,
                                                         int heads, int dim, int64_t table_rows, float sin_sign, uint32_t* status) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ rowpipe::Ctl ctl;
    const int half = dim / 2;
    const int chunks = half / 8;
    const int items = heads * chunks;
    const uint32_t row_bytes = static_cast<uint32_t>(heads) * dim * 2;
    rowpipe::init_ctl(&ctl, blockDim.x >> 5);
    rowpipe::WarpRing ring = rowpipe::make_ring(&ctl, smem, x, row_bytes, tokens);
    ring.start();
    const int lane = threadIdx.x & 31;
    const int c = lane % chunks;
    float cn[8], sn[8];
    int64_t r = ring.first;
    if (r < tokens) {
        load_angles8<TC>(cos_t + (r % table_rows) * half + c * 8, cn);
        load_angles8<TC>(sin_t + (r % table_rows) * half + c * 8, sn);
    }
    bool failed = false;
    int k = 0;
    for (; r < tokens; r += ring.stride, ++k) {
        float2 cc[4], ss[4], ns[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            cc[j] = make_float2(cn[2 * j], cn[2 * j + 1]);
            ss[j] = make_float2(sin_sign * sn[2 * j], sin_sign * sn[2 * j + 1]);
            ns[j] = make_float2(-ss[j].x, -ss[j].y);
        }
        const int64_t rn = r + ring.stride;
        if (rn < tokens) {
            load_angles8<TC>(cos_t + (rn % table_rows) * half + c * 8, cn);
            load_angles8<TC>(sin_t + (rn % table_rows) * half + c * 8, sn);
        }
        const unsigned char* slot = ring.acquire(k);
        if (slot == nullptr) {
            failed = true;
            break;
        }
        char* orow = reinterpret_cast<char*>(out) + r * static_cast<int64_t>(row_bytes);
#pragma unroll 2
        for (int it = lane; it < items; it += 32) {
            const size_t off = (static_cast<size_t>(it / chunks) * dim + static_cast<size_t>(c) * 8) * 2;
            const uint4 a = rowpipe::lds16(slot + off), b = rowpipe::lds16(slot + off + static_cast<size_t>(half) * 2);
            uint32_t o0[4], o1[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 va = Pair<T>::widen(word(a, j)), vb = Pair<T>::widen(word(b, j));
                o0[j] = Pair<T>::narrow(fma2(vb, ns[j], mul2(va, cc[j])));   // a * cos - b * sin
                o1[j] = Pair<T>::narrow(fma2(va, ss[j], mul2(vb, cc[j])));   // b * cos + a * sin
            }
            st16_stream_raw(orow + off, make_uint4(o0[0], o0[1], o0[2], o0[3]));
            st16_stream_raw(orow + off + static_cast<size_t>(half) * 2, make_uint4(o1[0], o1[1], o1[2], o1[3]));
        }
        ring.release(k);
    }
    if (failed) rowpipe::leave_after_timeout(status);
}

// General variant: any float dtype for x and the tables, either layout, one pair per thread.
template <typename C>
__global__ void rope_generic_kernel(const void* x, void* out, diopiDtype_t x_dt, const void* cos_t, const void* sin_t, diopiDtype_t t_dt,
                                    int64_t tokens, int heads, int dim, int64_t table_rows, int table_cols, C sin_sign, bool interleaved) {
    const int half = dim / 2;
    const int64_t total = tokens * heads * half;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
        const int p = static_cast<int>(i % half);
        const int64_t th = i / half;
        const int64_t t = th / heads;
        const int64_t row = t % table_rows;
        const int64_t i0 = th * dim + (interleaved ? 2 * p : p);
        const int64_t i1 = th * dim + (interleaved ? 2 * p + 1 : p + half);
        int64_t a0, a1;
        if (table_cols == dim) {
            a0 = row * table_cols + (interleaved ? 2 * p : p);
            a1 = row * table_cols + (interleaved ? 2 * p + 1 : p + half);
        } else {
            a0 = a1 = row * table_cols + p;
        }
        const C xa = load_as<C>(x, x_dt, i0), xb = load_as<C>(x, x_dt, i1);
        const C c0 = load_as<C>(cos_t, t_dt, a0), s0 = sin_sign * load_as<C>(sin_t, t_dt, a0);
        const C c1 = load_as<C>(cos_t, t_dt, a1), s1 = sin_sign * load_as<C>(sin_t, t_dt, a1);
        store_from<C>(out, x_dt, i0, xa * c0 - xb * s0);
        store_from<C>(out, x_dt, i1, xb * c1 + xa * s1);
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" diopiError_t diopiRotaryEmbedding(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t x, diopiConstTensorHandle_t cos,
                                             diopiConstTensorHandle_t sin, const bool conj, const bool interleaved) {
    B200_VIEW(vo, out);
    B200_VIEW(vx_raw, x);
    B200_VIEW(vc_raw, cos);
    B200_VIEW(vs_raw, sin);
    B200_CHECK(vx_raw.ndim >= 2, "diopiRotaryEmbedding: x needs at least [heads, dim]");
    B200_CHECK(vo.numel == vx_raw.numel && vo.dtype == vx_raw.dtype && vo.is_contiguous(),
               "diopiRotaryEmbedding: out must be dense and match x in shape and dtype");
    B200_CHECK(is_floating(vx_raw.dtype) && is_floating(vc_raw.dtype) && vc_raw.dtype == vs_raw.dtype, "diopiRotaryEmbedding: floating dtypes only, cos/sin alike");
    B200_CHECK(vc_raw.numel == vs_raw.numel && vc_raw.ndim >= 1, "diopiRotaryEmbedding: cos and sin must have the same shape");
    if (vo.numel == 0) return diopiSuccess;
    TensorView vx, vc, vs;
    if (make_contiguous(ctx, vx_raw, &vx) != diopiSuccess) return diopiErrorOccurred;
    if (make_contiguous(ctx, vc_raw, &vc) != diopiSuccess) return diopiErrorOccurred;
    if (make_contiguous(ctx, vs_raw, &vs) != diopiSuccess) return diopiErrorOccurred;
    const int64_t dim = vx.shape[vx.ndim - 1];
    const int64_t heads = vx.shape[vx.ndim - 2];
    const int64_t tokens = vx.numel / (dim * heads);
    const int64_t table_cols = vc.shape[vc.ndim - 1];
    B200_CHECK(dim % 2 == 0, "diopiRotaryEmbedding: head dim must be even");
    B200_CHECK(table_cols == dim || table_cols == dim / 2, "diopiRotaryEmbedding: cos/sin last dim must be dim or dim/2 (got %lld for dim %lld)",
               (long long)table_cols, (long long)dim);
    const int64_t table_rows = vc.numel / table_cols;
    B200_CHECK(table_rows > 0 && tokens % table_rows == 0, "diopiRotaryEmbedding: %lld table rows do not tile %lld tokens", (long long)table_rows,
               (long long)tokens);
    cudaStream_t stream = stream_of(ctx);
    const float sign = conj ? -1.f : 1.f;
    const bool two_byte = vx.dtype == diopi_dtype_bfloat16 || vx.dtype == diopi_dtype_float16;
    const bool tables_ok = (vc.dtype == vx.dtype || vc.dtype == diopi_dtype_float32) && vc.aligned(16) && vs.aligned(16) && (table_cols % 8 == 0);
    // pipelined kernel: one token (heads * dim elements, 1 to 16 KiB) per ring slot, [rows, dim/2] tables
    const int64_t token_bytes = heads * dim * 2;
    const int64_t chunks64 = dim / 16;
    static const bool pipe_off = std::getenv("B200_NO_ROW_PIPE") != nullptr;
    if (!pipe_off && !interleaved && two_byte && (dim / 2) % 8 == 0 && table_cols == dim / 2 && vx.aligned(16) && vo.aligned(16) && tables_ok && token_bytes >= 1024 &&
        token_bytes <= 16384 && chunks64 >= 1 && 32 % chunks64 == 0 && tokens < 0x7fffffffLL) {
        const int warps = rowpipe::warps_for(token_bytes, 0);
        const unsigned smem = static_cast<unsigned>(static_cast<int64_t>(warps) * rowpipe::kStages * token_bytes);
        uint32_t* status = tc_status_word();
        bool launched = false;
#define LAUNCH_ROPE_PIPE(T, TC)                                                                                                             \
    do {                                                                                                                                   \
        const void* kfn = reinterpret_cast<const void*>(rope_wpipe_kernel<T, TC>);                                                          \
        int occ = 0;                                                                                                                       \
        if (warps >= 4 && tc_ensure_smem_attr(kfn, static_cast<int>(smem)) == cudaSuccess &&                                               \
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, rope_wpipe_kernel<T, TC>, warps * 32, smem) == cudaSuccess && occ >= 1) {   \
            int64_t ctas = static_cast<int64_t>(sm_count()) * occ;                                                                         \
            const int64_t need = (tokens + warps - 1) / warps;                                                                             \
            if (ctas > need) ctas = need;                                                                                                  \
            rope_wpipe_kernel<T, TC><<<static_cast<unsigned>(ctas), warps * 32, smem, stream>>>(                                            \
                static_cast<const T*>(vx.data), static_cast<T*>(vo.data), static_cast<const TC*>(vc.data), static_cast<const TC*>(vs.data), \
                tokens, (int)heads, (int)dim, table_rows, sign, status);                                                                  \
            launched = true;                                                                                                               \
        } else {                                                                                                                           \
            (void)cudaGetLastError();                                                                                                      \
        }                                                                                                                                  \
    } while (0)
        if (vx.dtype == diopi_dtype_bfloat16) {
            if (vc.dtype == diopi_dtype_float32) LAUNCH_ROPE_PIPE(bf16, float); else LAUNCH_ROPE_PIPE(bf16, bf16);
        } else {
            if (vc.dtype == diopi_dtype_float32) LAUNCH_ROPE_PIPE(fp16, float); else LAUNCH_ROPE_PIPE(fp16, fp16);
        }
#undef LAUNCH_ROPE_PIPE
        if (launched) {
            B200_LAUNCH_CHECK("diopiRotaryEmbedding");
            return diopiSuccess;
        }
    }
    if (!interleaved && two_byte && (dim / 2) % 8 == 0 && dim / 16 <= 256 && vx.aligned(16) && vo.aligned(16) && tables_ok) {
        const int64_t rows_per_block = 256 / (dim / 16);
        int64_t blocks = (tokens * heads + rows_per_block - 1) / rows_per_block;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
        if (blocks > cap) blocks = cap;
        const unsigned grid = static_cast<unsigned>(blocks);
#define LAUNCH_ROPE(T, TC)                                                                                                                       \
    rope_half_kernel<T, TC><<<grid, 256, 0, stream>>>(static_cast<const T*>(vx.data), static_cast<T*>(vo.data), static_cast<const TC*>(vc.data), \
                                                      static_cast<const TC*>(vs.data), tokens, (int)heads, (int)dim, table_rows, (int)table_cols, sign)
        if (vx.dtype == diopi_dtype_bfloat16) {
            if (vc.dtype == diopi_dtype_float32) LAUNCH_ROPE(bf16, float); else LAUNCH_ROPE(bf16, bf16);
        } else {
            if (vc.dtype == diopi_dtype_float32) LAUNCH_ROPE(fp16, float); else LAUNCH_ROPE(fp16, fp16);
        }
#undef LAUNCH_ROPE
    } else {
        const int64_t total = tokens * heads * (dim / 2);
        int64_t blocks = (total + 255) / 256;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
        if (blocks > cap) blocks = cap;
        const unsigned grid = static_cast<unsigned>(blocks);
        if (vx.dtype == diopi_dtype_float64) {
            rope_generic_kernel<double><<<grid, 256, 0, stream>>>(vx.data, vo.data, vx.dtype, vc.data, vs.data, vc.dtype, tokens, (int)heads, (int)dim,
                                                                  table_rows, (int)table_cols, (double)sign, interleaved);
        } else {
            rope_generic_kernel<float><<<grid, 256, 0, stream>>>(vx.data, vo.data, vx.dtype, vc.data, vs.data, vc.dtype, tokens, (int)heads, (int)dim,
                                                                 table_rows, (int)table_cols, sign, interleaved);
        }
    }
    B200_LAUNCH_CHECK("diopiRotaryEmbedding");
    return diopiSuccess;
}
