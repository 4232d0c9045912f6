// Fused steps of a decode iteration (one new token per sequence), where the layer is a chain of small kernels and every
// launch costs as much as the work it carries. None of these has a counterpart among the reference's call sites, which
// dispatch the pieces one by one (dicp/test/model/llama/model.py:34-39 RMSNorm, :58-69 / dicp/dicp/vendor/AscendGraph/
// ext_ops.py:24-33 rotary, model.py:134-138 cache append, :193-201 residual adds); each kernel rounds where the op-by-op
// sequence rounds, so the results are the ones the separate calls give.
//
//   diopiB200AddRMSNorm     sum = x + residual (rounded to the element type, like diopiAdd), norm = RMSNorm(sum) * weight
//   diopiB200RopeAppendKV   from the output of ONE q/k/v projection [B, (Hq + 2 Hkv) * D]: rotated q -> q_out [B, Hq, D],
//                           rotated k -> k_cache[:, :, position, :], v -> v_cache[:, :, position, :] (half-split rotary layout)
#include "copy.h"
#include "device_utils.cuh"
#include "diopi/functions_b200.h"

namespace b200 {
namespace {

// One CTA per row; the row stays packed in registers. VPT vectors of 8 elements per thread.
template <typename T, int VPT>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ weight,
                                                           T* __restrict__ sum_out, T* __restrict__ norm_out, int cols, int64_t x_pitch,
                                                           int64_t res_pitch, float eps) {
    // A product that follows in the stream may set itself up while this grid runs (it touches global memory only after its own
    // griddepcontrol.wait); without such a dependent this does nothing.
    grid_launch_dependents();
    __shared__ float red[32];
    const int nvec = cols / 8;
    const int64_t r = blockIdx.x;
    uint4 s[VPT];
    float2 acc = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int iv = i * static_cast<int>(blockDim.x) + static_cast<int>(threadIdx.x);
        if (iv < nvec) {
            const uint4 a = *reinterpret_cast<const uint4*>(x + r * x_pitch + static_cast<int64_t>(iv) * 8);
            const uint4 b = *reinterpret_cast<const uint4*>(res + r * res_pitch + static_cast<int64_t>(iv) * 8);
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o[j] = Pair<T>::narrow(add2(Pair<T>::widen(word(a, j)), Pair<T>::widen(word(b, j))));
                const float2 v = Pair<T>::widen(o[j]);   // the norm sees the ROUNDED sum, as a separate RMSNorm call would
                acc = fma2(v, v, acc);
            }
            s[i] = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(sum_out + r * cols + static_cast<int64_t>(iv) * 8) = s[i];
        }
    }
    const float ss = block_sum(acc.x + acc.y, red);
    const float inv = rsqrtf(ss / static_cast<float>(cols) + eps);
    const float2 inv2 = make_float2(inv, inv);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int iv = i * static_cast<int>(blockDim.x) + static_cast<int>(threadIdx.x);
        if (iv < nvec) {
            uint32_t o[4];
            if (weight != nullptr) {
                const uint4 w = *reinterpret_cast<const uint4*>(weight + static_cast<int64_t>(iv) * 8);
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = Pair<T>::narrow(mul2(mul2(Pair<T>::widen(word(s[i], j)), inv2), Pair<T>::widen(word(w, j))));
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = Pair<T>::narrow(mul2(Pair<T>::widen(word(s[i], j)), inv2));
            }
            *reinterpret_cast<uint4*>(norm_out + r * cols + static_cast<int64_t>(iv) * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

struct RopeAppendParams {
    const void* qkv;
    int64_t qkv_pitch;                 // elements between sequences
    void* q_out;                       // [B, Hq, D] dense
    void* k_cache;
    void* v_cache;
    int64_t k_sb, k_sh, v_sb, v_sh;    // element pitches of batch and head; the slot offset is already in the pointers
    const float* cos_t;
    const float* sin_t;                // [table_rows, D / 2]
    int64_t table_rows;
    int B, Hq, Hkv, D;
};

// One thread per (sequence, head of q | k | v, chunk of 8 pairs): two 16-byte vectors in (the pair partners), two out.
template <typename T>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeAppendParams p) {
    const int half = p.D / 2, chunks = half / 8;
    const int heads = p.Hq + 2 * p.Hkv;
    const int64_t total = static_cast<int64_t>(p.B) * heads * chunks;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = static_cast<int>(i % chunks);
    const int h = static_cast<int>((i / chunks) % heads);
    const int b = static_cast<int>(i / (static_cast<int64_t>(chunks) * heads));
    const T* src = static_cast<const T*>(p.qkv) + b * p.qkv_pitch + static_cast<int64_t>(h) * p.D + c * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(src), bb = *reinterpret_cast<const uint4*>(src + half);
    T* dst;
    if (h < p.Hq) dst = static_cast<T*>(p.q_out) + (static_cast<int64_t>(b) * p.Hq + h) * p.D + c * 8;
    else if (h < p.Hq + p.Hkv) dst = static_cast<T*>(p.k_cache) + b * p.k_sb + static_cast<int64_t>(h - p.Hq) * p.k_sh + c * 8;
    else dst = static_cast<T*>(p.v_cache) + b * p.v_sb + static_cast<int64_t>(h - p.Hq - p.Hkv) * p.v_sh + c * 8;
    if (h >= p.Hq + p.Hkv) {  // values are stored as they are
        *reinterpret_cast<uint4*>(dst) = a;
        *reinterpret_cast<uint4*>(dst + half) = bb;
        return;
    }
    const int64_t row = b % p.table_rows;
    const float4 c0 = *reinterpret_cast<const float4*>(p.cos_t + row * half + c * 8), c1 = *reinterpret_cast<const float4*>(p.cos_t + row * half + c * 8 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(p.sin_t + row * half + c * 8), s1 = *reinterpret_cast<const float4*>(p.sin_t + row * half + c * 8 + 4);
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t o0[4], o1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 va = Pair<T>::widen(word(a, j)), vb = Pair<T>::widen(word(bb, j));
        const float2 cc = make_float2(cs[2 * j], cs[2 * j + 1]), ss = make_float2(sn[2 * j], sn[2 * j + 1]), ns = make_float2(-ss.x, -ss.y);
        o0[j] = Pair<T>::narrow(fma2(vb, ns, mul2(va, cc)));   // a * cos - b * sin
        o1[j] = Pair<T>::narrow(fma2(va, ss, mul2(vb, cc)));   // b * cos + a * sin
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(o0[0], o0[1], o0[2], o0[3]);
    *reinterpret_cast<uint4*>(dst + half) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

diopiError_t diopiB200AddRMSNorm(diopiContextHandle_t ctx, diopiTensorHandle_t sum_out, diopiTensorHandle_t norm_out, diopiConstTensorHandle_t input,
                                 diopiConstTensorHandle_t residual, diopiConstTensorHandle_t weight, double eps) {
    B200_VIEW(vs, sum_out);
    B200_VIEW(vn, norm_out);
    B200_VIEW(vx, input);
    B200_VIEW(vr, residual);
    TensorView vw;
    if (weight && !make_view(weight, &vw, "weight")) return diopiErrorOccurred;
    B200_CHECK(vx.ndim == 2 && vr.ndim == 2 && vs.ndim == 2 && vn.ndim == 2, "diopiB200AddRMSNorm: expected [rows, cols] tensors");
    const int64_t rows = vx.shape[0], cols = vx.shape[1];
    B200_CHECK(vr.shape[0] == rows && vr.shape[1] == cols && vs.shape[0] == rows && vs.shape[1] == cols && vn.shape[0] == rows && vn.shape[1] == cols,
               "diopiB200AddRMSNorm: shapes differ");
    B200_CHECK((vx.dtype == diopi_dtype_bfloat16 || vx.dtype == diopi_dtype_float16) && vr.dtype == vx.dtype && vs.dtype == vx.dtype && vn.dtype == vx.dtype,
               "diopiB200AddRMSNorm: bfloat16 or float16 tensors of one dtype");
    B200_CHECK(vs.is_contiguous() && vn.is_contiguous() && vx.stride[1] == 1 && vr.stride[1] == 1 && vx.stride[0] % 8 == 0 && vr.stride[0] % 8 == 0,
               "diopiB200AddRMSNorm: dense outputs, inputs with contiguous rows and row pitches that are multiples of 8 elements");
    B200_CHECK(vx.aligned(16) && vr.aligned(16) && vs.aligned(16) && vn.aligned(16) && cols % 8 == 0 && cols / 8 <= 8 * 1024 && rows <= 0x7fffffffLL,
               "diopiB200AddRMSNorm: 16-byte aligned tensors with a multiple of 8 and at most 65536 columns");
    B200_CHECK(weight == nullptr || (vw.dtype == vx.dtype && vw.numel == cols && vw.is_contiguous() && vw.aligned(16)),
               "diopiB200AddRMSNorm: weight must be a dense tensor of the input dtype with one entry per column");
    if (rows == 0) return diopiSuccess;
    const int64_t nvec = cols / 8;
    int threads = static_cast<int>(((nvec + 3) / 4 + 31) / 32 * 32);
    threads = threads < 32 ? 32 : (threads > 1024 ? 1024 : threads);
    const int64_t vpt64 = (nvec + threads - 1) / threads;
    const int vpt = vpt64 <= 1 ? 1 : (vpt64 <= 2 ? 2 : (vpt64 <= 4 ? 4 : 8));
    cudaStream_t stream = stream_of(ctx);
    const unsigned grid = static_cast<unsigned>(rows);
#define LAUNCH_ARN(T, V)                                                                                                                           \
    add_rmsnorm_kernel<T, V><<<grid, threads, 0, stream>>>(static_cast<const T*>(vx.data), static_cast<const T*>(vr.data),                          \
                                                           weight ? static_cast<const T*>(vw.data) : nullptr, static_cast<T*>(vs.data),            \
                                                           static_cast<T*>(vn.data), static_cast<int>(cols), vx.stride[0], vr.stride[0],           \
                                                           static_cast<float>(eps))
#define LAUNCH_ARN_T(T)                          \
    switch (vpt) {                               \
        case 1: LAUNCH_ARN(T, 1); break;         \
        case 2: LAUNCH_ARN(T, 2); break;         \
        case 4: LAUNCH_ARN(T, 4); break;         \
        default: LAUNCH_ARN(T, 8); break;        \
    }
    if (vx.dtype == diopi_dtype_bfloat16) { LAUNCH_ARN_T(bf16); }
    else { LAUNCH_ARN_T(fp16); }
#undef LAUNCH_ARN_T
#undef LAUNCH_ARN
    B200_LAUNCH_CHECK("diopiB200AddRMSNorm");
    return diopiSuccess;
}

diopiError_t diopiB200RopeAppendKV(diopiContextHandle_t ctx, diopiTensorHandle_t q_out, diopiConstTensorHandle_t qkv, diopiConstTensorHandle_t cos,
                                   diopiConstTensorHandle_t sin, diopiTensorHandle_t k_cache, diopiTensorHandle_t v_cache, int64_t position) {
    B200_VIEW(vq, q_out);
    B200_VIEW(vx, qkv);
    B200_VIEW(vc, cos);
    B200_VIEW(vsn, sin);
    B200_VIEW(vk, k_cache);
    B200_VIEW(vv, v_cache);
    B200_CHECK(vq.ndim == 3 && vx.ndim == 2 && vk.ndim == 4 && vv.ndim == 4, "diopiB200RopeAppendKV: q_out [B, Hq, D], qkv [B, (Hq + 2 Hkv) D], caches [B, Hkv, L, D]");
    const int64_t B = vq.shape[0], Hq = vq.shape[1], D = vq.shape[2], Hkv = vk.shape[1], L = vk.shape[2];
    B200_CHECK(vx.shape[0] == B && vx.shape[1] == (Hq + 2 * Hkv) * D && vk.shape[0] == B && vk.shape[3] == D && vv.shape[0] == B && vv.shape[1] == Hkv &&
                   vv.shape[2] == L && vv.shape[3] == D,
               "diopiB200RopeAppendKV: shapes do not fit together");
    B200_CHECK(position >= 0 && position < L, "diopiB200RopeAppendKV: position %lld outside the cache of %lld slots", (long long)position, (long long)L);
    B200_CHECK((vx.dtype == diopi_dtype_bfloat16 || vx.dtype == diopi_dtype_float16) && vq.dtype == vx.dtype && vk.dtype == vx.dtype && vv.dtype == vx.dtype,
               "diopiB200RopeAppendKV: bfloat16 or float16 tensors of one dtype");
    B200_CHECK(vc.dtype == diopi_dtype_float32 && vsn.dtype == diopi_dtype_float32 && vc.is_contiguous() && vsn.is_contiguous() && vc.numel == vsn.numel &&
                   vc.ndim >= 1 && vc.shape[vc.ndim - 1] == D / 2,
               "diopiB200RopeAppendKV: cos / sin must be dense float32 tables [rows, D / 2]");
    const int64_t table_rows = vc.numel / (D / 2);
    B200_CHECK(table_rows >= 1 && B % table_rows == 0, "diopiB200RopeAppendKV: %lld table rows do not tile %lld sequences", (long long)table_rows, (long long)B);
    B200_CHECK(D % 16 == 0 && vq.is_contiguous() && vx.stride[1] == 1 && vx.stride[0] % 8 == 0 && vk.stride[3] == 1 && vv.stride[3] == 1,
               "diopiB200RopeAppendKV: head dim a multiple of 16, dense q_out, contiguous rows");
    for (int d = 0; d < 3; ++d) {
        B200_CHECK(vk.stride[d] % 8 == 0 && vv.stride[d] % 8 == 0, "diopiB200RopeAppendKV: cache pitches must be multiples of 8 elements");
    }
    B200_CHECK(vq.aligned(16) && vx.aligned(16) && vk.aligned(16) && vv.aligned(16) && vc.aligned(16) && vsn.aligned(16),
               "diopiB200RopeAppendKV: 16-byte aligned tensors");
    if (B == 0) return diopiSuccess;
    RopeAppendParams p;
    p.qkv = vx.data; p.qkv_pitch = vx.stride[0];
    p.q_out = vq.data;
    p.k_cache = static_cast<char*>(vk.data) + position * vk.stride[2] * vk.itemsize;
    p.v_cache = static_cast<char*>(vv.data) + position * vv.stride[2] * vv.itemsize;
    p.k_sb = vk.stride[0]; p.k_sh = vk.stride[1]; p.v_sb = vv.stride[0]; p.v_sh = vv.stride[1];
    p.cos_t = static_cast<const float*>(vc.data); p.sin_t = static_cast<const float*>(vsn.data);
    p.table_rows = table_rows;
    p.B = static_cast<int>(B); p.Hq = static_cast<int>(Hq); p.Hkv = static_cast<int>(Hkv); p.D = static_cast<int>(D);
    const int64_t total = B * (Hq + 2 * Hkv) * (D / 16);
    B200_CHECK(total < 0x7fffffffLL * 256, "diopiB200RopeAppendKV: too many elements");
    const unsigned grid = static_cast<unsigned>((total + 255) / 256);
    cudaStream_t stream = stream_of(ctx);
    if (vx.dtype == diopi_dtype_bfloat16) rope_append_kernel<bf16><<<grid, 256, 0, stream>>>(p);
    else rope_append_kernel<fp16><<<grid, 256, 0, stream>>>(p);
    B200_LAUNCH_CHECK("diopiB200RopeAppendKV");
    return diopiSuccess;
}

}  // extern "C"
