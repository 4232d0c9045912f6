// Device-side helpers shared by the kernels: dtype-erased element access, 128-bit vector access,
// warp / block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "diopi/diopirt.h"

namespace b200 {

using bf16 = __nv_bfloat16;
using fp16 = __half;

// ---- typed <-> float conversions -----------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<fp16>(fp16 v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ fp16 from_f32<fp16>(float v) { return __float2half_rn(v); }

// ---- dtype-erased element access (used by the general strided kernels) ---------------------
// C is the compute type: float, double or int64_t.
template <typename C>
__device__ __forceinline__ C load_as(const void* base, diopiDtype_t dt, int64_t idx) {
    switch (dt) {
        case diopi_dtype_float32: return static_cast<C>(static_cast<const float*>(base)[idx]);
        case diopi_dtype_bfloat16: return static_cast<C>(__bfloat162float(static_cast<const bf16*>(base)[idx]));
        case diopi_dtype_float16: return static_cast<C>(__half2float(static_cast<const fp16*>(base)[idx]));
        case diopi_dtype_float64: return static_cast<C>(static_cast<const double*>(base)[idx]);
        case diopi_dtype_int64: return static_cast<C>(static_cast<const int64_t*>(base)[idx]);
        case diopi_dtype_uint64: return static_cast<C>(static_cast<const uint64_t*>(base)[idx]);
        case diopi_dtype_int32: return static_cast<C>(static_cast<const int32_t*>(base)[idx]);
        case diopi_dtype_uint32: return static_cast<C>(static_cast<const uint32_t*>(base)[idx]);
        case diopi_dtype_int16: return static_cast<C>(static_cast<const int16_t*>(base)[idx]);
        case diopi_dtype_uint16: return static_cast<C>(static_cast<const uint16_t*>(base)[idx]);
        case diopi_dtype_int8: return static_cast<C>(static_cast<const int8_t*>(base)[idx]);
        case diopi_dtype_uint8: return static_cast<C>(static_cast<const uint8_t*>(base)[idx]);
        case diopi_dtype_bool: return static_cast<C>(static_cast<const uint8_t*>(base)[idx] != 0 ? 1 : 0);
        default: return C(0);
    }
}

template <typename C>
__device__ __forceinline__ void store_from(void* base, diopiDtype_t dt, int64_t idx, C v) {
    switch (dt) {
        case diopi_dtype_float32: static_cast<float*>(base)[idx] = static_cast<float>(v); break;
        case diopi_dtype_bfloat16: static_cast<bf16*>(base)[idx] = __float2bfloat16_rn(static_cast<float>(v)); break;
        case diopi_dtype_float16: static_cast<fp16*>(base)[idx] = __float2half_rn(static_cast<float>(v)); break;
        case diopi_dtype_float64: static_cast<double*>(base)[idx] = static_cast<double>(v); break;
        case diopi_dtype_int64: static_cast<int64_t*>(base)[idx] = static_cast<int64_t>(v); break;
        case diopi_dtype_uint64: static_cast<uint64_t*>(base)[idx] = static_cast<uint64_t>(v); break;
        case diopi_dtype_int32: static_cast<int32_t*>(base)[idx] = static_cast<int32_t>(v); break;
        case diopi_dtype_uint32: static_cast<uint32_t*>(base)[idx] = static_cast<uint32_t>(v); break;
        case diopi_dtype_int16: static_cast<int16_t*>(base)[idx] = static_cast<int16_t>(v); break;
        case diopi_dtype_uint16: static_cast<uint16_t*>(base)[idx] = static_cast<uint16_t>(v); break;
        case diopi_dtype_int8: static_cast<int8_t*>(base)[idx] = static_cast<int8_t>(v); break;
        case diopi_dtype_uint8: static_cast<uint8_t*>(base)[idx] = static_cast<uint8_t>(v); break;
        case diopi_dtype_bool: static_cast<uint8_t*>(base)[idx] = (v != C(0)) ? 1 : 0; break;
        default: break;
    }
}

// ---- 128-bit vector of T ---------------------------------------------------------------------
template <typename T>
struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
    return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Vec16<T>& r) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}
// Streaming variants: the data is touched once, keep it from displacing reusable lines in L1.
template <typename T>
__device__ __forceinline__ Vec16<T> ld16_stream(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
    return r;
}
template <typename T>
__device__ __forceinline__ void st16_stream(T* p, const Vec16<T>& r) {
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&r));
}

// ---- packed pairs -------------------------------------------------------------------------------
// The row kernels work on two elements at a time: a 32-bit word of two 2-byte elements is widened to a float2 (bf16: a
// shift and a mask), the arithmetic uses the two-wide fp32 instructions of sm_100 (fma / mul / add .f32x2: one issue slot
// for two results), and a float2 is narrowed back with one cvt.rn.<t>x2.f32. Same values as the element-wise forms.
template <typename T> struct Pair;
template <> struct Pair<bf16> {
    static __device__ __forceinline__ float2 widen(uint32_t w) { return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u)); }
    static __device__ __forceinline__ uint32_t narrow(float2 v) {
        uint32_t r;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(v.y), "f"(v.x));
        return r;
    }
};
template <> struct Pair<fp16> {
    static __device__ __forceinline__ float2 widen(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
    static __device__ __forceinline__ uint32_t narrow(float2 v) {
        uint32_t r;
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(v.y), "f"(v.x));
        return r;
    }
};

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ uint32_t word(const uint4& v, int j) { return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w)); }
__device__ __forceinline__ uint4 ld16_stream_raw(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st16_stream_raw(void* p, const uint4& v) { __stcs(reinterpret_cast<uint4*>(p), v); }

// ---- reductions --------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum, result broadcast to every thread. `red` needs 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // protects `red` against a previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// Programmatic dependent launch. A kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization may start while
// the kernel before it in the stream is still running; grid_dependency_wait() returns once that kernel has completed and its
// writes are visible (at once when the launch carried no such attribute). grid_launch_dependents() lets a dependent kernel
// of THIS grid be scheduled as soon as every CTA has executed it or exited (no effect without such a dependent).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace b200
