// Shared host-side helpers of the operator library: tensor metadata snapshots taken through the
// diopirt callbacks, the thread-local error string, dtype utilities and launch helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "diopi/diopirt.h"
#include "diopi/functions.h"
#include "diopi/functions_ext.h"

namespace b200 {

constexpr int kMaxDims = 8;

// Plain snapshot of a host tensor. Taken once per call; kernels never see the opaque handle.
struct TensorView {
    void* data = nullptr;
    diopiDtype_t dtype = diopi_dtype_unsupported;
    diopiDevice_t device = diopi_device;
    int ndim = 0;
    int64_t shape[kMaxDims] = {0};
    int64_t stride[kMaxDims] = {0};
    int64_t numel = 0;
    int64_t itemsize = 0;
    bool defined = false;

    bool is_contiguous() const {
        int64_t expect = 1;
        for (int i = ndim - 1; i >= 0; --i) {
            if (shape[i] == 1) continue;
            if (stride[i] != expect) return false;
            expect *= shape[i];
        }
        return true;
    }
    bool aligned(size_t a) const { return (reinterpret_cast<uintptr_t>(data) % a) == 0; }
};

void set_last_error(const char* fmt, ...);
const char* last_error();

// Returns false (and sets the error string) if the handle cannot be described.
bool make_view(diopiConstTensorHandle_t th, TensorView* v, const char* what);

inline bool is_floating(diopiDtype_t t) {
    return t == diopi_dtype_float16 || t == diopi_dtype_bfloat16 || t == diopi_dtype_float32 || t == diopi_dtype_float64;
}
inline bool is_integral(diopiDtype_t t, bool include_bool) {
    switch (t) {
        case diopi_dtype_int8: case diopi_dtype_uint8: case diopi_dtype_int16: case diopi_dtype_uint16:
        case diopi_dtype_int32: case diopi_dtype_uint32: case diopi_dtype_int64: case diopi_dtype_uint64:
            return true;
        case diopi_dtype_bool:
            return include_bool;
        default:
            return false;
    }
}
int64_t dtype_size(diopiDtype_t t);
const char* dtype_name(diopiDtype_t t);

cudaStream_t stream_of(diopiContextHandle_t ctx);

// Programmatic dependent launch (the single-row-block product in gemm_tc.cu is launched that way); B200_NO_PDL in the
// environment turns the launch attribute off.
inline bool pdl_enabled() {
    static const bool on = std::getenv("B200_NO_PDL") == nullptr;
    return on;
}

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace b200

#define B200_FAIL(...)                      \
    do {                                    \
        ::b200::set_last_error(__VA_ARGS__); \
        return diopiErrorOccurred;          \
    } while (0)

#define B200_CHECK(cond, ...)        \
    do {                             \
        if (!(cond)) B200_FAIL(__VA_ARGS__); \
    } while (0)

#define B200_VIEW(var, handle)                                         \
    ::b200::TensorView var;                                            \
    if (!::b200::make_view((handle), &var, #handle)) return diopiErrorOccurred;

// A launch error is reported without synchronising; sticky faults surface on the host's next sync.
#define B200_LAUNCH_CHECK(name)                                                        \
    do {                                                                               \
        cudaError_t e__ = cudaPeekAtLastError();                                       \
        if (e__ != cudaSuccess) {                                                      \
            (void)cudaGetLastError();                                                  \
            B200_FAIL("%s: kernel launch failed: %s", (name), cudaGetErrorString(e__)); \
        }                                                                              \
    } while (0)

#define B200_CUDA(expr)                                                              \
    do {                                                                             \
        cudaError_t e__ = (expr);                                                    \
        if (e__ != cudaSuccess) {                                                    \
            (void)cudaGetLastError();                                                \
            B200_FAIL("%s failed: %s", #expr, cudaGetErrorString(e__));              \
        }                                                                            \
    } while (0)
