// Host-side common code of the operator library: error string, tensor snapshots, library identity.
#include "common.h"

#include <mutex>

namespace b200 {

namespace {
thread_local char g_err[1024] = "";
}

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
const char* last_error() { return g_err; }

int64_t dtype_size(diopiDtype_t t) {
    switch (t) {
        case diopi_dtype_int8: case diopi_dtype_uint8: case diopi_dtype_bool: return 1;
        case diopi_dtype_int16: case diopi_dtype_uint16: case diopi_dtype_float16: case diopi_dtype_bfloat16: return 2;
        case diopi_dtype_int32: case diopi_dtype_uint32: case diopi_dtype_float32: case diopi_dtype_tfloat32: return 4;
        case diopi_dtype_int64: case diopi_dtype_uint64: case diopi_dtype_float64: case diopi_dtype_complex64: return 8;
        case diopi_dtype_complex128: return 16;
        default: return 0;
    }
}

const char* dtype_name(diopiDtype_t t) {
    switch (t) {
        case diopi_dtype_int8: return "int8";
        case diopi_dtype_uint8: return "uint8";
        case diopi_dtype_int16: return "int16";
        case diopi_dtype_uint16: return "uint16";
        case diopi_dtype_int32: return "int32";
        case diopi_dtype_uint32: return "uint32";
        case diopi_dtype_int64: return "int64";
        case diopi_dtype_uint64: return "uint64";
        case diopi_dtype_float16: return "float16";
        case diopi_dtype_float32: return "float32";
        case diopi_dtype_float64: return "float64";
        case diopi_dtype_bool: return "bool";
        case diopi_dtype_bfloat16: return "bfloat16";
        case diopi_dtype_tfloat32: return "tfloat32";
        case diopi_dtype_complex64: return "complex64";
        case diopi_dtype_complex128: return "complex128";
        default: return "unsupported";
    }
}

bool make_view(diopiConstTensorHandle_t th, TensorView* v, const char* what) {
    if (th == nullptr) {
        set_last_error("%s: tensor handle is NULL", what);
        return false;
    }
    diopiSize_t shape{nullptr, 0}, stride{nullptr, 0};
    const void* ptr = nullptr;
    if (diopiGetTensorShape(th, &shape) != diopiSuccess || diopiGetTensorStride(th, &stride) != diopiSuccess ||
        diopiGetTensorDtype(th, &v->dtype) != diopiSuccess || diopiGetTensorDevice(th, &v->device) != diopiSuccess ||
        diopiGetTensorDataConst(th, &ptr) != diopiSuccess) {
        set_last_error("%s: host callback failed while reading tensor metadata", what);
        return false;
    }
    if (shape.len > kMaxDims || shape.len != stride.len) {
        set_last_error("%s: rank %lld not supported (max %d)", what, (long long)shape.len, kMaxDims);
        return false;
    }
    v->ndim = static_cast<int>(shape.len);
    v->numel = 1;
    for (int i = 0; i < v->ndim; ++i) {
        v->shape[i] = shape.data[i];
        v->stride[i] = stride.data[i];
        v->numel *= shape.data[i];
    }
    v->itemsize = dtype_size(v->dtype);
    if (v->itemsize == 0) {
        set_last_error("%s: dtype %d not supported", what, (int)v->dtype);
        return false;
    }
    v->data = const_cast<void*>(ptr);
    v->defined = true;
    return true;
}

cudaStream_t stream_of(diopiContextHandle_t ctx) {
    diopiStreamHandle_t s = nullptr;
    diopiGetStream(ctx, &s);
    return static_cast<cudaStream_t>(s);
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace b200

extern "C" {
DIOPI_API const char* diopiGetVendorName(void) { return "b200"; }
DIOPI_API const char* diopiGetImplVersion(void) { return "b200-sm_100a diopi impl 0.1 (CUDA 12.9)"; }
DIOPI_API const char* diopiGetLastErrorString(void) { return b200::last_error(); }
}
