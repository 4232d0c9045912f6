// Minimal DIOPI host: plays DIPU's part of the diopirt contract for tests, benchmarks and non-torch callers.
//
// DIPU hands the operator library `at::Tensor*` as the opaque tensor handle and a stack-allocated context holding the
// current stream plus the workspace tensors requested during the call
// (dipu/torch_dipu/csrc_dipu/diopirt/diopirt_impl.h:19-26, diopirt_impl.cpp:24-173). This host does the same with a
// plain struct instead of at::Tensor, so the boundary is exercised without linking libtorch: the caller describes
// memory it owns (pointer, shape, strides, dtype, device) and workspace comes from the vendor runtime's caching
// allocator exactly as diopiRequireTensor routes to DIPU's allocator.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <vector>

#include "diopi/diopirt.h"
#include "dipu_b200/vendor_c_api.h"
#include "minihost_structs.h"

namespace {

int64_t elem_size(diopiDtype_t t) {
    switch (t) {
        case diopi_dtype_int8: case diopi_dtype_uint8: case diopi_dtype_bool: return 1;
        case diopi_dtype_int16: case diopi_dtype_uint16: case diopi_dtype_float16: case diopi_dtype_bfloat16: return 2;
        case diopi_dtype_int32: case diopi_dtype_uint32: case diopi_dtype_float32: case diopi_dtype_tfloat32: return 4;
        case diopi_dtype_int64: case diopi_dtype_uint64: case diopi_dtype_float64: case diopi_dtype_complex64: return 8;
        case diopi_dtype_complex128: return 16;
        default: return 0;
    }
}

}  // namespace

extern "C" {

// ---- host-side construction API (what a non-torch caller uses) -------------------------------------------------
DIOPI_RT_API diopiTensorHandle_t minihostMakeTensor(void* data, int64_t ndim, const int64_t* shape, const int64_t* stride /* NULL = dense */,
                                                    int dtype, int device, int device_index) {
    if (ndim < 0 || ndim > 8 || elem_size(static_cast<diopiDtype_t>(dtype)) == 0) return nullptr;
    diopiTensor* t = new diopiTensor();
    t->data = data;
    t->dtype = static_cast<diopiDtype_t>(dtype);
    t->device = static_cast<diopiDevice_t>(device);
    t->device_index = device_index;
    t->ndim = ndim;
    t->numel = 1;
    t->itemsize = elem_size(t->dtype);
    int64_t dense = 1;
    for (int64_t d = ndim - 1; d >= 0; --d) {
        t->shape[d] = shape[d];
        t->stride[d] = stride ? stride[d] : dense;
        dense *= shape[d];
        t->numel *= shape[d];
    }
    int64_t span = t->numel > 0 ? 1 : 0;
    for (int64_t d = 0; d < ndim && t->numel > 0; ++d) span += (t->shape[d] - 1) * (t->stride[d] < 0 ? 0 : t->stride[d]);
    t->storage_nbytes = static_cast<size_t>(span * t->itemsize);
    return t;
}

DIOPI_RT_API void minihostFreeTensor(diopiTensorHandle_t t) {
    if (t == nullptr) return;
    if (t->owns_memory && t->data != nullptr) (void)b200_cache_free(t->data);
    if (t->owns_host_memory && t->data != nullptr) (void)b200_host_cache_free(t->data);
    delete t;
}

DIOPI_RT_API diopiContextHandle_t minihostMakeContext(void* stream, int device_index) {
    diopiContext* c = new diopiContext();
    c->stream = stream;
    c->device_index = device_index;
    return c;
}

// Releases the workspace tensors (stream-ordered reuse keeps this safe: they were allocated for ctx->stream).
DIOPI_RT_API void minihostResetContext(diopiContextHandle_t ctx) {
    if (ctx == nullptr) return;
    for (diopiTensor* t : ctx->arrays) minihostFreeTensor(t);
    ctx->arrays.clear();
}

DIOPI_RT_API void minihostFreeContext(diopiContextHandle_t ctx) {
    if (ctx == nullptr) return;
    minihostResetContext(ctx);
    delete ctx;
}

DIOPI_RT_API diopiGeneratorHandle_t minihostMakeGenerator(uint64_t seed) {
    diopiGenerator* g = new diopiGenerator();
    g->seed = seed;
    return g;
}
DIOPI_RT_API void minihostFreeGenerator(diopiGeneratorHandle_t g) { delete g; }

DIOPI_RT_API diopiError_t diopiGeneratorGetSeedAndOffset(diopiGeneratorHandle_t th, uint64_t* seed, uint64_t* offset) {
    if (th == nullptr) return diopiErrorOccurred;
    *seed = th->seed;
    *offset = th->offset;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGeneratorSetSeedAndOffset(diopiGeneratorHandle_t th, uint64_t seed, uint64_t offset) {
    if (th == nullptr) return diopiErrorOccurred;
    th->seed = seed;
    th->offset = offset;
    return diopiSuccess;
}

DIOPI_RT_API int64_t minihostWorkspaceCount(diopiContextHandle_t ctx) { return ctx ? static_cast<int64_t>(ctx->arrays.size()) : 0; }

// ---- diopirt callbacks -------------------------------------------------------------------------------------------
DIOPI_RT_API const char* diopiGetVersion(void) { return "DIOPI minihost (b200) 1.0"; }

DIOPI_RT_API diopiError_t diopiGetTensorData(diopiTensorHandle_t th, void** pptr) {
    *pptr = th->data;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorDataConst(diopiConstTensorHandle_t th, const void** pptr) {
    *pptr = th->data;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorShape(diopiConstTensorHandle_t th, diopiSize_t* size) {
    size->data = th->shape;
    size->len = th->ndim;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorStride(diopiConstTensorHandle_t th, diopiSize_t* stride) {
    stride->data = th->stride;
    stride->len = th->ndim;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorDtype(diopiConstTensorHandle_t th, diopiDtype_t* dtype) {
    *dtype = th->dtype;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorDevice(diopiConstTensorHandle_t th, diopiDevice_t* device) {
    *device = th->device;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorNumel(diopiConstTensorHandle_t th, int64_t* numel) {
    *numel = th->numel;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorElemSize(diopiConstTensorHandle_t th, int64_t* itemsize) {
    *itemsize = th->itemsize;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorStoragePtr(diopiConstTensorHandle_t th, void** pStoragePtr) {
    *pStoragePtr = static_cast<char*>(th->data) - th->storage_offset * th->itemsize;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorStorageOffset(diopiConstTensorHandle_t th, int64_t* pOffset) {
    *pOffset = th->storage_offset;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorStorageNbytes(diopiConstTensorHandle_t th, size_t* pNbytes) {
    *pNbytes = th->storage_nbytes;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetTensorDeviceIndex(diopiConstTensorHandle_t th, diopiDeviceIndex_t* pDevIndex) {
    *pDevIndex = th->device_index;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetCurrentDeviceIndex(diopiDeviceIndex_t* pDevIndex) {
    int dev = 0;
    if (b200_current_device(&dev) != B200_SUCCESS) return diopiErrorOccurred;
    *pDevIndex = dev;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiGetStream(diopiContextHandle_t ctx, diopiStreamHandle_t* stream) {
    *stream = ctx->stream;
    return diopiSuccess;
}

DIOPI_RT_API diopiError_t diopiRequireTensor(diopiContextHandle_t ctx, diopiTensorHandle_t* tensor, const diopiSize_t* size,
                                             const diopiSize_t* stride, const diopiDtype_t dtype, const diopiDevice_t device) {
    if (ctx == nullptr || tensor == nullptr || size == nullptr || size->len > 8) return diopiErrorOccurred;
    diopiTensor* t = minihostMakeTensor(nullptr, size->len, size->data, (stride && stride->data) ? stride->data : nullptr, dtype, device,
                                        ctx->device_index);
    if (t == nullptr) return diopiErrorOccurred;
    if (t->storage_nbytes > 0) {
        void* p = nullptr;
        b200Status_t st;
        if (device == diopi_device) {
            st = b200_cache_alloc(&p, t->storage_nbytes, ctx->device_index, ctx->stream);
        } else {
            st = b200_host_cache_alloc(&p, t->storage_nbytes);
        }
        if (st != B200_SUCCESS) {
            delete t;
            return diopiErrorOccurred;
        }
        t->data = p;
        t->owns_memory = (device == diopi_device);
        t->owns_host_memory = (device != diopi_device);
    }
    ctx->arrays.push_back(t);
    *tensor = t;
    return diopiSuccess;
}

DIOPI_RT_API diopiError_t diopiRequireBuffer(diopiContextHandle_t ctx, diopiTensorHandle_t* tensor, int64_t num_bytes, diopiDevice_t device) {
    diopiSize_t size{&num_bytes, 1};
    return diopiRequireTensor(ctx, tensor, &size, nullptr, diopi_dtype_int8, device);
}

// Profiler hooks: no-ops here (DIPU brackets them with kineto records, diopirt_impl.cpp:224-237).
DIOPI_RT_API diopiError_t diopiRecordStart(const char*, void** record) {
    if (record) *record = nullptr;
    return diopiSuccess;
}
DIOPI_RT_API diopiError_t diopiRecordEnd(void** record) {
    if (record) *record = nullptr;
    return diopiSuccess;
}

}  // extern "C"
