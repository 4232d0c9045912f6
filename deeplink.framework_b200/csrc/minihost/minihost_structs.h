// The two structs behind the opaque diopiTensorHandle_t / diopiContextHandle_t of the minimal DIOPI host. Callers that
// build them in place (the torch adapter wraps an at::Tensor per argument, on the stack) include this header; everyone
// else goes through minihostMakeTensor / minihostMakeContext.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

#include "diopi/diopirt.h"

struct diopiTensor {
    void* data = nullptr;
    diopiDtype_t dtype = diopi_dtype_float32;
    diopiDevice_t device = diopi_device;
    int32_t device_index = 0;
    int64_t ndim = 0;
    int64_t shape[8] = {0};
    int64_t stride[8] = {0};
    int64_t numel = 0;
    int64_t itemsize = 0;
    int64_t storage_offset = 0;  // elements
    size_t storage_nbytes = 0;
    bool owns_memory = false;    // workspace allocated through the caching device allocator
    bool owns_host_memory = false;  // workspace allocated through the pinned-host cache
};

struct diopiContext {
    diopiStreamHandle_t stream = nullptr;
    int32_t device_index = 0;
    std::vector<diopiTensor*> arrays;  // workspace, released with the context
};

struct diopiGenerator {
    uint64_t seed = 67280421310721ull;
    uint64_t offset = 0;
};
