// vendorapi.h of the B200 vendor: the per-vendor header DIPU symlinks to csrc_dipu/vendor/vendorapi.h
// (reference: dipu/torch_dipu/csrc_dipu/vendor/cuda/vendorapi.h:37-49 defines the same five names for the CUDA vendor).
#pragma once

#include <cuda_runtime.h>

#include <c10/util/Exception.h>

#include "dipu_b200/vendor_c_api.h"

namespace dipu {

using deviceStream_t = cudaStream_t;
#define deviceDefaultStreamLiteral cudaStreamLegacy
using deviceEvent_t = cudaEvent_t;
using diclComm_t = b200Comm_t;
using commUniqueId = b200UniqueId;  // trivially copyable; travels through the c10d store as DICL_UNIQUE_ID_BYTES_SIZE bytes

// Void devapis functions report failure by throwing c10::Error, as the CUDA vendor's DIPU_CALLCUDA does.
#define DIPU_CALLB200(Expr)                                                                                          \
    {                                                                                                                \
        b200Status_t ret_ = (Expr);                                                                                  \
        TORCH_CHECK(ret_ == B200_SUCCESS, "call b200 error, expr = ", #Expr, ", ret = ", static_cast<int>(ret_), ": ", \
                    b200_last_error());                                                                              \
    }

}  // namespace dipu
