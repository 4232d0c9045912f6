// A thin eager adapter in DIPU's shape: aten ops of the transformer-inference hot path registered on the PrivateUse1
// dispatch key (named "dipu"), each one the wrapper recipe of the reference's generated code - check the arguments,
// allocate the outputs through the caching allocator, build a diopiContext on the current stream, call ::diopiXxx, release
// the workspace (reference dipu/scripts/autogen_diopi_wrapper/diopi_wrapper_template.py:100-142, the per-op entries of
// diopi_functions.yaml, tensor wrapping as in dipu/torch_dipu/csrc_dipu/aten/ops/DIPUOpInferrer.cpp and
// diopirt/diopirt_impl.cpp:24-173). There is no CPU fallback: an op that is not registered here raises torch's own
// "not implemented for PrivateUse1" error.
#pragma once

#include <ATen/ATen.h>
#include <c10/core/Allocator.h>
#include <c10/core/Device.h>
#include <c10/core/Stream.h>

#include "diopi/diopirt.h"
#include "diopi/functions.h"
#include "diopi/functions_ext.h"
#include "dipu_b200/vendor_c_api.h"
#include "../minihost/minihost_structs.h"

extern "C" void minihostResetContext(diopiContextHandle_t ctx);
extern "C" const char* diopiGetLastErrorString(void);

namespace dipu_b200 {

constexpr c10::DeviceType kDevice = c10::DeviceType::PrivateUse1;

// Counters of the wrapper layer (read from Python): how many DIOPI calls were issued.
struct AdapterStats {
    int64_t diopi_calls = 0;
    int64_t allocations = 0;
    int64_t host_copies = 0;
};
// exported: the c10d backend library links against them
#define DIPU_B200_EXPORT __attribute__((visibility("default")))
DIPU_B200_EXPORT AdapterStats& stats();

DIPU_B200_EXPORT b200Stream_t current_stream(int device);
DIPU_B200_EXPORT c10::Allocator* device_allocator();

DIPU_B200_EXPORT diopiDtype_t to_diopi_dtype(at::ScalarType t);

// An at::Tensor described for the operator library (no ownership; valid while the tensor lives).
struct Wrapped : diopiTensor {
    Wrapped() = default;
    explicit Wrapped(const at::Tensor& t);
};

// Stack context of one wrapper call: the current stream; workspace requested by the library is released on exit.
struct CallContext : diopiContext {
    explicit CallContext(const at::Tensor& device_tensor);
    ~CallContext() { minihostResetContext(this); }
};

inline diopiScalar_t to_diopi_scalar(const at::Scalar& s) {
    diopiScalar_t r;
    if (s.isFloatingPoint()) {
        r.stype = diopi_dtype_float64;
        r.fval = s.toDouble();
    } else {
        r.stype = diopi_dtype_int64;
        r.ival = s.toLong();  // booleans travel as int64, like the reference's helper (diopi_helper.cpp:74-119)
    }
    return r;
}

#define DIPU_B200_CALL(expr)                                                                                                 \
    do {                                                                                                                     \
        ++::dipu_b200::stats().diopi_calls;                                                                                  \
        const diopiError_t rc__ = (expr);                                                                                    \
        TORCH_CHECK(rc__ == diopiSuccess, #expr, " failed with code ", static_cast<int>(rc__), ": ", diopiGetLastErrorString()); \
    } while (0)

}  // namespace dipu_b200
