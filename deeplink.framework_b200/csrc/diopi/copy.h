// Internal copy services used by other ops (layout normalisation of non-contiguous inputs, cat, ...).
#pragma once

#include "common.h"

namespace b200 {

// dst <- src with dtype conversion, broadcast of src and arbitrary strides; enqueued on the context's stream.
diopiError_t copy_impl(diopiContextHandle_t ctx, const TensorView& src, const TensorView& dst);

// Returns `v` itself when it is dense, else a dense copy held in context-owned workspace.
diopiError_t make_contiguous(diopiContextHandle_t ctx, const TensorView& v, TensorView* out);

}  // namespace b200
