// Runtime half of the eager adapter: backend name, device allocator on the caching allocator, device guard, tensor
// wrapping, factory ops and copies (reference: DIPU registers its allocator with c10::SetAllocator,
// runtime/core/allocator/DIPUCachingAllocator.cpp:336-342; guard runtime/core/guardimpl/DIPUGuardImpl.h; copy strategy
// aten/ops/DIPUCopy.hpp:361-527).
#include <cuda_runtime.h>

#include <ATen/EmptyTensor.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <ATen/native/Resize.h>
#include <ATen/native/TensorShape.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <torch/library.h>

#include "adapter_common.h"

namespace dipu_b200 {

#define VENDOR_CHECK(expr)                                                                                        \
    do {                                                                                                          \
        const b200Status_t st__ = (expr);                                                                         \
        TORCH_CHECK(st__ == B200_SUCCESS, #expr, " failed with status ", static_cast<int>(st__), ": ", b200_last_error()); \
    } while (0)

AdapterStats& stats() {
    static AdapterStats s;
    return s;
}

b200Stream_t current_stream(int device) {
    b200Stream_t s = nullptr;
    VENDOR_CHECK(b200_default_stream(device, &s));
    return s;
}

diopiDtype_t to_diopi_dtype(at::ScalarType t) {
    switch (t) {
        case at::kBool: return diopi_dtype_bool;
        case at::kChar: return diopi_dtype_int8;
        case at::kByte: return diopi_dtype_uint8;
        case at::kShort: return diopi_dtype_int16;
        case at::kInt: return diopi_dtype_int32;
        case at::kLong: return diopi_dtype_int64;
        case at::kHalf: return diopi_dtype_float16;
        case at::kBFloat16: return diopi_dtype_bfloat16;
        case at::kFloat: return diopi_dtype_float32;
        case at::kDouble: return diopi_dtype_float64;
        case at::kComplexFloat: return diopi_dtype_complex64;
        case at::kComplexDouble: return diopi_dtype_complex128;
        default: TORCH_CHECK(false, "dtype ", t, " has no DIOPI counterpart");
    }
}

Wrapped::Wrapped(const at::Tensor& t) {
    TORCH_CHECK(t.dim() <= 8, "tensors of more than 8 dimensions are not supported");
    data = t.data_ptr();
    dtype = to_diopi_dtype(t.scalar_type());
    device = t.is_cpu() ? diopi_host : diopi_device;
    device_index = t.is_cpu() ? 0 : t.device().index();
    ndim = t.dim();
    for (int64_t d = 0; d < ndim; ++d) {
        shape[d] = t.size(d);
        stride[d] = t.stride(d);
    }
    numel = t.numel();
    itemsize = static_cast<int64_t>(t.element_size());
    storage_offset = t.storage_offset();
    storage_nbytes = t.storage().nbytes();
}

CallContext::CallContext(const at::Tensor& device_tensor) {
    device_index = device_tensor.device().index();
    stream = current_stream(device_index);
}

// ---- allocator ------------------------------------------------------------------------------------------------------------
namespace {

void delete_block(void* p) {
    if (p != nullptr) (void)b200_cache_free(p);
}

struct DeviceAllocator final : c10::Allocator {
    c10::DataPtr allocate(size_t nbytes) override {
        int dev = 0;
        VENDOR_CHECK(b200_current_device(&dev));
        void* p = nullptr;
        if (nbytes > 0) {
            const b200Status_t st = b200_cache_alloc(&p, nbytes, dev, current_stream(dev));
            TORCH_CHECK(st == B200_SUCCESS, "dipu: out of memory allocating ", nbytes, " bytes: ", b200_last_error());
            ++stats().allocations;
        }
        return {p, p, &delete_block, c10::Device(kDevice, static_cast<c10::DeviceIndex>(dev))};
    }
    c10::DeleterFnPtr raw_deleter() const override { return &delete_block; }
    void copy_data(void* dest, const void* src, std::size_t count) const override {
        int dev = 0;
        (void)b200_current_device(&dev);
        (void)b200_memcpy_d2d(count, dev, dest, dev, src);
    }
};

DeviceAllocator g_allocator;
}  // namespace

c10::Allocator* device_allocator() { return &g_allocator; }

namespace {

// ---- device guard ----------------------------------------------------------------------------------------------------------
struct GuardImpl final : c10::impl::DeviceGuardImplInterface {
    c10::DeviceType type() const override { return kDevice; }
    c10::Device exchangeDevice(c10::Device d) const override {
        const c10::Device old = getDevice();
        if (old.index() != d.index()) setDevice(d);
        return old;
    }
    c10::Device getDevice() const override {
        int dev = 0;
        VENDOR_CHECK(b200_current_device(&dev));
        return c10::Device(kDevice, static_cast<c10::DeviceIndex>(dev));
    }
    void setDevice(c10::Device d) const override { VENDOR_CHECK(b200_set_device(d.index())); }
    void uncheckedSetDevice(c10::Device d) const noexcept override { (void)b200_set_device(d.index()); }
    c10::Stream getStream(c10::Device d) const noexcept override { return c10::Stream(c10::Stream::DEFAULT, d); }
    c10::Stream getDefaultStream(c10::Device d) const override { return c10::Stream(c10::Stream::DEFAULT, d); }
    c10::Stream exchangeStream(c10::Stream s) const noexcept override { return c10::Stream(c10::Stream::DEFAULT, s.device()); }
    c10::DeviceIndex deviceCount() const noexcept override {
        int n = 0;
        if (b200_get_device_count(&n) != B200_SUCCESS) return 0;
        return static_cast<c10::DeviceIndex>(n);
    }
    bool queryStream(const c10::Stream& s) const override { return b200_is_stream_empty(current_stream(s.device_index())) != 0; }
    void synchronizeStream(const c10::Stream& s) const override { VENDOR_CHECK(b200_sync_stream(current_stream(s.device_index()))); }
    void synchronizeDevice(const c10::DeviceIndex) const override { VENDOR_CHECK(b200_sync_device()); }
};

C10_REGISTER_GUARD_IMPL(PrivateUse1, GuardImpl);

// What torch asks an accelerator backend outside of operator dispatch (torch.accelerator, torch.distributed.barrier, ...).
struct Hooks final : at::PrivateUse1HooksInterface {
    bool isBuilt() const override { return true; }
    bool isAvailable() const override { return deviceCount() > 0; }
    bool hasPrimaryContext(c10::DeviceIndex) const override { return true; }
    c10::DeviceIndex deviceCount() const override {
        int n = 0;
        if (b200_get_device_count(&n) != B200_SUCCESS) return 0;
        return static_cast<c10::DeviceIndex>(n);
    }
    void setCurrentDevice(c10::DeviceIndex device) const override { VENDOR_CHECK(b200_set_device(device)); }
    c10::DeviceIndex getCurrentDevice() const override {
        int dev = 0;
        VENDOR_CHECK(b200_current_device(&dev));
        return static_cast<c10::DeviceIndex>(dev);
    }
    c10::DeviceIndex exchangeDevice(c10::DeviceIndex device) const override {
        const c10::DeviceIndex old = getCurrentDevice();
        if (old != device) setCurrentDevice(device);
        return old;
    }
    c10::DeviceIndex maybeExchangeDevice(c10::DeviceIndex device) const override { return exchangeDevice(device); }
    bool isPinnedPtr(const void* data) const override { return b200_is_pinned_ptr(const_cast<void*>(data)) != 0; }
};

struct Registrar {
    Registrar() {
        c10::register_privateuse1_backend("dipu");
        c10::SetAllocator(kDevice, &g_allocator);
        at::RegisterPrivateUse1HooksInterface(new Hooks());  // owned by torch for the life of the process
    }
};
Registrar g_registrar;

// ---- factories ---------------------------------------------------------------------------------------------------------------
at::Tensor empty_memory_format(c10::IntArrayRef size, std::optional<at::ScalarType> dtype, std::optional<at::Layout>, std::optional<at::Device> device,
                               std::optional<bool>, std::optional<at::MemoryFormat> memory_format) {
    const c10::DeviceGuard guard(device.value_or(c10::Device(kDevice, 0)));
    return at::detail::empty_generic(size, &g_allocator, c10::DispatchKeySet(c10::DispatchKey::PrivateUse1), dtype.value_or(at::kFloat), memory_format);
}

at::Tensor empty_strided(c10::IntArrayRef size, c10::IntArrayRef stride, std::optional<at::ScalarType> dtype, std::optional<at::Layout>,
                         std::optional<at::Device> device, std::optional<bool>) {
    const c10::DeviceGuard guard(device.value_or(c10::Device(kDevice, 0)));
    return at::detail::empty_strided_generic(size, stride, &g_allocator, c10::DispatchKeySet(c10::DispatchKey::PrivateUse1), dtype.value_or(at::kFloat));
}

// ---- copies ----------------------------------------------------------------------------------------------------------------
// device <-> device (any dtype / stride pair) goes to diopiCopyInp; host <-> device moves dense bytes of one dtype with the
// vendor's copy calls and leaves casts / strides to a device-side diopiCopyInp, as DIPU's copy strategy does.
void device_copy(const at::Tensor& src, const at::Tensor& dst) {
    CallContext ctx(dst);
    Wrapped s(src), d(dst);
    DIPU_B200_CALL(diopiCopyInp(&ctx, &s, &d));
}

// Between two devices the bytes travel dense and in one dtype through the copy engines (memCopyD2DAsync with the SOURCE device
// current and on the source's stream, as DIPU does it, ops/DIPUCopy.hpp:142-148,371-372); a strided or differently typed side
// is relayed through a dense tensor on its own device first / afterwards. The two devices' streams are ordered by events:
// the source stream waits for what the destination stream has enqueued on the landing buffer, and the destination stream
// waits for the transfer.
void peer_copy(const at::Tensor& src, const at::Tensor& dst) {
    const int sdev = src.device().index(), ddev = dst.device().index();
    at::Tensor dense = src;
    if (!src.is_contiguous()) {
        const c10::DeviceGuard guard(src.device());
        dense = at::empty(src.sizes(), src.options());
        device_copy(src, dense);
    }
    const bool direct = dst.is_contiguous() && dst.scalar_type() == dense.scalar_type();
    at::Tensor landing = dst;
    if (!direct) {
        const c10::DeviceGuard guard(dst.device());
        landing = at::empty(dst.sizes(), dst.options().dtype(dense.scalar_type()));
    }
    b200Stream_t sstream = nullptr, dstream = nullptr;
    b200Event_t ev = nullptr;
    {
        const c10::DeviceGuard guard(dst.device());
        dstream = current_stream(ddev);
        VENDOR_CHECK(b200_event_from_pool(&ev));
        VENDOR_CHECK(b200_record_event(ev, dstream));
    }
    {
        const c10::DeviceGuard guard(src.device());
        sstream = current_stream(sdev);
        VENDOR_CHECK(b200_stream_wait_event(sstream, ev));
        VENDOR_CHECK(b200_event_to_pool(ev));
        VENDOR_CHECK(b200_memcpy_d2d_async(sstream, dense.nbytes(), ddev, landing.data_ptr(), sdev, dense.data_ptr()));
        VENDOR_CHECK(b200_event_from_pool(&ev));
        VENDOR_CHECK(b200_record_event(ev, sstream));
        // the landing buffer belongs to the destination's stream for the allocator; it is also in use on the source's
        if (landing.has_storage() && landing.storage().data() != nullptr) (void)b200_cache_record_stream(landing.storage().mutable_data(), sstream);
    }
    {
        const c10::DeviceGuard guard(dst.device());
        VENDOR_CHECK(b200_stream_wait_event(dstream, ev));
        VENDOR_CHECK(b200_event_to_pool(ev));
        if (dense.has_storage() && dense.storage().data() != nullptr) (void)b200_cache_record_stream(dense.storage().mutable_data(), dstream);
        if (!direct) device_copy(landing, dst);
    }
}

at::Tensor copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
    if (dst.numel() == 0) return dst;
    TORCH_CHECK(self.numel() == dst.numel() || self.sizes() != dst.sizes(), "copy_: size mismatch");
    if (!self.is_cpu() && !dst.is_cpu()) {
        const at::Tensor src = self.sizes() == dst.sizes() ? self : self.expand(dst.sizes());
        if (src.device() == dst.device()) {
            const c10::DeviceGuard guard(dst.device());
            device_copy(src, dst);
            return dst;
        }
        peer_copy(src, dst);
        return dst;
    }
    ++stats().host_copies;
    if (self.is_cpu()) {
        // host -> device: a dense host tensor of the source dtype lands in a dense device tensor, then one device copy
        const c10::DeviceGuard guard(dst.device());
        const at::Tensor host = self.expand(dst.sizes()).contiguous();
        const bool direct = dst.is_contiguous() && dst.scalar_type() == host.scalar_type();
        at::Tensor staging = direct ? dst : at::empty(dst.sizes(), dst.options().dtype(host.scalar_type()));
        b200Stream_t stream = current_stream(dst.device().index());
        VENDOR_CHECK(b200_memcpy_h2d_async(stream, host.nbytes(), staging.data_ptr(), host.data_ptr()));
        // pageable host memory: the source tensor may die when this call returns, so the copy must have read it
        VENDOR_CHECK(b200_sync_stream(stream));
        if (!direct) device_copy(staging, dst);
        return dst;
    }
    // device -> host
    const c10::DeviceGuard guard(self.device());
    at::Tensor dev = self.sizes() == dst.sizes() ? self : self.expand(dst.sizes());
    if (!dev.is_contiguous() || dev.scalar_type() != dst.scalar_type()) {
        at::Tensor dense = at::empty(dst.sizes(), self.options().dtype(dst.scalar_type()));
        device_copy(dev, dense);
        dev = dense;
    }
    at::Tensor host = dst.is_contiguous() ? dst : at::empty(dst.sizes(), dst.options());
    b200Stream_t stream = current_stream(self.device().index());
    VENDOR_CHECK(b200_memcpy_d2h_async(stream, dev.nbytes(), host.data_ptr(), dev.data_ptr()));
    VENDOR_CHECK(b200_sync_stream(stream));
    (void)non_blocking;
    if (!dst.is_contiguous()) dst.copy_(host);
    return dst;
}

at::Scalar local_scalar_dense(const at::Tensor& self) {
    at::Tensor host = at::empty({}, self.options().device(at::kCPU));
    copy_from(self.reshape({}), host, false);
    return host.item();
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("empty.memory_format", &empty_memory_format);
    m.impl("empty_strided", &empty_strided);
    m.impl("_copy_from", &copy_from);
    m.impl("_local_scalar_dense", &local_scalar_dense);
    m.impl("as_strided", &at::native::as_strided_tensorimpl);
    m.impl("view", &at::native::view);
    m.impl("_reshape_alias", &at::native::_reshape_alias);
}

}  // namespace
}  // namespace dipu_b200

// Read from Python (ctypes): counters of the wrapper layer.
extern "C" __attribute__((visibility("default"))) void dipu_b200_adapter_stats(int64_t* diopi_calls, int64_t* allocations, int64_t* host_copies) {
    const dipu_b200::AdapterStats& s = dipu_b200::stats();
    *diopi_calls = s.diopi_calls;
    *allocations = s.allocations;
    *host_copies = s.host_copies;
}
