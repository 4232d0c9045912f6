// vendorMakeGenerator for the B200 vendor: the RNG state container DIPU asks its vendor for
// (reference dipu/torch_dipu/csrc_dipu/vendor/cuda/CudaGeneratorImpl.cpp:17-85; base class and factory declaration
// runtime/core/DIPUGeneratorImpl.h:10-63). The state a Philox-based device generator needs is a 64-bit seed and a 64-bit
// offset (a multiple of 4); get_state() serialises them as 16 bytes, set_state() accepts 16 bytes or the seed alone.
// In a DIPU build the base class is DIPU's own header; it is restated here (same members, own implementation) so that the
// file compiles and can be exercised without the DIPU tree.
#include <cstring>
#include <memory>
#include <mutex>

#include <ATen/Utils.h>
#include <ATen/core/Generator.h>
#include <ATen/core/Tensor.h>
#include <ATen/ops/empty.h>
#include <c10/core/GeneratorImpl.h>

#if __has_include(<csrc_dipu/runtime/core/DIPUGeneratorImpl.h>)
#include <csrc_dipu/runtime/core/DIPUGeneratorImpl.h>
#else
namespace dipu {

class DIPUGeneratorImpl : public c10::GeneratorImpl {
  public:
    explicit DIPUGeneratorImpl(at::DeviceIndex device_index = -1)
        : c10::GeneratorImpl(c10::Device(c10::DeviceType::PrivateUse1, device_index), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1)) {}
    ~DIPUGeneratorImpl() override = default;

    void set_current_seed(uint64_t seed) override {
        seed_ = seed;
        offset_ = 0;
        state_need_reset_ = true;
    }
    uint64_t current_seed() const override { return seed_; }
    uint64_t seed() override {
        const uint64_t s = c10::detail::getNonDeterministicRandom(true);
        set_current_seed(s);
        return s;
    }
    static at::DeviceType device_type() { return c10::DeviceType::PrivateUse1; }
    c10::intrusive_ptr<c10::TensorImpl> get_state() const override {
        update_state();
        return state_.getIntrusivePtr();
    }
    void set_offset(uint64_t offset) override {
        offset_ = offset;
        state_need_reset_ = true;
    }
    uint64_t get_offset() const override { return offset_; }

  protected:
    virtual void update_state() const = 0;
    uint64_t offset_ = 0;
    uint64_t seed_ = c10::default_rng_seed_val;
    mutable at::Tensor state_;
    mutable bool state_need_reset_ = true;
};

}  // namespace dipu
#endif

namespace dipu {
namespace {

constexpr size_t kSeedBytes = sizeof(uint64_t);
constexpr size_t kOffsetBytes = sizeof(int64_t);
constexpr size_t kStateBytes = kSeedBytes + kOffsetBytes;

class B200GeneratorImpl final : public DIPUGeneratorImpl {
  public:
    explicit B200GeneratorImpl(at::DeviceIndex device_index) : DIPUGeneratorImpl(device_index) {}

    void set_state(const c10::TensorImpl& state) override {
        at::detail::check_rng_state(state);
        const auto n = static_cast<size_t>(state.numel());
        TORCH_CHECK(n == kStateBytes || n == kSeedBytes, "RNG state is wrong size: expected ", kStateBytes, " or ", kSeedBytes, " bytes, got ", n);
        const auto* bytes = state.data_dtype_initialized<uint8_t>();
        uint64_t seed = 0;
        int64_t offset = 0;
        std::memcpy(&seed, bytes, kSeedBytes);
        if (n == kStateBytes) std::memcpy(&offset, bytes + kSeedBytes, kOffsetBytes);
        set_current_seed(seed);
        set_offset(static_cast<uint64_t>(offset));
    }

    void set_offset(uint64_t offset) override {
        TORCH_CHECK(offset % 4 == 0, "offset must be a multiple of 4");
        DIPUGeneratorImpl::set_offset(offset);
    }

  protected:
    void update_state() const override {
        if (!state_need_reset_) return;
        state_ = at::empty({static_cast<int64_t>(kStateBytes)}, at::TensorOptions().dtype(at::kByte).device(at::kCPU));
        auto* bytes = state_.data_ptr<uint8_t>();
        const uint64_t seed = current_seed();
        const int64_t offset = static_cast<int64_t>(get_offset());
        std::memcpy(bytes, &seed, kSeedBytes);
        std::memcpy(bytes + kSeedBytes, &offset, kOffsetBytes);
        state_need_reset_ = false;
    }

    B200GeneratorImpl* clone_impl() const override {
        auto* g = new B200GeneratorImpl(device().index());
        g->set_current_seed(current_seed());
        g->set_offset(get_offset());
        return g;
    }
};

}  // namespace

// NOLINTNEXTLINE(readability-const-return-type)
__attribute__((visibility("default"))) const at::Generator vendorMakeGenerator(at::DeviceIndex device_index) {
    return at::make_generator<B200GeneratorImpl>(device_index);
}

}  // namespace dipu

// Exercises the container from plain C (tests load this library with ctypes): seed / offset round trip through
// get_state -> set_state, clone independence, the offset rule. Returns 0 when everything holds, else the failed check's number.
extern "C" __attribute__((visibility("default"))) int b200_torchabi_generator_selftest(void) {
    try {
        at::Generator a = dipu::vendorMakeGenerator(0);
        at::Generator b = dipu::vendorMakeGenerator(0);
        if (a.device().type() != c10::DeviceType::PrivateUse1 || a.device().index() != 0) return 1;
        a.set_current_seed(1234567);
        a.set_offset(64);
        const at::Tensor st = a.get_state();
        if (st.numel() != 16 || st.scalar_type() != at::kByte) return 2;
        b.set_state(st);
        if (b.current_seed() != 1234567 || b.get_offset() != 64) return 3;
        at::Generator c = a.clone();
        a.set_current_seed(7);
        if (c.current_seed() != 1234567 || c.get_offset() != 64 || a.get_offset() != 0) return 4;
        bool threw = false;
        try {
            a.set_offset(3);
        } catch (const c10::Error&) {
            threw = true;
        }
        if (!threw) return 5;
        const at::Tensor seed_only = st.slice(0, 0, 8).clone();
        b.set_state(seed_only);
        if (b.current_seed() != 1234567 || b.get_offset() != 0) return 6;
        return 0;
    } catch (...) {
        return 100;
    }
}
