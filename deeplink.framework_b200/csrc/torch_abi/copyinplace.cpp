// The B200 vendor's copy_ policy object, registered with setDipuCopyInstance (reference
// dipu/torch_dipu/csrc_dipu/vendor/cuda/CUDACopyInplace.cpp:12-76; interface aten/ops/DIPUCopy.hpp:38-83 (copy types),
// 171-220 (CopyParamsInfo), 343-350 (DIPUCopyBase), 727-729 (get / setDipuCopyInstance)).
//
// What run(dst, src, non_blocking) decides, in the reference's order:
//   nothing to do      dst is empty, dst and src are the same tensor, or they alias the same elements with the same
//                      offset / strides / dtype
//   same device        one diopiCopyInp (cast x stride x broadcast in one kernel), always non-blocking: the kernel is
//                      ordered on the current stream like any other operator
//   other device       NVLink is there on every B200 pair of a node: a dense same-layout copy goes through the copy engines
//                      (devapis::memCopyD2DAsync, cudaMemcpyPeerAsync) with the stream hand-over the reference does; anything
//                      that needs a cast or a re-layout first becomes dense on the source device by diopiCopyInp
//   host <-> device    DIPU's relay path (copyAll) followed by record-or-synchronise on the current stream
// In a DIPU tree the actions are DIPU's own helpers. Without the tree (this repository's build) the interface is restated
// here, the actions are counted instead of executed, and b200_torchabi_copy_selftest() checks the decisions on tensors that
// carry only metadata.
#include <cstdint>
#include <cstring>

#include <ATen/core/Tensor.h>
#include <ATen/ops/empty.h>
#include <c10/core/Storage.h>
#include <c10/core/TensorImpl.h>
#include <c10/util/Exception.h>

#if __has_include(<csrc_dipu/aten/ops/DIPUCopy.hpp>)
#include <csrc_dipu/aten/ops/DIPUCopy.hpp>
#include <csrc_dipu/common.h>
#include <csrc_dipu/diopirt/diopirt_impl.h>
#include <csrc_dipu/runtime/core/DIPUStream.h>
#define B200_IN_DIPU_TREE 1
#else
#define B200_IN_DIPU_TREE 0
namespace dipu {

enum class DIPUCopyType { D2Self, D2OtherD, D2H, H2D, H2H };

inline bool isDeviceTensor(const at::Tensor& t) { return t.device().type() == c10::DeviceType::PrivateUse1; }

inline DIPUCopyType getCopyType(const at::Tensor& dst, const at::Tensor& src) {
    const bool s = isDeviceTensor(src), d = isDeviceTensor(dst);
    if (s && d) return src.device().index() == dst.device().index() ? DIPUCopyType::D2Self : DIPUCopyType::D2OtherD;
    if (d) return DIPUCopyType::H2D;
    if (s) return DIPUCopyType::D2H;
    return DIPUCopyType::H2H;
}

struct CopyParamsInfo {
    DIPUCopyType copyType_;
    bool sameDtype_ = false, sameSize_ = false, sameStride_ = false, denseAndNoOverlap_ = false, directMemCopy_ = false;
    c10::DeviceIndex srcDevice_ = -1, dstDevice_ = -1;

    CopyParamsInfo(const at::Tensor& dst, const at::Tensor& src) {
        TORCH_CHECK(dst.options().layout() == c10::Layout::Strided, "only Strided layout is supported");
        copyType_ = getCopyType(dst, src);
        sameDtype_ = dst.scalar_type() == src.scalar_type();
        sameSize_ = dst.sizes().equals(src.sizes());
        sameStride_ = dst.strides().equals(src.strides());
        denseAndNoOverlap_ = dst.is_non_overlapping_and_dense() && src.is_non_overlapping_and_dense();
        directMemCopy_ = sameDtype_ && sameSize_ && sameStride_ && denseAndNoOverlap_;
        srcDevice_ = src.device().index();
        dstDevice_ = dst.device().index();
    }
};

class DIPUCopyBase {
  public:
    DIPUCopyBase() = default;
    virtual ~DIPUCopyBase() = default;
    virtual void run(at::Tensor& dst, const at::Tensor& src, bool non_blocking) = 0;
};

// In the DIPU tree: DIPUCopyInplace<true, false>. Only what this file calls is restated.
class DIPUCopyInpOnDIOPI : public DIPUCopyBase {};

namespace {
DIPUCopyBase*& copy_instance_slot() {
    static DIPUCopyBase* inst = nullptr;
    return inst;
}
}  // namespace
DIPUCopyBase* getDipuCopyInstance() { return copy_instance_slot(); }
void setDipuCopyInstance(DIPUCopyBase* op) { copy_instance_slot() = op; }

}  // namespace dipu
#endif

namespace dipu {

class B200CopyInplace : public DIPUCopyInpOnDIOPI {
  public:
    enum class Action { Nothing, DiopiCopy, PeerEngineCopy, PeerRelayThenEngineCopy, HostRelay };

    struct Counters {
        int64_t nothing = 0, diopi = 0, peer_engine = 0, peer_relay = 0, host = 0, forced_non_blocking = 0;
    };

    B200CopyInplace() = default;
    ~B200CopyInplace() override = default;

    // The decision alone (no side effects): which path a copy takes and whether it may return before the data has landed.
    static Action plan(const at::Tensor& dst, const at::Tensor& src, bool* non_blocking) {
        TORCH_CHECK(dst.defined(), "dst is undefined");
        TORCH_CHECK(src.defined(), "src is undefined");
        if (dst.numel() == 0 || dst.is_same(src)) return Action::Nothing;
        const CopyParamsInfo info(dst, src);
        if (info.copyType_ == DIPUCopyType::D2Self) *non_blocking = true;
        if (dst.is_alias_of(src) && dst.storage_offset() == src.storage_offset() && info.sameStride_ && info.sameDtype_) return Action::Nothing;
        switch (info.copyType_) {
            case DIPUCopyType::D2Self:
                return Action::DiopiCopy;
            case DIPUCopyType::D2OtherD:
                return info.directMemCopy_ ? Action::PeerEngineCopy : Action::PeerRelayThenEngineCopy;
            default:
                return Action::HostRelay;
        }
    }

    void run(at::Tensor& dst, const at::Tensor& src, bool non_blocking) override {
        const bool asked = non_blocking;
        const Action act = plan(dst, src, &non_blocking);
        if (non_blocking && !asked) ++counters_.forced_non_blocking;
        switch (act) {
            case Action::Nothing:
                ++counters_.nothing;
                return;
            case Action::DiopiCopy:
                ++counters_.diopi;
                break;
            case Action::PeerEngineCopy:
                ++counters_.peer_engine;
                break;
            case Action::PeerRelayThenEngineCopy:
                ++counters_.peer_relay;
                break;
            case Action::HostRelay:
                ++counters_.host;
                break;
        }
#if B200_IN_DIPU_TREE
        execute(act, dst, src, non_blocking);
#endif
    }

    const Counters& counters() const { return counters_; }

  private:
#if B200_IN_DIPU_TREE
    void execute(Action act, at::Tensor& dst, const at::Tensor& src, bool non_blocking) {
        using dipu::native::dipu_wrap_diopi_copy_inp;
        if (act == Action::DiopiCopy) {
            dipu_wrap_diopi_copy_inp(dst, src, non_blocking);
            return;
        }
        CopyParamsInfo info(dst, src);
        const DIPUGuard guard((!src.is_cpu()) ? src.device() : dst.device());
        auto curStream = dipu::getCurrentDIPUStream();
        info.updateCurrentStream(curStream);
        if (act == Action::PeerRelayThenEngineCopy) {
            // cast / re-layout on the source device, then one engine copy of dense bytes into a dense landing tensor;
            // a destination that is not dense receives its elements by a second diopiCopyInp on its own device
            at::Tensor dense = at::empty(dst.sizes(), src.options().dtype(dst.scalar_type()));
            dipu_wrap_diopi_copy_inp(dense, src, true);
            if (dst.is_non_overlapping_and_dense() && dst.is_contiguous()) {
                CopyParamsInfo direct(dst, dense);
                direct.updateCurrentStream(curStream);
                copyAll(dst, dense, non_blocking, direct);
            } else {
                at::Tensor landing = at::empty(dst.sizes(), dst.options());
                CopyParamsInfo direct(landing, dense);
                direct.updateCurrentStream(curStream);
                copyAll(landing, dense, non_blocking, direct);
                const DIPUGuard dst_guard(dst.device());
                dipu_wrap_diopi_copy_inp(dst, landing, true);
            }
        } else {
            copyAll(dst, src, non_blocking, info);
        }
        tryRecordOrSyncStream(info, dst, src, curStream, non_blocking, /* block_cpu_d2d = */ false, /* block_cpu_h2d = */ false);
    }
#endif
    Counters counters_;
};

// not const: DIPU's registry hands out a mutable pointer
// NOLINTNEXTLINE(cppcoreguidelines-avoid-non-const-global-variables)
static B200CopyInplace b200_copy_inplace;

// only there to run setDipuCopyInstance when the library is loaded
static const int32_t b200_copy_init = []() {
    setDipuCopyInstance(&b200_copy_inplace);
    return 1;
}();

}  // namespace dipu

namespace {

// A tensor that carries device, dtype, sizes and strides but no memory: enough for the decisions, which read metadata only.
at::Tensor metadata_tensor(c10::Device dev, at::ScalarType dtype, at::IntArrayRef sizes, at::IntArrayRef strides, int64_t offset = 0,
                           c10::Storage* share = nullptr) {
    int64_t span = 1;
    for (size_t i = 0; i < sizes.size(); ++i) span += (sizes[i] > 0 ? sizes[i] - 1 : 0) * strides[i];
    const size_t nbytes = static_cast<size_t>(span + offset) * c10::elementSize(dtype);
    c10::Storage storage = share != nullptr ? *share
                                            : c10::Storage(c10::Storage::use_byte_size_t(), nbytes, c10::DataPtr(nullptr, dev), /*allocator=*/nullptr,
                                                           /*resizable=*/false);
    const c10::DispatchKey key = dev.type() == c10::DeviceType::CPU ? c10::DispatchKey::CPU : c10::DispatchKey::PrivateUse1;
    at::Tensor t = at::detail::make_tensor<c10::TensorImpl>(std::move(storage), c10::DispatchKeySet(key), c10::scalarTypeToTypeMeta(dtype));
    t.unsafeGetTensorImpl()->set_sizes_and_strides(sizes, strides);
    t.unsafeGetTensorImpl()->set_storage_offset(offset);
    return t;
}

}  // namespace

// Exercises the policy from plain C (tests load this library with ctypes). Returns 0 when every decision is the expected
// one, else the number of the failed check.
extern "C" __attribute__((visibility("default"))) int b200_torchabi_copy_selftest(void) {
    using dipu::B200CopyInplace;
    using A = B200CopyInplace::Action;
    try {
        if (dipu::getDipuCopyInstance() == nullptr) return 1;  // registered at load time
        const c10::Device d0(c10::DeviceType::PrivateUse1, 0), d1(c10::DeviceType::PrivateUse1, 1), cpu(c10::DeviceType::CPU);
        at::Tensor a = metadata_tensor(d0, at::kBFloat16, {4, 8}, {8, 1});
        at::Tensor b = metadata_tensor(d0, at::kBFloat16, {4, 8}, {8, 1});
        at::Tensor b_t = metadata_tensor(d0, at::kBFloat16, {4, 8}, {1, 4});
        at::Tensor b_f32 = metadata_tensor(d0, at::kFloat, {4, 8}, {8, 1});
        at::Tensor c = metadata_tensor(d1, at::kBFloat16, {4, 8}, {8, 1});
        at::Tensor c_t = metadata_tensor(d1, at::kBFloat16, {4, 8}, {1, 4});
        at::Tensor h = metadata_tensor(cpu, at::kBFloat16, {4, 8}, {8, 1});
        at::Tensor empty = metadata_tensor(d0, at::kBFloat16, {0, 8}, {8, 1});
        bool nb = false;
        // same device: one operator call, non-blocking whatever the caller asked; cast and transposed layouts included
        if (B200CopyInplace::plan(a, b, &nb) != A::DiopiCopy || !nb) return 2;
        nb = false;
        if (B200CopyInplace::plan(a, b_t, &nb) != A::DiopiCopy || B200CopyInplace::plan(a, b_f32, &nb) != A::DiopiCopy) return 3;
        // nothing to do: empty destination, the same tensor, an alias of the same elements
        if (B200CopyInplace::plan(empty, empty, &nb) != A::Nothing || B200CopyInplace::plan(a, a, &nb) != A::Nothing) return 4;
        c10::Storage shared = a.storage();
        at::Tensor alias = metadata_tensor(d0, at::kBFloat16, {4, 8}, {8, 1}, 0, &shared);
        if (B200CopyInplace::plan(a, alias, &nb) != A::Nothing) return 5;
        at::Tensor alias_t = metadata_tensor(d0, at::kBFloat16, {4, 8}, {1, 4}, 0, &shared);  // same memory, other layout: a real copy
        if (B200CopyInplace::plan(a, alias_t, &nb) != A::DiopiCopy) return 6;
        // other device: copy engines for dense same-layout bytes, relay through a dense tensor otherwise; blocking stays as asked
        nb = false;
        if (B200CopyInplace::plan(c, a, &nb) != A::PeerEngineCopy || nb) return 7;
        if (B200CopyInplace::plan(c_t, a, &nb) != A::PeerRelayThenEngineCopy || B200CopyInplace::plan(c, b_f32, &nb) != A::PeerRelayThenEngineCopy) return 8;
        // host on either side
        if (B200CopyInplace::plan(a, h, &nb) != A::HostRelay || B200CopyInplace::plan(h, a, &nb) != A::HostRelay || nb) return 9;
        // through the registered instance: decisions are counted
        dipu::DIPUCopyBase* inst = dipu::getDipuCopyInstance();
#if !B200_IN_DIPU_TREE
        const B200CopyInplace* mine = dynamic_cast<const B200CopyInplace*>(inst);
        if (mine == nullptr) return 10;
        const B200CopyInplace::Counters before = mine->counters();
        inst->run(a, b, false);
        inst->run(a, a, false);
        inst->run(c, a, true);
        inst->run(h, a, false);
        const B200CopyInplace::Counters after = mine->counters();
        if (after.diopi != before.diopi + 1 || after.nothing != before.nothing + 1 || after.peer_engine != before.peer_engine + 1 ||
            after.host != before.host + 1 || after.forced_non_blocking != before.forced_non_blocking + 1) return 11;
#else
        (void)inst;
#endif
        bool threw = false;
        try {
            at::Tensor undefined;
            B200CopyInplace::plan(undefined, a, &nb);
        } catch (const c10::Error&) {
            threw = true;
        }
        if (!threw) return 12;
        return 0;
    } catch (...) {
        return 100;
    }
}
