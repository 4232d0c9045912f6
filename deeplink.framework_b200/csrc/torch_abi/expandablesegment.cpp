// vendorCreateExpandableSegment for the B200 vendor: the symbol DIPU's caching allocator null-tests before it enables
// expandable_segments:True (reference dipu/torch_dipu/csrc_dipu/runtime/core/allocator/ExpandableSegment.h:105-136 declares
// the interface and the weak factory; DIPUCachingDeviceAllocator.cpp:481-486 is the null test). In a DIPU build the
// abstract class comes from DIPU's header; it is restated here so that this file compiles without the DIPU tree.
#include <cstddef>
#include <vector>

#include "vendorapi.h"

#if __has_include(<csrc_dipu/runtime/core/allocator/ExpandableSegment.h>)
#include <csrc_dipu/runtime/core/allocator/ExpandableSegment.h>
namespace dipu {
#else
namespace dipu {

struct SegmentRange {
    char* ptr;
    size_t size;
    SegmentRange(void* p, size_t s) : ptr(static_cast<char*>(p)), size(s) {}
};

class ExpandableSegment {
  public:
    virtual ~ExpandableSegment() = default;
    virtual SegmentRange map(SegmentRange range) = 0;
    virtual SegmentRange unmap(SegmentRange range) = 0;
    virtual void addPeer(int) = 0;
    virtual char* ptr() const = 0;
    virtual size_t size() const = 0;
};
#endif

namespace {

class B200ExpandableSegment final : public ExpandableSegment {
  public:
    B200ExpandableSegment(int device, deviceStream_t stream, size_t page_size, const std::vector<int>& peers) {
        DIPU_CALLB200(b200_expandable_create(&seg_, device, stream, page_size, peers.empty() ? nullptr : peers.data(), static_cast<int>(peers.size())));
    }
    ~B200ExpandableSegment() override { (void)b200_expandable_destroy(seg_); }
    SegmentRange map(SegmentRange range) override {
        void* p = nullptr;
        size_t n = 0;
        DIPU_CALLB200(b200_expandable_map(seg_, range.ptr, range.size, &p, &n));
        return SegmentRange(n == 0 ? range.ptr : p, n);  // size 0: the device is out of memory, nothing was mapped
    }
    SegmentRange unmap(SegmentRange range) override {
        void* p = nullptr;
        size_t n = 0;
        DIPU_CALLB200(b200_expandable_unmap(seg_, range.ptr, range.size, &p, &n));
        return SegmentRange(n == 0 ? range.ptr : p, n);
    }
    void addPeer(int device) override { DIPU_CALLB200(b200_expandable_add_peer(seg_, device)); }
    char* ptr() const override { return static_cast<char*>(b200_expandable_ptr(seg_)); }
    size_t size() const override { return b200_expandable_size(seg_); }

  private:
    void* seg_ = nullptr;
};

}  // namespace

__attribute__((visibility("default"))) ExpandableSegment* vendorCreateExpandableSegment(int device, deviceStream_t stream, size_t size,
                                                                                       std::vector<int> peers) {
    return new B200ExpandableSegment(device, stream, size, peers);
}

}  // namespace dipu
