// dipu::devapis device / stream / event / memory functions of the B200 vendor: thin C++ forwarding onto the C-ABI runtime
// (include/dipu_b200/vendor_c_api.h). This is the file a DIPU tree compiles as csrc_dipu/vendor/b200/deviceimpl.cpp.
// Error behaviour follows the CUDA vendor (dipu/torch_dipu/csrc_dipu/vendor/cuda/deviceimpl.cpp:18-241): void functions throw,
// mallocDevice(…, false) reports ERR_NOMEM, getEventStatus maps "not ready" to PENDING.
#include "devapis_decl.h"

namespace dipu {
namespace devapis {

void initializeVendor() { DIPU_CALLB200(b200_initialize_vendor()) }
void finalizeVendor() { DIPU_CALLB200(b200_finalize_vendor()) }

deviceId_t current_device() {
    int d = -1;
    DIPU_CALLB200(b200_current_device(&d))
    return static_cast<deviceId_t>(d);
}

DIPUDeviceProperties getDeviceProperties(int32_t device_index) {
    b200DeviceProperties p;
    DIPU_CALLB200(b200_get_device_properties(device_index, &p))
    DIPUDeviceProperties out;
    out.name = p.name;
    out.totalGlobalMem = p.total_global_mem;
    out.major = p.major;
    out.minor = p.minor;
    out.multiProcessorCount = p.multi_processor_count;
    return out;
}

DIPUDeviceStatus getDeviceStatus(int32_t device_index) {
    DIPUDeviceStatus st;
    DIPU_CALLB200(b200_get_device_status(device_index, &st.freeGlobalMem, &st.totalGlobalMem))
    return st;
}

void setDevice(deviceId_t devId) { DIPU_CALLB200(b200_set_device(devId)) }
void resetDevice(deviceId_t devId) { DIPU_CALLB200(b200_reset_device(devId)) }
void syncDevice() { DIPU_CALLB200(b200_sync_device()) }
void checkLastError() { DIPU_CALLB200(b200_check_last_error()) }

int getDeviceCount() {
    int n = 0;
    DIPU_CALLB200(b200_get_device_count(&n))
    return n;
}
void getDriverVersion(int* version) { DIPU_CALLB200(b200_get_driver_version(version)) }
void getRuntimeVersion(int* version) { DIPU_CALLB200(b200_get_runtime_version(version)) }

void createStream(deviceStream_t* stream, bool prior) {
    b200Stream_t s = nullptr;
    DIPU_CALLB200(b200_create_stream(&s, prior ? 1 : 0))
    *stream = static_cast<deviceStream_t>(s);
}
void destroyStream(deviceStream_t stream) { DIPU_CALLB200(b200_destroy_stream(stream)) }
void destroyStream(deviceStream_t stream, deviceId_t devId) { DIPU_CALLB200(b200_destroy_stream_on(stream, devId)) }
void releaseStream() { DIPU_CALLB200(b200_release_stream()) }
void syncStream(deviceStream_t stream) { DIPU_CALLB200(b200_sync_stream(stream)) }
bool streamNotNull(deviceStream_t stream) { return b200_stream_not_null(stream) != 0; }
void streamWaitEvent(deviceStream_t stream, deviceEvent_t event) { DIPU_CALLB200(b200_stream_wait_event(stream, event)) }
bool isStreamEmpty(deviceStream_t stream) { return b200_is_stream_empty(stream) != 0; }

void createEvent(deviceEvent_t* event) {
    b200Event_t e = nullptr;
    DIPU_CALLB200(b200_create_event(&e))
    *event = static_cast<deviceEvent_t>(e);
}
void destroyEvent(deviceEvent_t event) { DIPU_CALLB200(b200_destroy_event(event)) }
void waitEvent(deviceEvent_t event) { DIPU_CALLB200(b200_wait_event(event)) }
void recordEvent(deviceEvent_t event, deviceStream_t stream) { DIPU_CALLB200(b200_record_event(event, stream)) }
void eventElapsedTime(float* time, deviceEvent_t start, deviceEvent_t end) { DIPU_CALLB200(b200_event_elapsed_time(time, start, end)) }

EventStatus getEventStatus(deviceEvent_t event) {
    b200EventStatus_t st = B200_EVENT_READY;
    DIPU_CALLB200(b200_get_event_status(event, &st))
    return st == B200_EVENT_READY ? EventStatus::READY : EventStatus::PENDING;
}

void mallocHost(void** p, size_t nbytes) { DIPU_CALLB200(b200_malloc_host(p, nbytes)) }
void freeHost(void* p) { DIPU_CALLB200(b200_free_host(p)) }

OpStatus mallocDevice(void** p, size_t nbytes, bool throwExcepion) {
    const b200Status_t st = b200_malloc_device(p, nbytes);
    if (st == B200_SUCCESS) return OpStatus::SUCCESS;
    if (st == B200_ERR_NOMEM && !throwExcepion) return OpStatus::ERR_NOMEM;
    TORCH_CHECK(false, "mallocDevice failed, size = ", nbytes, ": ", b200_last_error());
}
void freeDevice(void* p) { DIPU_CALLB200(b200_free_device(p)) }
bool isPinnedPtr(const void* p) { return b200_is_pinned_ptr(p) != 0; }
void memSetAsync(deviceStream_t stream, void* ptr, int val, size_t size) { DIPU_CALLB200(b200_memset_async(stream, ptr, val, size)) }

void memCopyD2D(size_t nbytes, deviceId_t dstDevId, void* dst, deviceId_t srcDevId, const void* src) {
    DIPU_CALLB200(b200_memcpy_d2d(nbytes, dstDevId, dst, srcDevId, src))
}
void memCopyH2D(size_t nbytes, void* dst, const void* src) { DIPU_CALLB200(b200_memcpy_h2d(nbytes, dst, src)) }
void memCopyD2H(size_t nbytes, void* dst, const void* src) { DIPU_CALLB200(b200_memcpy_d2h(nbytes, dst, src)) }
void memCopyD2DAsync(deviceStream_t stream, size_t nbytes, deviceId_t dstDevId, void* dst, deviceId_t srcDevId, const void* src) {
    DIPU_CALLB200(b200_memcpy_d2d_async(stream, nbytes, dstDevId, dst, srcDevId, src))
}
void memCopyH2DAsync(deviceStream_t stream, size_t nbytes, void* dst, const void* src) {
    DIPU_CALLB200(b200_memcpy_h2d_async(stream, nbytes, dst, src))
}
void memCopyD2HAsync(deviceStream_t stream, size_t nbytes, void* dst, const void* src) {
    DIPU_CALLB200(b200_memcpy_d2h_async(stream, nbytes, dst, src))
}

}  // namespace devapis
}  // namespace dipu
