// Declarations of the vendor contract exactly as DIPU's runtime expects to link them (namespace dipu::devapis, C++ linkage,
// default visibility). In a DIPU build these come from DIPU's own headers
// (dipu/torch_dipu/csrc_dipu/runtime/device/basedef.h:35-90, deviceapis.h:21-125, diclapis.h:13-84); this file restates the
// signatures so that the wrappers in this directory can be compiled and checked without the DIPU tree.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

#include <c10/core/Device.h>
#include <c10/core/ScalarType.h>
#include <torch/csrc/distributed/c10d/Types.hpp>

#include "vendorapi.h"

#define B200_DIPU_API __attribute__((visibility("default")))

namespace dipu {
namespace devapis {

using enum_t = int32_t;
enum class VendorDeviceType : enum_t { CUDA, MLU, NPU, MUXI, GCU, DROPLET, SUPA, KLX };
enum class EventStatus : enum_t { PENDING, RUNNING, DEFERRED, READY };
enum class OpStatus : enum_t { SUCCESS, ERR_UNKNOWN, ERR_NOMEM };
enum diclResult_t { DICL_SUCCESS = 0x0, DICL_ERR_UNDEF = 0x01000 };

struct DIPUDeviceStatus {
    size_t freeGlobalMem = 0;
    size_t totalGlobalMem = 0;
};
struct DIPUDeviceProperties {
    std::string name;
    size_t totalGlobalMem = 0;
    int32_t major = 0;
    int32_t minor = 0;
    int32_t multiProcessorCount = 0;
};
using deviceId_t = c10::DeviceIndex;
using ReduceOp = c10d::ReduceOp;

B200_DIPU_API void initializeVendor();
B200_DIPU_API void finalizeVendor();
B200_DIPU_API deviceId_t current_device();
B200_DIPU_API DIPUDeviceProperties getDeviceProperties(int32_t device_index);
B200_DIPU_API DIPUDeviceStatus getDeviceStatus(int32_t device_index);
B200_DIPU_API void setDevice(deviceId_t devId);
B200_DIPU_API void resetDevice(deviceId_t devId = 0);
B200_DIPU_API void syncDevice();
B200_DIPU_API void checkLastError();
B200_DIPU_API int getDeviceCount();
B200_DIPU_API void getDriverVersion(int* version);
B200_DIPU_API void getRuntimeVersion(int* version);

B200_DIPU_API void createStream(deviceStream_t* stream, bool prior = false);
B200_DIPU_API void destroyStream(deviceStream_t stream);
B200_DIPU_API void destroyStream(deviceStream_t stream, deviceId_t devId);
B200_DIPU_API void releaseStream();
B200_DIPU_API void syncStream(deviceStream_t stream);
B200_DIPU_API bool streamNotNull(deviceStream_t stream);
B200_DIPU_API void streamWaitEvent(deviceStream_t stream, deviceEvent_t event);
B200_DIPU_API bool isStreamEmpty(deviceStream_t stream);

B200_DIPU_API void createEvent(deviceEvent_t* event);
B200_DIPU_API void destroyEvent(deviceEvent_t event);
B200_DIPU_API void waitEvent(deviceEvent_t event);
B200_DIPU_API void recordEvent(deviceEvent_t event, deviceStream_t stream);
B200_DIPU_API void eventElapsedTime(float* time, deviceEvent_t start, deviceEvent_t end);
B200_DIPU_API EventStatus getEventStatus(deviceEvent_t event);

B200_DIPU_API void mallocHost(void** p, size_t nbytes);
B200_DIPU_API void freeHost(void* p);
B200_DIPU_API OpStatus mallocDevice(void** p, size_t nbytes, bool throwExcepion = true);
B200_DIPU_API void freeDevice(void* p);
B200_DIPU_API bool isPinnedPtr(const void* p);
B200_DIPU_API void memSetAsync(deviceStream_t stream, void* ptr, int val, size_t size);
B200_DIPU_API void memCopyD2D(size_t nbytes, deviceId_t dstDevId, void* dst, deviceId_t srcDevId, const void* src);
B200_DIPU_API void memCopyH2D(size_t nbytes, void* dst, const void* src);
B200_DIPU_API void memCopyD2H(size_t nbytes, void* dst, const void* src);
B200_DIPU_API void memCopyD2DAsync(deviceStream_t stream, size_t nbytes, deviceId_t dstDevId, void* dst, deviceId_t srcDevId, const void* src);
B200_DIPU_API void memCopyH2DAsync(deviceStream_t stream, size_t nbytes, void* dst, const void* src);
B200_DIPU_API void memCopyD2HAsync(deviceStream_t stream, size_t nbytes, void* dst, const void* src);

extern B200_DIPU_API const int DICL_UNIQUE_ID_BYTES_SIZE;
B200_DIPU_API diclResult_t diclGetCommAsyncError(diclComm_t comm);
B200_DIPU_API diclResult_t diclGetUniqueId(commUniqueId* uniqueId);
B200_DIPU_API diclResult_t diclCommInitRank(diclComm_t* comm, int nranks, commUniqueId uniqueId, int rank, int localDeviceId = -1);
B200_DIPU_API diclResult_t diclCommDestroy(diclComm_t comm);
B200_DIPU_API diclResult_t diclAllReduce(const void* sendBuf, void* recvBuf, size_t count, at::ScalarType datatype, const ReduceOp& reduceOp,
                                         diclComm_t comm, deviceStream_t stream);
B200_DIPU_API diclResult_t diclBroadcast(const void* sendBuf, void* recvBuf, size_t count, at::ScalarType datatype, int root, diclComm_t comm,
                                         deviceStream_t stream);
B200_DIPU_API diclResult_t diclAllGather(const void* sendBuf, void* recvBuf, size_t sendCount, at::ScalarType datatype, diclComm_t comm,
                                         deviceStream_t stream);
B200_DIPU_API diclResult_t diclReduce(const void* sendbuf, void* recvBuf, size_t count, at::ScalarType datatype, const ReduceOp& reduceOp, int root,
                                      diclComm_t comm, deviceStream_t stream);
B200_DIPU_API diclResult_t diclReduceScatter(void* sendBuf, void* recvBuf, size_t recvCount, at::ScalarType datatype, const ReduceOp& op,
                                             diclComm_t comm, deviceStream_t stream);
B200_DIPU_API diclResult_t diclAllToAllEqualSplit(const void* sendBuf, void* recvBuf, size_t count, at::ScalarType dataType, diclComm_t comm,
                                                  deviceStream_t stream);
B200_DIPU_API diclResult_t diclAllToAllUnequalSplit(const void* sendBuf, const size_t* sendCounts, const size_t* sendDisplacements, void* recvBuf,
                                                    const size_t* recvCounts, const size_t* recvDisplacements, at::ScalarType dataType,
                                                    diclComm_t comm, deviceStream_t stream);
B200_DIPU_API diclResult_t diclSend(const void* sendBuf, size_t count, at::ScalarType datatype, int peer, diclComm_t comm, deviceStream_t stream);
B200_DIPU_API diclResult_t diclRecv(void* recvBuf, size_t count, at::ScalarType datatype, int peer, diclComm_t comm, deviceStream_t stream);
B200_DIPU_API diclResult_t diclGetCommName(std::string& commName, diclComm_t comm);

}  // namespace devapis
}  // namespace dipu
