// dipu::devapis::dicl* of the B200 vendor: forwarding onto the C-ABI communicator (NCCL over NVLink underneath).
// The file a DIPU tree compiles as csrc_dipu/vendor/b200/communicatorimpl.cpp; contract in
// dipu/torch_dipu/csrc_dipu/runtime/device/diclapis.h:20-82, call pattern in runtime/distributed/ProcessGroupDICL.cpp:438-567.
#include "devapis_decl.h"

#include "diopi/diopirt.h"

namespace dipu {
namespace devapis {

const int DICL_UNIQUE_ID_BYTES_SIZE = B200_UNIQUE_ID_BYTES;

namespace {

int to_dtype(at::ScalarType t) {
    switch (t) {
        case at::kChar: return diopi_dtype_int8;
        case at::kByte: return diopi_dtype_uint8;
        case at::kBool: return diopi_dtype_bool;  // reduced as uint8 with SUM mapped to MAX so that the result stays boolean
        case at::kInt: return diopi_dtype_int32;
        case at::kLong: return diopi_dtype_int64;
        case at::kHalf: return diopi_dtype_float16;
        case at::kFloat: return diopi_dtype_float32;
        case at::kDouble: return diopi_dtype_float64;
        case at::kBFloat16: return diopi_dtype_bfloat16;
        default: TORCH_CHECK(false, "dicl: scalar type ", t, " is not supported");
    }
}

int to_op(const ReduceOp& op) {
    switch (static_cast<uint8_t>(op)) {
        case ReduceOp::SUM: return B200_REDUCE_SUM;
        case ReduceOp::AVG: return B200_REDUCE_AVG;
        case ReduceOp::PRODUCT: return B200_REDUCE_PRODUCT;
        case ReduceOp::MIN: return B200_REDUCE_MIN;
        case ReduceOp::MAX: return B200_REDUCE_MAX;
        default: TORCH_CHECK(false, "dicl: reduce op ", static_cast<int>(static_cast<uint8_t>(op)), " is not supported");
    }
}

}  // namespace

diclResult_t diclGetCommAsyncError(diclComm_t comm) {
    return b200_dicl_get_comm_async_error(comm) == B200_SUCCESS ? DICL_SUCCESS : DICL_ERR_UNDEF;
}
diclResult_t diclGetUniqueId(commUniqueId* uniqueId) {
    DIPU_CALLB200(b200_dicl_get_unique_id(uniqueId))
    return DICL_SUCCESS;
}
diclResult_t diclCommInitRank(diclComm_t* comm, int nranks, commUniqueId uniqueId, int rank, int localDeviceId) {
    DIPU_CALLB200(b200_dicl_comm_init_rank(comm, nranks, &uniqueId, rank, localDeviceId))
    return DICL_SUCCESS;
}
diclResult_t diclCommDestroy(diclComm_t comm) {
    DIPU_CALLB200(b200_dicl_comm_destroy(comm))
    return DICL_SUCCESS;
}
diclResult_t diclAllReduce(const void* sendBuf, void* recvBuf, size_t count, at::ScalarType datatype, const ReduceOp& reduceOp, diclComm_t comm,
                           deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_all_reduce(sendBuf, recvBuf, count, to_dtype(datatype), to_op(reduceOp), comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclBroadcast(const void* sendBuf, void* recvBuf, size_t count, at::ScalarType datatype, int root, diclComm_t comm,
                           deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_broadcast(sendBuf, recvBuf, count, to_dtype(datatype), root, comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclAllGather(const void* sendBuf, void* recvBuf, size_t sendCount, at::ScalarType datatype, diclComm_t comm, deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_all_gather(sendBuf, recvBuf, sendCount, to_dtype(datatype), comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclReduce(const void* sendbuf, void* recvBuf, size_t count, at::ScalarType datatype, const ReduceOp& reduceOp, int root,
                        diclComm_t comm, deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_reduce(sendbuf, recvBuf, count, to_dtype(datatype), to_op(reduceOp), root, comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclReduceScatter(void* sendBuf, void* recvBuf, size_t recvCount, at::ScalarType datatype, const ReduceOp& op, diclComm_t comm,
                               deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_reduce_scatter(sendBuf, recvBuf, recvCount, to_dtype(datatype), to_op(op), comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclAllToAllEqualSplit(const void* sendBuf, void* recvBuf, size_t count, at::ScalarType dataType, diclComm_t comm,
                                    deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_all_to_all_equal_split(sendBuf, recvBuf, count, to_dtype(dataType), comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclAllToAllUnequalSplit(const void* sendBuf, const size_t* sendCounts, const size_t* sendDisplacements, void* recvBuf,
                                      const size_t* recvCounts, const size_t* recvDisplacements, at::ScalarType dataType, diclComm_t comm,
                                      deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_all_to_all_unequal_split(sendBuf, sendCounts, sendDisplacements, recvBuf, recvCounts, recvDisplacements,
                                                     to_dtype(dataType), comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclSend(const void* sendBuf, size_t count, at::ScalarType datatype, int peer, diclComm_t comm, deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_send(sendBuf, count, to_dtype(datatype), peer, comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclRecv(void* recvBuf, size_t count, at::ScalarType datatype, int peer, diclComm_t comm, deviceStream_t stream) {
    DIPU_CALLB200(b200_dicl_recv(recvBuf, count, to_dtype(datatype), peer, comm, stream))
    return DICL_SUCCESS;
}
diclResult_t diclGetCommName(std::string& commName, diclComm_t comm) {
    char buf[64];
    DIPU_CALLB200(b200_dicl_get_comm_name(buf, sizeof(buf), comm))
    commName = buf;
    return DICL_SUCCESS;
}

}  // namespace devapis
}  // namespace dipu
