/*
 * DIOPI runtime interface (types + host callbacks) as seen from the operator library.
 *
 * PROVISIONAL: the upstream DIOPI proto headers are not vendored in the reference tree
 * (dipu/third_party/DIOPI is an empty submodule), so this header is authored from the
 * reference's call sites.  Enum numeric values and struct padding follow the public DIOPI
 * proto as far as it is known and must be re-checked against the pinned upstream header
 * before linking into a real DIPU build ("signature unpinned").
 *
 * Evidence for each declaration (paths inside the reference project):
 *   - handles are opaque pointers; the host passes its own tensor object
 *       dipu/torch_dipu/csrc_dipu/diopirt/diopi_helper.cpp:9-34
 *   - diopiSize_t {data,len}            diopirt/diopirt_impl.cpp:36-48
 *   - diopiScalar_t {stype, fval|ival}  diopirt/diopi_helper.cpp:74-119
 *   - dtype enumerators                 diopirt/diopi_helper.cpp:121-216
 *   - diopiDevice_t                     diopirt/diopirt_impl.cpp:58-63
 *   - host callbacks                    diopirt/diopirt_impl.cpp:17-237
 */
#ifndef DIOPI_DIOPIRT_H_
#define DIOPI_DIOPIRT_H_

#include <stddef.h>
#include <stdint.h>
#ifndef __cplusplus
#include <stdbool.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define DIOPI_API __attribute__((visibility("default")))
#define DIOPI_RT_API __attribute__((visibility("default")))

typedef enum {
    diopiSuccess = 0,
    diopiErrorOccurred = 1,
    diopiNotInited = 2,
    diopiNoRegisteredStreamCreateFunction = 3,
    diopiNoRegisteredStreamDestoryFunction = 4,
    diopiNoRegisteredStreamSyncFunction = 5,
    diopiNoRegisteredDeviceMemoryMallocFunction = 6,
    diopiNoRegisteredDeviceMemoryFreeFunction = 7,
    diopiNoRegisteredDevice2DdeviceMemoryCopyFunction = 8,
    diopiNoRegisteredDevice2HostMemoryCopyFunction = 9,
    diopiNoRegisteredHost2DeviceMemoryCopyFunction = 10,
    diopiNoRegisteredGetLastErrorFunction = 11,
    diopi5DNotSupported = 12,
    diopiNoImplement = 13,
    diopiDtypeNotSupported = 1000,
    /* The host turns this code into a D2H / CPU aten / H2D round trip
     * (dipu/scripts/autogen_diopi_wrapper/autogen_diopi_wrapper.py:404-439).
     * This library never returns it: there is no CPU path behind it. */
    diopiForceFallbackToCPU = 1001,
} diopiError_t;

typedef enum {
    diopi_host = 0,
    diopi_device = 1,
} diopiDevice_t;

typedef enum {
    diopi_dtype_int8 = 0,
    diopi_dtype_uint8 = 1,
    diopi_dtype_int16 = 2,
    diopi_dtype_uint16 = 3,
    diopi_dtype_int32 = 4,
    diopi_dtype_uint32 = 5,
    diopi_dtype_int64 = 6,
    diopi_dtype_uint64 = 7,
    diopi_dtype_float16 = 8,
    diopi_dtype_float32 = 9,
    diopi_dtype_float64 = 10,
    diopi_dtype_bool = 11,
    diopi_dtype_bfloat16 = 12,
    diopi_dtype_tfloat32 = 13,
    diopi_dtype_complex32 = 14,
    diopi_dtype_complex64 = 15,
    diopi_dtype_complex128 = 16,
    diopi_dtype_unsupported = 255
} diopiDtype_t;

typedef enum {
    RoundModeNone = 0,
    RoundModeTrunc = 1,
    RoundModeFloor = 2,
    RoundModeEND = 3
} diopiRoundMode_t;

typedef struct diopiSize_t_ {
    const int64_t* data;
    int64_t len;
} diopiSize_t;

typedef struct diopiScalar_t_ {
    diopiDtype_t stype; /* only diopi_dtype_int64 / diopi_dtype_float64 are produced by DIPU */
    union {
        double fval;
        int64_t ival;
    };
} diopiScalar_t;

typedef int32_t diopiDeviceIndex_t;

struct diopiContext;   /* defined by the host, opaque here */
struct diopiTensor;    /* defined by the host, opaque here */
struct diopiGenerator; /* defined by the host, opaque here */

typedef struct diopiContext* diopiContextHandle_t;
typedef struct diopiTensor* diopiTensorHandle_t;
typedef const struct diopiTensor* diopiConstTensorHandle_t;
typedef struct diopiGenerator* diopiGeneratorHandle_t;
typedef void* diopiStreamHandle_t;

/* ---- callbacks the HOST exports and the operator library imports ---------------------- */
extern DIOPI_RT_API const char* diopiGetVersion(void);

extern DIOPI_RT_API diopiError_t diopiGetTensorData(diopiTensorHandle_t th, void** pptr);
extern DIOPI_RT_API diopiError_t diopiGetTensorDataConst(diopiConstTensorHandle_t th, const void** pptr);
extern DIOPI_RT_API diopiError_t diopiGetTensorShape(diopiConstTensorHandle_t th, diopiSize_t* size);
extern DIOPI_RT_API diopiError_t diopiGetTensorStride(diopiConstTensorHandle_t th, diopiSize_t* stride);
extern DIOPI_RT_API diopiError_t diopiGetTensorDtype(diopiConstTensorHandle_t th, diopiDtype_t* dtype);
extern DIOPI_RT_API diopiError_t diopiGetTensorDevice(diopiConstTensorHandle_t th, diopiDevice_t* device);
extern DIOPI_RT_API diopiError_t diopiGetTensorNumel(diopiConstTensorHandle_t th, int64_t* numel);
extern DIOPI_RT_API diopiError_t diopiGetTensorElemSize(diopiConstTensorHandle_t th, int64_t* itemsize);
extern DIOPI_RT_API diopiError_t diopiGetTensorStoragePtr(diopiConstTensorHandle_t th, void** pStoragePtr);
extern DIOPI_RT_API diopiError_t diopiGetTensorStorageOffset(diopiConstTensorHandle_t th, int64_t* pOffset);
extern DIOPI_RT_API diopiError_t diopiGetTensorStorageNbytes(diopiConstTensorHandle_t th, size_t* pNbytes);
extern DIOPI_RT_API diopiError_t diopiGetTensorDeviceIndex(diopiConstTensorHandle_t th, diopiDeviceIndex_t* pDevIndex);
extern DIOPI_RT_API diopiError_t diopiGetCurrentDeviceIndex(diopiDeviceIndex_t* pDevIndex);

extern DIOPI_RT_API diopiError_t diopiGetStream(diopiContextHandle_t ctx, diopiStreamHandle_t* stream);

/* Workspace tensors: owned by the context, released when the host's wrapper returns. */
extern DIOPI_RT_API diopiError_t diopiRequireTensor(diopiContextHandle_t ctx, diopiTensorHandle_t* tensor, const diopiSize_t* size,
                                                    const diopiSize_t* stride /* may be NULL */, const diopiDtype_t dtype,
                                                    const diopiDevice_t device);
extern DIOPI_RT_API diopiError_t diopiRequireBuffer(diopiContextHandle_t ctx, diopiTensorHandle_t* tensor, int64_t num_bytes,
                                                    diopiDevice_t device);
/* RNG state of the host's generator (diopirt_impl.cpp:175-222): seed and Philox offset; an op that consumes random numbers
 * reads them and stores the advanced offset back. */
extern DIOPI_RT_API diopiError_t diopiGeneratorGetSeedAndOffset(diopiGeneratorHandle_t th, uint64_t* seed, uint64_t* offset);
extern DIOPI_RT_API diopiError_t diopiGeneratorSetSeedAndOffset(diopiGeneratorHandle_t th, uint64_t seed, uint64_t offset);

/* ---- exported by the operator library --------------------------------------------------- */
extern DIOPI_API const char* diopiGetVendorName(void);
extern DIOPI_API const char* diopiGetImplVersion(void);
/* The host prints this string when a call returns anything but diopiSuccess
 * (dipu/scripts/autogen_diopi_wrapper/autogen_diopi_wrapper.py:1001-1003). Thread-local. */
extern DIOPI_API const char* diopiGetLastErrorString(void);

#ifdef __cplusplus
}
#endif
#endif /* DIOPI_DIOPIRT_H_ */
