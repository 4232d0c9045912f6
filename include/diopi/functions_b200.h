/*
 * Entry points of libdiopi_impl.so that are additions of this implementation, not part of DIOPI.
 */
#ifndef DIOPI_FUNCTIONS_B200_H_
#define DIOPI_FUNCTIONS_B200_H_

#include "diopi/diopirt.h"

#ifdef __cplusplus
extern "C" {
#endif

/* No counterpart in the reference. Health word of the tensor-core kernels on the current device: 0 while no bounded
 * device-side wait has ever timed out, 1 afterwards, -1 if it cannot be read. Synchronises the device. */
DIOPI_API int diopiB200GemmStatus(void);

#ifdef __cplusplus
}
#endif
#endif /* DIOPI_FUNCTIONS_B200_H_ */
