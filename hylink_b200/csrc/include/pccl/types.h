/* PCCL-compatible basic types (result codes, communicator and stream handles,
 * the 128-byte unique id). Binary compatible with the reference's
 * pcie-ccl-cuda/include/pccl/types.h:8-22 so that programs written against
 * that library link against this one unchanged. */
#ifndef PCCL_TYPES_H
#define PCCL_TYPES_H

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  pcclSuccess = 0,
  pcclInvalidArgument = 1,
  pcclSystemError = 2,
  pcclInternalError = 3,
  pcclDeviceError = 4,
  pcclNetworkError = 5,
  pcclTimeout = 6
} pcclResult_t;

typedef struct hlComm* pcclComm_t; /* opaque */
typedef void* pcclStream_t;        /* cudaStream_t */

#define PCCL_UNIQUE_ID_BYTES 128
typedef struct { char internal[PCCL_UNIQUE_ID_BYTES]; } pcclUniqueId;

#ifdef __cplusplus
}
#endif
#endif /* PCCL_TYPES_H */
