/*
 * PCCL-compatible C API: the host-staged (PCIe) collective path on its own.
 *
 * Function names, argument order and count semantics follow the reference's
 * two headers — the CUDA library's untyped set
 * (pcie-ccl-cuda/include/pccl/pccl.h:14-131) and the Ascend port's typed set
 * (pcie-ccl-ascend/include/pccl/pccl.h:13-135) — so code written for either
 * links here. Untyped calls mean fp32 / sum.
 *
 * Strided variants: the first `stride` elements of every per-rank segment are
 * left to another transport (the NVLink kernels); this library moves elements
 * [stride, segment_length) of each segment.
 *   pcclAllGatherStrided:      count = elements per segment (the send count)
 *   pcclReduceScatterStrided:  count = total elements (receive count * nranks)
 *   pcclAllToAllStrided:       count = total elements (per-peer count * nranks)
 */
#ifndef PCCL_H
#define PCCL_H

#include <stddef.h>

#include "types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  pcclInvalidDataType = -1,
  pcclInt8 = 0, pcclUint8 = 1, pcclInt32 = 2, pcclUint32 = 3, pcclInt64 = 4, pcclUint64 = 5,
  pcclFloat16 = 6, pcclFloat32 = 7, pcclFloat64 = 8, pcclBfloat16 = 9
} pcclDataType_t;

typedef enum { pcclInvalidReduceOp = -1, pcclReduceSum = 0, pcclReduceMax = 1, pcclReduceMin = 2 } pcclReduceOp_t;

pcclResult_t pcclGetUniqueId(pcclUniqueId* uniqueId);
pcclResult_t pcclFinalize(void);
/* A zeroed id selects single-process mode (one thread per rank). */
pcclResult_t pcclCommInitRank(pcclComm_t* comm, int nranks, pcclUniqueId uniqueId, int rank);
pcclResult_t pcclCommDestroy(pcclComm_t comm);
pcclResult_t pcclCommRank(pcclComm_t comm, int* rank);
pcclResult_t pcclCommSize(pcclComm_t comm, int* size);
const char* pcclGetErrorString(pcclResult_t result);

pcclResult_t pcclAllReduce(const void* sendbuff, void* recvbuff, size_t count, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclAllToAll(const void* sendbuff, void* recvbuff, size_t count, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclBroadcastRoot(const void* sendbuff, void* recvbuff, size_t count, int root, pcclComm_t comm, pcclStream_t stream);

pcclResult_t pcclAllGatherStrided(const void* sendbuff, void* recvbuff, size_t count, size_t stride, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclReduceScatterStrided(const void* sendbuff, void* recvbuff, size_t count, size_t stride, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclAllToAllStrided(const void* sendbuff, void* recvbuff, size_t count, size_t stride, pcclComm_t comm, pcclStream_t stream);

pcclResult_t pcclAllReduceTyped(const void* sendbuff, void* recvbuff, size_t count, pcclDataType_t datatype, pcclReduceOp_t op, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclAllGatherTyped(const void* sendbuff, void* recvbuff, size_t sendcount, pcclDataType_t datatype, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclReduceScatterTyped(const void* sendbuff, void* recvbuff, size_t recvcount, pcclDataType_t datatype, pcclReduceOp_t op, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclAllToAllTyped(const void* sendbuff, void* recvbuff, size_t count, pcclDataType_t datatype, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclBroadcastRootTyped(const void* sendbuff, void* recvbuff, size_t count, pcclDataType_t datatype, int root, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclAllGatherStridedTyped(const void* sendbuff, void* recvbuff, size_t count, size_t stride, pcclDataType_t datatype, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclReduceScatterStridedTyped(const void* sendbuff, void* recvbuff, size_t count, size_t stride, pcclDataType_t datatype, pcclReduceOp_t op, pcclComm_t comm, pcclStream_t stream);
pcclResult_t pcclAllToAllStridedTyped(const void* sendbuff, void* recvbuff, size_t count, size_t stride, pcclDataType_t datatype, pcclComm_t comm, pcclStream_t stream);

/* Runs a caller-supplied schedule (XML text) with the layout of a collective
 * that has `send_segs` / `recv_segs` segments of `seg_count` elements. */
pcclResult_t pcclSubmitIR(pcclComm_t comm, const char* ir_xml, const void* sendbuff, void* recvbuff, size_t seg_count,
                          size_t stride, int send_segs, int recv_segs, pcclDataType_t datatype, pcclReduceOp_t op,
                          pcclStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PCCL_H */
