// pccl* spelling of the PCIe path (see include/pccl/pccl.h).
#include <cstring>

#include "api/comm.h"
#include "hylink/hylink_ext.h"
#include "pccl/config.h"
#include "pccl/pccl.h"
#include "pcie/pcie_path.h"

using namespace hl;

namespace hl {
hlResult_t commInit(hlComm_t* out, int nranks, hlUniqueId id, int rank, int device, unsigned flags);
}

static pcclResult_t toPccl(hlResult_t r) {
  switch (r) {
    case hlSuccess: return pcclSuccess;
    case hlInvalidArgument: return pcclInvalidArgument;
    case hlSystemError: return pcclSystemError;
    case hlDeviceError: return pcclDeviceError;
    case hlNetworkError: case hlRemoteError: return pcclNetworkError;
    case hlTimeout: return pcclTimeout;
    case hlUnsupported: return pcclInvalidArgument;
    default: return pcclInternalError;
  }
}
static bool mapOp(pcclReduceOp_t op, hlRedOp_t* out) {
  switch (op) {
    case pcclReduceSum: *out = hlSum; return true;
    case pcclReduceMax: *out = hlMax; return true;
    case pcclReduceMin: *out = hlMin; return true;
    default: return false;
  }
}
static bool mapType(pcclDataType_t t, hlDataType_t* out) {
  if ((int)t < 0 || (int)t >= hlNumTypes) return false;
  *out = (hlDataType_t)t;
  return true;
}

#define PCCL_PRE(comm)                                                         \
  if (!(comm) || !(comm)->pcie) return toPccl(fail(hlInvalidArgument, "communicator has no PCIe path")); \
  std::lock_guard<std::mutex> _lk((comm)->mu)

extern "C" {

int pcclSetConfig(const pcclConfig_t* c) {
  if (!c) return 1;
  if (c->bootstrap_addr) return (int)toPccl(fail(hlUnsupported, "multi-node bootstrap is not supported (single node only)"));
  char buf[64];
  if (c->host_buffer_size) {
    snprintf(buf, sizeof(buf), "%zu", c->host_buffer_size);
    setenv("HYLINK_HOST_BUFFER_SIZE", buf, 1);
  }
  if (c->gpu_numa_map) setenv("HYLINK_GPU_NUMA_MAP", c->gpu_numa_map, 1);
  if (c->ir_path) setenv("HYLINK_IR_PATH", c->ir_path, 1);
  Config::reload();
  return 0;
}

pcclResult_t pcclGetUniqueId(pcclUniqueId* id) { return toPccl(hlGetUniqueId(reinterpret_cast<hlUniqueId*>(id))); }
pcclResult_t pcclFinalize(void) { return toPccl(hlFinalize()); }
pcclResult_t pcclCommInitRank(pcclComm_t* comm, int nranks, pcclUniqueId id, int rank) {
  hlUniqueId u;
  memcpy(&u, &id, sizeof(u));
  return toPccl(commInit(comm, nranks, u, rank, -1, /*pcie only*/ 1u | 4u));
}
pcclResult_t pcclCommDestroy(pcclComm_t comm) { return toPccl(hlCommDestroy(comm)); }
pcclResult_t pcclCommRank(pcclComm_t comm, int* rank) { return toPccl(hlCommRank(comm, rank)); }
pcclResult_t pcclCommSize(pcclComm_t comm, int* size) { return toPccl(hlCommSize(comm, size)); }
const char* pcclGetErrorString(pcclResult_t r) {
  switch (r) {
    case pcclSuccess: return "success";
    case pcclInvalidArgument: return "invalid argument";
    case pcclSystemError: return "system error";
    case pcclInternalError: return "internal error";
    case pcclDeviceError: return "device error";
    case pcclNetworkError: return "network error";
    case pcclTimeout: return "timeout";
    default: return "unknown error";
  }
}

pcclResult_t pcclAllReduceTyped(const void* s, void* r, size_t count, pcclDataType_t dt, pcclReduceOp_t op, pcclComm_t comm, pcclStream_t st) {
  hlDataType_t t;
  hlRedOp_t o;
  if (!mapType(dt, &t) || !mapOp(op, &o)) return pcclInvalidArgument;
  PCCL_PRE(comm);
  return toPccl(comm->pcie->allReduce(s, r, count, t, o, 1.0f, st));
}
pcclResult_t pcclAllGatherStridedTyped(const void* s, void* r, size_t count, size_t stride, pcclDataType_t dt, pcclComm_t comm, pcclStream_t st) {
  hlDataType_t t;
  if (!mapType(dt, &t)) return pcclInvalidArgument;
  PCCL_PRE(comm);
  return toPccl(comm->pcie->allGather(s, r, count, stride, t, st));
}
pcclResult_t pcclReduceScatterStridedTyped(const void* s, void* r, size_t count, size_t stride, pcclDataType_t dt, pcclReduceOp_t op, pcclComm_t comm, pcclStream_t st) {
  hlDataType_t t;
  hlRedOp_t o;
  if (!mapType(dt, &t) || !mapOp(op, &o)) return pcclInvalidArgument;
  PCCL_PRE(comm);
  if (count % (size_t)comm->nranks) return toPccl(fail(hlInvalidArgument, "reduce-scatter count %zu is not a multiple of %d ranks", count, comm->nranks));
  return toPccl(comm->pcie->reduceScatter(s, r, count / (size_t)comm->nranks, stride, t, o, 1.0f, st));
}
pcclResult_t pcclAllToAllStridedTyped(const void* s, void* r, size_t count, size_t stride, pcclDataType_t dt, pcclComm_t comm, pcclStream_t st) {
  hlDataType_t t;
  if (!mapType(dt, &t)) return pcclInvalidArgument;
  PCCL_PRE(comm);
  if (count % (size_t)comm->nranks) return toPccl(fail(hlInvalidArgument, "all-to-all count %zu is not a multiple of %d ranks", count, comm->nranks));
  return toPccl(comm->pcie->allToAll(s, r, count / (size_t)comm->nranks, stride, t, st));
}
pcclResult_t pcclBroadcastRootTyped(const void* s, void* r, size_t count, pcclDataType_t dt, int root, pcclComm_t comm, pcclStream_t st) {
  hlDataType_t t;
  if (!mapType(dt, &t)) return pcclInvalidArgument;
  PCCL_PRE(comm);
  if (root < 0 || root >= comm->nranks) return pcclInvalidArgument;
  return toPccl(comm->pcie->broadcast(s, r, count, t, root, st));
}

pcclResult_t pcclAllGatherTyped(const void* s, void* r, size_t n, pcclDataType_t dt, pcclComm_t c, pcclStream_t st) { return pcclAllGatherStridedTyped(s, r, n, 0, dt, c, st); }
pcclResult_t pcclReduceScatterTyped(const void* s, void* r, size_t recvcount, pcclDataType_t dt, pcclReduceOp_t op, pcclComm_t c, pcclStream_t st) {
  if (!c) return pcclInvalidArgument;
  return pcclReduceScatterStridedTyped(s, r, recvcount * (size_t)c->nranks, 0, dt, op, c, st);
}
pcclResult_t pcclAllToAllTyped(const void* s, void* r, size_t count, pcclDataType_t dt, pcclComm_t c, pcclStream_t st) {
  if (!c) return pcclInvalidArgument;
  return pcclAllToAllStridedTyped(s, r, count * (size_t)c->nranks, 0, dt, c, st);
}

pcclResult_t pcclAllReduce(const void* s, void* r, size_t n, pcclComm_t c, pcclStream_t st) { return pcclAllReduceTyped(s, r, n, pcclFloat32, pcclReduceSum, c, st); }
pcclResult_t pcclAllGather(const void* s, void* r, size_t n, pcclComm_t c, pcclStream_t st) { return pcclAllGatherTyped(s, r, n, pcclFloat32, c, st); }
pcclResult_t pcclReduceScatter(const void* s, void* r, size_t n, pcclComm_t c, pcclStream_t st) { return pcclReduceScatterTyped(s, r, n, pcclFloat32, pcclReduceSum, c, st); }
pcclResult_t pcclAllToAll(const void* s, void* r, size_t n, pcclComm_t c, pcclStream_t st) { return pcclAllToAllTyped(s, r, n, pcclFloat32, c, st); }
pcclResult_t pcclBroadcastRoot(const void* s, void* r, size_t n, int root, pcclComm_t c, pcclStream_t st) { return pcclBroadcastRootTyped(s, r, n, pcclFloat32, root, c, st); }
pcclResult_t pcclAllGatherStrided(const void* s, void* r, size_t n, size_t stride, pcclComm_t c, pcclStream_t st) { return pcclAllGatherStridedTyped(s, r, n, stride, pcclFloat32, c, st); }
pcclResult_t pcclReduceScatterStrided(const void* s, void* r, size_t n, size_t stride, pcclComm_t c, pcclStream_t st) { return pcclReduceScatterStridedTyped(s, r, n, stride, pcclFloat32, pcclReduceSum, c, st); }
pcclResult_t pcclAllToAllStrided(const void* s, void* r, size_t n, size_t stride, pcclComm_t c, pcclStream_t st) { return pcclAllToAllStridedTyped(s, r, n, stride, pcclFloat32, c, st); }

pcclResult_t pcclSubmitIR(pcclComm_t comm, const char* xml, const void* s, void* r, size_t seg_count, size_t stride, int send_segs,
                          int recv_segs, pcclDataType_t dt, pcclReduceOp_t op, pcclStream_t st) {
  hlDataType_t t;
  hlRedOp_t o;
  if (!mapType(dt, &t) || !mapOp(op, &o)) return pcclInvalidArgument;
  return toPccl(hlSubmitIr(comm, xml, s, r, seg_count, stride, send_segs, recv_segs, t, o, st));
}

}  // extern "C"
