/*
 * hylink-b200 public C API.
 *
 * One library carries both transports of a single-node multipath collective
 * stack for B200: the NVLink/NVSwitch path (hand-written sm_100a kernels over
 * peer-mapped symmetric memory) and the PCIe path (CPU-driven schedule IR,
 * copy engines, pinned host staging), plus the orchestrator that splits each
 * collective between them.
 *
 * Capability parity: the reference exposes this surface through three
 * libraries (pcie-ccl-cuda/include/pccl/pccl.h:14-131 for the PCIe CCL,
 * pcie-ccl-ascend/include/pccl/pccl.h:13-135 for the typed variants, and
 * multipath-orchestrator/libampccl/hook/nccl_hook.cc:293-648 for the
 * orchestrated NCCL symbols). The `pccl*` spelling of the same calls lives in
 * <pccl/pccl.h>; the `nccl*` spelling is exported by libhylink_nccl.so.
 */
#ifndef HYLINK_HYLINK_H_
#define HYLINK_HYLINK_H_

#include <stddef.h>
#include <sys/types.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  hlSuccess = 0,
  hlInvalidArgument = 1,
  hlSystemError = 2,
  hlInternalError = 3,
  hlDeviceError = 4,
  hlNetworkError = 5,
  hlTimeout = 6,
  hlUnsupported = 7,
  hlRemoteError = 8
} hlResult_t;

/* Numbering follows ncclDataType_t so the interception layer is a cast. */
typedef enum {
  hlInt8 = 0,
  hlUint8 = 1,
  hlInt32 = 2,
  hlUint32 = 3,
  hlInt64 = 4,
  hlUint64 = 5,
  hlFloat16 = 6,
  hlFloat32 = 7,
  hlFloat64 = 8,
  hlBfloat16 = 9,
  hlNumTypes = 10
} hlDataType_t;

/* Numbering follows ncclRedOp_t. */
typedef enum { hlSum = 0, hlProd = 1, hlMax = 2, hlMin = 3, hlAvg = 4, hlNumOps = 5 } hlRedOp_t;

/* Which transport(s) a call may use. */
typedef enum {
  hlPathAuto = 0,    /* orchestrator decides (split when it pays) */
  hlPathNvlink = 1,  /* dedicated-link kernels only */
  hlPathPcie = 2,    /* host-staged copy-engine path only */
  hlPathSplit = 3    /* always fork on both paths with the current ratio */
} hlPath_t;

/* Algorithm selector for the NVLink path. */
typedef enum {
  hlAlgoAuto = 0,
  hlAlgoOneShot = 1,     /* every rank reads all peers, one barrier pair */
  hlAlgoTwoShotP2p = 2,  /* pull-reduce of the owned shard, pull all-gather; fixed sum order */
  hlAlgoNvls = 3,        /* multimem.ld_reduce + multimem.st through NVSwitch */
  hlAlgoPipelined = 4,   /* warp-specialised tiles: copy-in, link exchange and copy-out overlap */
  hlAlgoPush = 5,        /* peer stores only: push shards to their owner, fold locally, push results */
  hlAlgoZeroCopy = 6,    /* registered (hlMemAlloc) buffers read and written in place on every rank; refused for others */
  hlAlgoZeroCopyNvls = 7,/* ... through NVSwitch (multimem) */
  hlAlgoZeroCopyP2p = 8, /* ... with plain peer loads and stores, fixed sum order */
  hlAlgoLowLatency = 9   /* small messages: every 16-byte store carries its arrival flag, no cross-GPU barrier; fixed sum order */
} hlAlgo_t;

#define HL_UNIQUE_ID_BYTES 128
typedef struct { char internal[HL_UNIQUE_ID_BYTES]; } hlUniqueId;

typedef struct hlComm* hlComm_t;
typedef void* hlStream_t; /* cudaStream_t, or NULL with the host-memory device */

/* Element size in bytes, 0 for an unknown type. */
size_t hlTypeSize(hlDataType_t t);
const char* hlGetErrorString(hlResult_t r);
/* Text of the last error raised on the calling thread (empty if none). */
const char* hlGetLastError(void);
int hlVersion(void);

/* ---- communicator ------------------------------------------------------ */
hlResult_t hlGetUniqueId(hlUniqueId* id);
/* A zeroed id selects single-process mode: the ranks are threads of one
 * process, one per device. Otherwise one process per rank on one node. */
hlResult_t hlCommInitRank(hlComm_t* comm, int nranks, hlUniqueId id, int rank);
/* Same, with the device chosen explicitly (-1 = current CUDA device, -2 = the
 * host-memory stand-in device that needs no GPU). */
hlResult_t hlCommInitRankDevice(hlComm_t* comm, int nranks, hlUniqueId id, int rank, int device);
hlResult_t hlCommDestroy(hlComm_t comm);
hlResult_t hlCommAbort(hlComm_t comm);
hlResult_t hlCommRank(hlComm_t comm, int* rank);
hlResult_t hlCommSize(hlComm_t comm, int* size);
hlResult_t hlCommDevice(hlComm_t comm, int* device);
/* Latched asynchronous error of the communicator (device waits that ran out,
 * executor failures). hlSuccess while healthy. */
hlResult_t hlCommGetAsyncError(hlComm_t comm, hlResult_t* async_error);
/* Host-blocking: returns once everything this communicator submitted to the
 * CPU-driven (PCIe / host-memory) path has completed. */
hlResult_t hlCommDrain(hlComm_t comm);
hlResult_t hlFinalize(void);

/* ---- collectives ------------------------------------------------------- */
/* Extended call descriptor; zero-initialise, then fill what differs. */
typedef struct {
  hlPath_t path;          /* default hlPathAuto */
  hlAlgo_t algo;          /* default hlAlgoAuto */
  hlDataType_t out_type;  /* result type; set has_out_type to use */
  int has_out_type;
  hlDataType_t wire_type; /* type carried over the link; set has_wire_type to use */
  int has_wire_type;
  float scale;            /* multiplies the reduced value; 0 means 1.0 */
  int max_blocks;         /* cap on CTAs (0 = table) */
  int deterministic;      /* force the fixed-order P2P kernels */
} hlCallOpts;

hlResult_t hlAllReduce(const void* send, void* recv, size_t count, hlDataType_t t, hlRedOp_t op,
                       hlComm_t comm, hlStream_t stream);
hlResult_t hlAllReduceEx(const void* send, void* recv, size_t count, hlDataType_t t, hlRedOp_t op,
                         const hlCallOpts* opts, hlComm_t comm, hlStream_t stream);
hlResult_t hlReduceScatter(const void* send, void* recv, size_t recvcount, hlDataType_t t,
                           hlRedOp_t op, hlComm_t comm, hlStream_t stream);
hlResult_t hlReduceScatterEx(const void* send, void* recv, size_t recvcount, hlDataType_t t,
                             hlRedOp_t op, const hlCallOpts* opts, hlComm_t comm,
                             hlStream_t stream);
hlResult_t hlAllGather(const void* send, void* recv, size_t sendcount, hlDataType_t t,
                       hlComm_t comm, hlStream_t stream);
hlResult_t hlAllGatherEx(const void* send, void* recv, size_t sendcount, hlDataType_t t,
                         const hlCallOpts* opts, hlComm_t comm, hlStream_t stream);
hlResult_t hlBroadcast(const void* send, void* recv, size_t count, hlDataType_t t, int root,
                       hlComm_t comm, hlStream_t stream);
hlResult_t hlBroadcastEx(const void* send, void* recv, size_t count, hlDataType_t t, int root,
                         const hlCallOpts* opts, hlComm_t comm, hlStream_t stream);
hlResult_t hlAllToAll(const void* send, void* recv, size_t count_per_peer, hlDataType_t t,
                      hlComm_t comm, hlStream_t stream);
hlResult_t hlAllToAllEx(const void* send, void* recv, size_t count_per_peer, hlDataType_t t,
                        const hlCallOpts* opts, hlComm_t comm, hlStream_t stream);
/* Device-side barrier over the NVLink flags (an 8-byte exchange). */
hlResult_t hlBarrier(hlComm_t comm, hlStream_t stream);

/* ---- registered device memory --------------------------------------------
 * hlMemAlloc returns memory of the communicator's device. When the communicator
 * has a dedicated-link path with two or more ranks the memory is REGISTERED: it
 * comes from a symmetric heap (HYLINK_SYMM_HEAP_BYTES per rank, created at the
 * first call) that every peer maps and, with NVLS, that is bound to one
 * multicast object. Collectives whose buffers are registered run zero-copy:
 * peers' inputs are read and peers' outputs written in place (multimem
 * load-reduce / store through NVSwitch, or plain peer loads and stores), with
 * no staging copy at all. Rules, as for any symmetric allocator: every rank
 * calls hlMemAlloc / hlMemFree in the same order with the same sizes (a buffer
 * then has the same heap offset everywhere; a collective whose ranks disagree
 * is stopped with an error before it touches memory), no collective of the
 * communicator may be in flight during the very first allocation, and zero-copy
 * needs 16-byte aligned buffers of whole 16-byte packets (anything else is
 * staged as usual). Unregistered pointers keep working everywhere. When the
 * heap is exhausted or unavailable the call falls back to cudaMalloc. With the
 * host-memory device the memory is host memory. */
hlResult_t hlMemAlloc(hlComm_t comm, size_t bytes, void** ptr);
hlResult_t hlMemFree(hlComm_t comm, void* ptr);
/* 1 when [ptr, ptr + bytes) lies in the communicator's registered heap. */
int hlMemIsRegistered(hlComm_t comm, const void* ptr, size_t bytes);
/* Allocator hooks with the signature of PyTorch's pluggable CUDA allocator; they serve from the heap of the
 * communicator that hlSetAllocatorComm named for the device (plain cudaMalloc / cudaFree when there is none). */
void hlSetAllocatorComm(hlComm_t comm);
hlComm_t hlGetAllocatorComm(int device);
void* hlTorchAlloc(ssize_t size, int device, void* stream);
void hlTorchFree(void* ptr, ssize_t size, int device, void* stream);

/* ---- observability ----------------------------------------------------- */
typedef struct {
  uint64_t calls;
  uint64_t bytes;
  uint64_t nvl_bytes;
  uint64_t pcie_bytes;
  uint64_t kernel_launches;   /* launches of this library's own kernels */
  uint64_t copy_engine_ops;   /* cudaMemcpyAsync issued by the PCIe executor */
  double last_alpha;          /* PCIe byte share used by the latest split call */
  double last_fast_ms;
  double last_pcie_ms;
  int nvls;                   /* 1 if a multicast mapping is active */
  int symm_mode;              /* 0 none, 1 cuMem+fd, 2 cudaIpc, 3 in-process */
  uint64_t fused_landing_slices; /* PCIe path: reduce launches that read landed host chunks themselves (no H2D copy) */
  uint64_t folded_sources;    /* ... and further sources folded into such launches */
  uint64_t registered_bytes;  /* bytes handed out from the registered-memory heap */
  uint64_t small_path_calls;  /* PCIe path: collectives served by the stream-ordered small-message path (no CPU thread) */
  uint64_t h2h_range_jobs;    /* PCIe path: host-to-host nodes handed to a worker team as a whole (worker-side progress) */
  uint64_t composed_allreduces; /* PCIe path: all-reduces run as reduce-scatter + in-place all-gather (HYLINK_PCIE_AR_COMPOSE=1) */
} hlCommStats;
hlResult_t hlCommGetStats(hlComm_t comm, hlCommStats* out);
/* Serialises the tuned (op-key -> alpha, bandwidth) table as JSON into buf;
 * returns the needed length in *len. */
hlResult_t hlCommDumpTuning(hlComm_t comm, char* buf, size_t* len);
hlResult_t hlCommLoadTuning(hlComm_t comm, const char* json);

#ifdef __cplusplus
}
#endif
#endif /* HYLINK_HYLINK_H_ */
