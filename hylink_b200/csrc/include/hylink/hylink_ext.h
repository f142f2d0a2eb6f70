/*
 * Low-level entry points: the single-GPU emulation of a multi-rank NVLink
 * group (used to test the cross-rank kernels where only one GPU is present),
 * the landing-reduce kernel, the host SIMD kernels, the schedule-IR tools and
 * the controller objects. Everything here is also reachable from Python
 * through ctypes.
 */
#ifndef HYLINK_HYLINK_EXT_H_
#define HYLINK_HYLINK_EXT_H_

#include "hylink/hylink.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- emulated NVLink group: N ranks on one device, one cooperative launch */
typedef struct hlEmu* hlEmu_t;
hlResult_t hlEmuCreate(int nranks, int device, size_t stage_bytes, int timeout_ms, hlEmu_t* out);
hlResult_t hlEmuDestroy(hlEmu_t e);
/* ins/outs: one pointer per rank. kind: 0 all-reduce, 1 reduce-scatter,
 * 2 all-gather, 3 broadcast, 4 all-to-all, 5 barrier. */
hlResult_t hlEmuCollective(hlEmu_t e, int kind, const void* const* ins, void* const* outs, size_t count,
                           size_t in_seg_stride, size_t out_seg_stride, int in_dt, int out_dt, int wire_dt,
                           int op, float scale, int root, int algo, int max_blocks, hlStream_t stream);
/* Registered memory of the emulated group: one buffer per emulated rank at the same heap offset. */
hlResult_t hlEmuHeapAlloc(hlEmu_t e, size_t bytes, void** ptrs);
hlResult_t hlEmuHeapFree(hlEmu_t e, void* ptr_rank0);
hlResult_t hlEmuSetActiveRanks(hlEmu_t e, int k);
/* status of emulated rank i: 0 ok, 1 a bounded wait ran out. detail = step<<32 | peer. */
hlResult_t hlEmuStatus(hlEmu_t e, int i, uint64_t* code, uint64_t* detail, uint64_t* block);
hlResult_t hlEmuReset(hlEmu_t e);
hlResult_t hlEmuLaunches(hlEmu_t e, uint64_t* n);

/* ---- landing reduce: dst = scale * op(srcs...) (+dst when accumulate) ---- */
hlResult_t hlReduceLanding(void* dst, const void* const* srcs, int nsrc, int accumulate, size_t count,
                           hlDataType_t t, hlRedOp_t op, float scale, int blocks, hlStream_t stream);

/* Limits how long the NEXT hlCommInitRank* on the calling thread waits for
 * its peers to show up (then reverts to the configured timeout). */
hlResult_t hlSetRendezvousTimeoutMs(int ms);

/* ---- schedule IR tools ---------------------------------------------------- */
typedef struct {
  int nranks, instructions, dependency_edges;
  int input_chunks, output_chunks, internal_chunks, host_chunks, numa_nodes;
  int uses_remote_device, uses_host_reduce;
} hlIrInfo;
/* Emits reference-format schedule XML for any gpu->NUMA pattern ("00001111").
 * Returns the needed length in *len; call with buf == NULL to size. */
hlResult_t hlIrGenerate(const char* collective, const char* numa_pattern, const char* variant, int root, char* buf,
                        size_t* len);
/* Parses and compiles a schedule; in_place: 0 none, 1 same buffer, 2 gather slot, 3 scatter slot. */
hlResult_t hlIrInspect(const char* xml, const char* numa_pattern, int send_segs, int recv_segs, int in_place,
                       hlIrInfo* info);
hlResult_t hlIrRoundTrip(const char* xml, char* buf, size_t* len);
/* An id for a group whose ranks are threads of the calling process (they rendezvous in process memory, not through
 * shared-memory files). Every call names a new group; the all-zero id names one more. */
hlResult_t hlGetInProcessId(hlUniqueId* id);

/* Collectives whose segments are `stride` elements apart (>= count; 0 = adjacent) in the gathered / scattered buffer.
 * Dedicated-link path only. */
hlResult_t hlAllGatherSeg(const void* send, void* recv, size_t count, size_t recv_stride, hlDataType_t t, hlComm_t comm, hlStream_t stream);
hlResult_t hlReduceScatterSeg(const void* send, void* recv, size_t count, size_t send_stride, hlDataType_t t, hlRedOp_t op, hlComm_t comm,
                              hlStream_t stream);
hlResult_t hlAllToAllSeg(const void* send, void* recv, size_t count, size_t send_stride, size_t recv_stride, hlDataType_t t, hlComm_t comm,
                         hlStream_t stream);
/* Pair topology (NVML through dlopen; HYLINK_NVML_LIB names another library). hlTopoPairQuery: 1 when NVML answered;
 * *same_switch = the two PCI functions sit under one PCIe switch, *nvlink = NVLink joins them.
 * hlTopoDirectAllowed: the selection rule of the `_direct` schedule files for n x n matrices (row-major). */
int hlTopoPairQuery(const char* bus_a, const char* bus_b, int* same_switch, int* nvlink);
int hlTopoDirectAllowed(const char* collective, const char* pattern, const unsigned char* same_switch, const unsigned char* nvlink,
                        const unsigned char* peer, int n);
/* Node scope: registers (rank, pid, device) of a communicator (named by its hash) in this machine's shared table and
 * waits up to wait_ms for the other ranks. Returns the ranks seen here; *flags = all on this machine | no two on one
 * device << 1 | devices in rank order << 2. hlNodeScopeLeave drops the entry (the last rank removes the table). */
int hlNodeScopeDetect(uint64_t comm_hash, int nranks, int rank, int device, int wait_ms, int* flags);
void hlNodeScopeLeave(uint64_t comm_hash, int nranks, int rank);
/* Copy-engine lanes per direction the PCIe executor uses for a collective of this size (the lane policy table). */
int hlDmaLaneCount(const char* collective, size_t message_bytes, int world, int max_lanes, int forced);
/* Runs a caller-supplied schedule on the PCIe path of `comm`. */
hlResult_t hlSubmitIr(hlComm_t comm, const char* xml, const void* send, void* recv, size_t seg_count, size_t stride,
                      int send_segs, int recv_segs, hlDataType_t t, hlRedOp_t op, hlStream_t stream);
hlResult_t hlCommNumaPattern(hlComm_t comm, char* buf, size_t* len);

/* ---- kernel timeline ---------------------------------------------------------
 * With HYLINK_KERNEL_TIMELINE=1 at communicator creation every NVLink-path kernel records, for its first 148 CTAs,
 * %globaltimer at entry, at arrival at and release from each cross-GPU barrier, and at exit, in a ring of the last 16
 * launches. Returns the ring (words; call with out == NULL for the length): stamps [call][cta][8], then 4 words per
 * call (flag base, kind << 32 | CTAs, element count, 0). Synchronises the device. */
hlResult_t hlCommKernelTimeline(hlComm_t comm, uint64_t* out, size_t* words);
/* Same for emulated rank i of a single-GPU group. */
hlResult_t hlEmuKernelTimeline(hlEmu_t e, int i, uint64_t* out, size_t* words);

/* ---- link probe -------------------------------------------------------------
 * Copies `bytes` between the first half of this rank's staging region and the second half of the next rank's with a
 * bare kernel of the given shape. mode: 0 push (local load, peer store), 1 pull (peer load, local store), 2 local
 * copy, 3 peer stores only, 4 peer loads only. layout: 0 grid-strided, 1 one contiguous range per CTA. unroll: 2, 4,
 * 8 (16 up to 512 threads). Waits on nothing; time it with events on `stream`. */
hlResult_t hlNvlLinkProbe(hlComm_t comm, int mode, int blocks, int threads, int unroll, int layout, size_t bytes, hlStream_t stream);
/* Modes 5 (to the peer) and 6 (local) run the copy on the bulk-copy engine instead: one thread per CTA drives a
 * ring of 8 shared-memory tiles with asynchronous bulk loads and stores; `threads` then gives the tile size in
 * bytes (1 KiB..24 KiB, a multiple of 128), `unroll` and `layout` are ignored. */
/* Test aid: copies between host memory and this rank's staging region at `offset` (the probe's source is the first
 * half of the region, its destination the second half; hlNvlStageBytes gives the size). */
hlResult_t hlNvlStageAccess(hlComm_t comm, int write, size_t offset, void* host, size_t bytes);
size_t hlNvlStageBytes(hlComm_t comm);

/* ---- host SIMD kernels ------------------------------------------------------ */
int hlHostReduce(void* dst, const void* a, const void* b, size_t count, int dtype, int op, int level_cap);
void hlHostCopy(void* dst, const void* src, size_t bytes, int non_temporal);
int hlHostSimdLevel(void);
/* Copy (reduce = 0) or three-address sum (reduce = 1) of `bytes` through `threads` pool workers pinned to dst_numa,
 * sources placed on src_numa (-1 = wherever). *gbs = mean rate over `iters` runs in GB/s of destination bytes. */
hlResult_t hlHostBench(int reduce, size_t bytes, int threads, int src_numa, int dst_numa, int iters, int non_temporal,
                       int dtype, double* gbs, double* best_gbs);
int hlHostNumaNodes(void);

/* ---- tracing and configuration --------------------------------------------- */
void hlTraceOpen(const char* path, int rank);
void hlTraceFlush(void);
void hlConfigReload(void);
/* A setting by name as resolved from the environment (zero_copy, small_msg_timeout_ms, host_buffer_bytes, ...); -1 for an unknown name. */
long long hlConfigValue(const char* name);
/* Arms the SIGUSR1 all-threads stack dump (needs HYLINK_SIGDUMP=1). */
void hlInstallSigdump(void);

/* ---- control-plane self check (no GPU): barrier, mailbox, fd passing ------ */
hlResult_t hlCtrlSelfTest(hlUniqueId id, int nranks, int rank, int rounds);

#ifdef __cplusplus
}
#endif
#endif
