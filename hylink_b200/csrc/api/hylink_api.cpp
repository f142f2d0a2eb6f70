// hl* C API: communicator life cycle and collective dispatch.
//
// Parity: the dispatcher role of pcie-ccl-cuda/src/api/pccl_api.cpp:389-629
// (submitCollective) and of multipath-orchestrator/libampccl/hook/
// nccl_hook.cc:464-646 (gate, then fast-only / hybrid / PCIe-only), in one place.
#include "api/comm.h"
#include "hylink/hylink_ext.h"
#include "orch/orchestrator.h"
#include "pcie/pcie_path.h"

#include <cstring>

#include "core/trace.h"

using namespace hl;

namespace hl {

hlResult_t pollDeviceStatus(hlComm* c) {
  if (c->nvl) {
    uint64_t detail = 0, block = 0;
    const uint64_t code = c->nvl->deviceStatus(0, &detail, &block);
    if (code != HL_DEV_OK && c->async_error.load() == hlSuccess) {
      if (code == HL_DEV_ASYMMETRIC) {
        c->async_error.store(hlInvalidArgument);
        HL_ERR("rank %d: rank %llu passed a registered buffer at another heap offset than this rank (registered buffers must be "
               "allocated in the same order on every rank)", c->rank, (unsigned long long)(detail & 0xffffffffu));
      } else {
        c->async_error.store(hlTimeout);
        HL_ERR("rank %d: a device-side wait ran out (code %llu, barrier %llu, peer %llu, block %llu)", c->rank,
               (unsigned long long)code, (unsigned long long)(detail >> 32), (unsigned long long)(detail & 0xffffffffu),
               (unsigned long long)block);
      }
      if (c->bs) c->bs->latchFailure();
    }
  }
  return (hlResult_t)c->async_error.load();
}

static bool isTrio(int d) { return d == hlFloat32 || d == hlFloat16 || d == hlBfloat16; }

struct Resolved {
  int in_dt, out_dt, wire_dt;
  float scale;
  hlPath_t path;
  int algo, max_blocks;
  bool deterministic;
};

static hlResult_t resolve(hlDataType_t t, const hlCallOpts* o, Resolved* r) {
  if (!hlTypeSize(t)) return fail(hlInvalidArgument, "unknown data type %d", (int)t);
  r->in_dt = t;
  r->out_dt = (o && o->has_out_type) ? o->out_type : t;
  r->wire_dt = (o && o->has_wire_type) ? o->wire_type : t;
  r->scale = (o && o->scale != 0.0f) ? o->scale : 1.0f;
  r->path = o ? o->path : hlPathAuto;
  r->algo = o ? o->algo : hlAlgoAuto;
  r->max_blocks = o ? o->max_blocks : 0;
  r->deterministic = o ? o->deterministic != 0 : false;
  if (!hlTypeSize((hlDataType_t)r->out_dt) || !hlTypeSize((hlDataType_t)r->wire_dt)) return fail(hlInvalidArgument, "unknown out/wire type");
  if ((r->out_dt != t || r->wire_dt != t) && !(isTrio(t) && isTrio(r->out_dt) && isTrio(r->wire_dt)))
    return fail(hlUnsupported, "conversions exist only between fp32, fp16 and bf16");
  return hlSuccess;
}

static hlResult_t precheck(hlComm_t comm) {
  if (!comm) return fail(hlInvalidArgument, "null communicator");
  hlResult_t e = pollDeviceStatus(comm);
  if (e != hlSuccess) return fail(e, "communicator is in an error state");
  return hlSuccess;
}

static void account(hlComm* c, size_t bytes, size_t nvl_bytes, size_t pcie_bytes) {
  c->stats.calls++;
  c->stats.bytes += bytes;
  c->stats.nvl_bytes += nvl_bytes;
  c->stats.pcie_bytes += pcie_bytes;
}

// One rank: every collective is the identity on `bytes` bytes. Served here as nothing at all (in place) or one
// launch of the vectorised copy kernel (the landing-reduce kernel with one source) on the caller's stream, unless
// the call converts types, scales, or asks for a kernel by name (then the ordinary kernels run on the one-rank group). The reference does the same in its NCCL
// personality (pcie-ccl-cuda/src/api/nccl_compat/compat_common.cpp:453-472).
static bool singleRankIdentity(hlComm* c, const Resolved& r, const void* send, void* recv, size_t bytes, hlStream_t stream,
                               hlResult_t* result) {
  if (c->nranks != 1 || c->host_device) return false;
  if (r.in_dt != r.out_dt || r.in_dt != r.wire_dt || r.scale != 1.0f || r.algo != hlAlgoAuto) return false;
  *result = hlSuccess;
  c->stats.calls++;
  c->stats.bytes += bytes;
  if (send == recv) return true;
  c->stats.kernel_launches++;
  if (bytes % 16 == 0 && (((uintptr_t)send | (uintptr_t)recv) & 15) == 0) {
    *result = nvl::launchCopy(recv, send, bytes, (cudaStream_t)stream);
    return true;
  }
  nvl::ReduceLandingArgs a;
  memset(&a, 0, sizeof(a));
  a.dst = recv;
  a.src[0] = send;
  a.nsrc = 1;
  a.scale = 1.0f;
  const bool words = bytes % 4 == 0 && (((uintptr_t)send | (uintptr_t)recv) & 3) == 0;   // plain 32-bit lanes: no conversion at all
  a.dtype = words ? hlUint32 : hlUint8;
  a.count = words ? bytes / 4 : bytes;
  *result = nvl::launchReduceLanding(a, 0, (cudaStream_t)stream);
  return true;
}

// Decides which transport(s) serve a call.
static hlPath_t choosePath(hlComm* c, hlPath_t asked, size_t bytes) {
  if (c->host_device) return hlPathPcie;
  if (asked == hlPathNvlink || asked == hlPathPcie) return (asked == hlPathPcie && !c->pcie) ? hlPathNvlink : asked;
  if (!c->orch || !c->pcie) return hlPathNvlink;
  if (asked == hlPathSplit) return hlPathSplit;
  return c->orch->shouldSplit(bytes) ? hlPathSplit : hlPathNvlink;
}

// flags: 1 = create the PCIe path, 2 = create the orchestrator, 4 = no NVLink path.
hlResult_t commInit(hlComm_t* out, int nranks, hlUniqueId id, int rank, int device, unsigned flags) {
  if (!out) return fail(hlInvalidArgument, "null comm pointer");
  const Config& cfg = Config::get();
  installSigdump();
  std::unique_ptr<hlComm> c(new hlComm());
  c->rank = rank;
  c->nranks = nranks;
  c->id_hash = hashId(id);
  if (device == -2 || (device == -1 && !cudaAvailable())) {
    c->host_device = true;
    c->device = -2;
  } else {
    if (device == -1) HL_CUDA(cudaGetDevice(&device));
    c->device = device;
    HL_CUDA(cudaSetDevice(device));
  }
  HL_CHECK(Bootstrap::create(id, nranks, rank, PciePath::ctrlBytes(nranks) + Orchestrator::ctrlBytes(nranks),
                             cfg.barrier_timeout_ms, &c->bs));
  if (!c->host_device) {
    if (cfg.warmup_kernel) {
      HL_CHECK(nvl::launchWarmup(nullptr));
      HL_CUDA(cudaDeviceSynchronize());
    }
    HL_CHECK(nvl::prepareReduceLanding());
    if (!(flags & 4u)) {
      if (nranks > 1) {
        HL_CHECK(NvlPath::createReal(c->bs, device, &c->nvl));
      } else {
        HL_CHECK(NvlPath::createEmu(1, device, std::min<size_t>(cfg.symm_stage_bytes, (size_t)64 << 20), cfg.nvl_timeout_ms, &c->nvl));
      }
      c->stats.nvls = c->nvl->hasNvls() ? 1 : 0;
      c->stats.symm_mode = c->nvl->symmMode();
    }
  }
  const bool want_pcie = c->host_device || (flags & 1u);
  if (want_pcie && nranks > 1) {
    char* area = (char*)c->bs->extra();
    HL_CHECK(PciePath::create(c->bs, c->device, area, &c->pcie));
    if (!c->host_device && (flags & 2u) && c->nvl)
      HL_CHECK(Orchestrator::create(c.get(), area + PciePath::ctrlBytes(nranks), &c->orch));
  }
  HL_CHECK(c->bs->barrier(kBarInit));
  *out = c.release();
  return hlSuccess;
}

}  // namespace hl

static std::atomic<hlComm_t> g_alloc_comm[64];   // per device: the communicator whose heap serves the allocator hooks

extern "C" {

hlResult_t hlCommInitRank(hlComm_t* comm, int nranks, hlUniqueId id, int rank) {
  return hlCommInitRankDevice(comm, nranks, id, rank, -1);
}

hlResult_t hlCommInitRankDevice(hlComm_t* out, int nranks, hlUniqueId id, int rank, int device) {
  const Config& cfg = Config::get();
  unsigned flags = 0;
  if (cfg.orch_enable) flags |= 1u | 2u;
  if (envBool({"HYLINK_PCIE_ENABLE"}, false)) flags |= 1u;
  return hl::commInit(out, nranks, id, rank, device, flags);
}

hlResult_t hlSetRendezvousTimeoutMs(int ms) {
  hl::setAttachTimeoutMs(ms);
  return hlSuccess;
}

hlResult_t hlCommDestroy(hlComm_t comm) {
  if (!comm) return hlSuccess;
  if (comm->device >= 0 && comm->device < 64) {
    hlComm_t expect = comm;
    g_alloc_comm[comm->device].compare_exchange_strong(expect, nullptr);
  }
  if (!comm->host_device) {
    cudaSetDevice(comm->device);
    cudaDeviceSynchronize();
  }
  delete comm->orch;
  delete comm->pcie;
  delete comm->nvl;
  delete comm->bs;
  delete comm;
  return hlSuccess;
}

hlResult_t hlCommAbort(hlComm_t comm) {
  if (!comm) return hlSuccess;
  if (comm->bs) comm->bs->latchFailure();
  return hlCommDestroy(comm);
}

hlResult_t hlCommRank(hlComm_t comm, int* rank) {
  if (!comm || !rank) return hlInvalidArgument;
  *rank = comm->rank;
  return hlSuccess;
}
hlResult_t hlCommSize(hlComm_t comm, int* size) {
  if (!comm || !size) return hlInvalidArgument;
  *size = comm->nranks;
  return hlSuccess;
}
hlResult_t hlCommDevice(hlComm_t comm, int* device) {
  if (!comm || !device) return hlInvalidArgument;
  *device = comm->device;
  return hlSuccess;
}
hlResult_t hlCommGetAsyncError(hlComm_t comm, hlResult_t* e) {
  if (!comm || !e) return hlInvalidArgument;
  *e = pollDeviceStatus(comm);
  if (*e == hlSuccess && comm->pcie) *e = comm->pcie->lastResult();
  return hlSuccess;
}
hlResult_t hlCommDrain(hlComm_t comm) {
  if (!comm) return hlInvalidArgument;
  return comm->pcie ? comm->pcie->drain() : hlSuccess;
}
hlResult_t hlFinalize(void) { return hlSuccess; }

// ------------------------------------------------------------ collectives
hlResult_t hlAllReduce(const void* send, void* recv, size_t count, hlDataType_t t, hlRedOp_t op, hlComm_t comm,
                       hlStream_t stream) {
  return hlAllReduceEx(send, recv, count, t, op, nullptr, comm, stream);
}

hlResult_t hlAllReduceEx(const void* send, void* recv, size_t count, hlDataType_t t, hlRedOp_t op,
                         const hlCallOpts* opts, hlComm_t comm, hlStream_t stream) {
  HL_CHECK(precheck(comm));
  TraceScope range("collective", "hylink all_reduce", comm->rank);   // also an NVTX range
  if (!send || !recv) return fail(hlInvalidArgument, "null buffer");
  if ((int)op < 0 || op >= hlNumOps) return fail(hlInvalidArgument, "bad reduction op %d", (int)op);
  Resolved r;
  HL_CHECK(resolve(t, opts, &r));
  if (count == 0) return hlSuccess;
  const size_t bytes = count * hlTypeSize(t);
  std::lock_guard<std::mutex> lk(comm->mu);
  {
    hlResult_t one;
    if (singleRankIdentity(comm, r, send, recv, bytes, stream, &one)) return one;
  }
  const hlPath_t path = choosePath(comm, r.path, bytes);
  if (path == hlPathPcie) {
    if (!comm->pcie) return fail(hlUnsupported, "PCIe path not initialised (single rank or disabled)");
    if (r.out_dt != r.in_dt || r.wire_dt != r.in_dt) return fail(hlUnsupported, "the PCIe path does not convert types");
    account(comm, bytes, 0, bytes);
    return comm->pcie->allReduce(send, recv, count, t, op, r.scale, stream);
  }
  if (path == hlPathSplit) return comm->orch->allReduce(send, recv, count, t, op, r.scale, r.algo, stream);
  NvlBufs b;
  memset(&b, 0, sizeof(b));
  b.in[0] = send;
  b.out[0] = recv;
  NvlCall c;
  c.count = count;
  c.in_dt = r.in_dt;
  c.out_dt = r.out_dt;
  c.wire_dt = r.wire_dt;
  c.op = op;
  c.scale = r.scale;
  c.algo = r.algo;
  c.max_blocks = r.max_blocks;
  c.deterministic = r.deterministic;
  account(comm, bytes, bytes, 0);
  return comm->nvl->allReduce(b, c, (cudaStream_t)stream);
}

hlResult_t hlReduceScatter(const void* send, void* recv, size_t recvcount, hlDataType_t t, hlRedOp_t op, hlComm_t comm,
                           hlStream_t stream) {
  return hlReduceScatterEx(send, recv, recvcount, t, op, nullptr, comm, stream);
}

hlResult_t hlReduceScatterEx(const void* send, void* recv, size_t recvcount, hlDataType_t t, hlRedOp_t op,
                             const hlCallOpts* opts, hlComm_t comm, hlStream_t stream) {
  HL_CHECK(precheck(comm));
  TraceScope range("collective", "hylink reduce_scatter", comm->rank);   // also an NVTX range
  if (!send || !recv) return fail(hlInvalidArgument, "null buffer");
  Resolved r;
  HL_CHECK(resolve(t, opts, &r));
  if (recvcount == 0) return hlSuccess;
  const size_t bytes = recvcount * hlTypeSize(t);
  std::lock_guard<std::mutex> lk(comm->mu);
  {
    hlResult_t one;
    if (singleRankIdentity(comm, r, send, recv, bytes, stream, &one)) return one;
  }
  const hlPath_t path = choosePath(comm, r.path, bytes);
  if (path == hlPathPcie) {
    if (!comm->pcie) return fail(hlUnsupported, "PCIe path not initialised");
    account(comm, bytes, 0, bytes);
    return comm->pcie->reduceScatter(send, recv, recvcount, 0, t, op, r.scale, stream);
  }
  if (path == hlPathSplit) return comm->orch->reduceScatter(send, recv, recvcount, t, op, r.scale, stream);
  NvlBufs b;
  memset(&b, 0, sizeof(b));
  b.in[0] = send;
  b.out[0] = recv;
  NvlCall c;
  c.count = recvcount;
  c.in_seg_stride = recvcount;
  c.in_dt = r.in_dt;
  c.out_dt = r.out_dt;
  c.wire_dt = r.wire_dt;
  c.op = op;
  c.scale = r.scale;
  c.algo = r.algo;
  c.max_blocks = r.max_blocks;
  c.deterministic = r.deterministic;
  account(comm, bytes, bytes, 0);
  return comm->nvl->reduceScatter(b, c, (cudaStream_t)stream);
}

hlResult_t hlAllGather(const void* send, void* recv, size_t sendcount, hlDataType_t t, hlComm_t comm, hlStream_t stream) {
  return hlAllGatherEx(send, recv, sendcount, t, nullptr, comm, stream);
}

hlResult_t hlAllGatherEx(const void* send, void* recv, size_t sendcount, hlDataType_t t, const hlCallOpts* opts,
                         hlComm_t comm, hlStream_t stream) {
  HL_CHECK(precheck(comm));
  TraceScope range("collective", "hylink all_gather", comm->rank);   // also an NVTX range
  if (!send || !recv) return fail(hlInvalidArgument, "null buffer");
  Resolved r;
  HL_CHECK(resolve(t, opts, &r));
  if (sendcount == 0) return hlSuccess;
  const size_t bytes = sendcount * hlTypeSize(t);
  std::lock_guard<std::mutex> lk(comm->mu);
  {
    hlResult_t one;
    if (singleRankIdentity(comm, r, send, recv, bytes, stream, &one)) return one;
  }
  const hlPath_t path = choosePath(comm, r.path, bytes);
  if (path == hlPathPcie) {
    if (!comm->pcie) return fail(hlUnsupported, "PCIe path not initialised");
    account(comm, bytes, 0, bytes);
    return comm->pcie->allGather(send, recv, sendcount, 0, t, stream);
  }
  if (path == hlPathSplit) return comm->orch->allGather(send, recv, sendcount, t, stream);
  NvlBufs b;
  memset(&b, 0, sizeof(b));
  b.in[0] = send;
  b.out[0] = recv;
  NvlCall c;
  c.count = sendcount;
  c.out_seg_stride = sendcount;
  c.in_dt = r.in_dt;
  c.out_dt = r.out_dt;
  c.wire_dt = r.wire_dt;
  c.algo = r.algo;
  c.max_blocks = r.max_blocks;
  account(comm, bytes, bytes, 0);
  return comm->nvl->allGather(b, c, (cudaStream_t)stream);
}

hlResult_t hlBroadcast(const void* send, void* recv, size_t count, hlDataType_t t, int root, hlComm_t comm,
                       hlStream_t stream) {
  return hlBroadcastEx(send, recv, count, t, root, nullptr, comm, stream);
}

hlResult_t hlBroadcastEx(const void* send, void* recv, size_t count, hlDataType_t t, int root, const hlCallOpts* opts,
                         hlComm_t comm, hlStream_t stream) {
  HL_CHECK(precheck(comm));
  TraceScope range("collective", "hylink broadcast", comm->rank);   // also an NVTX range
  if (!recv) return fail(hlInvalidArgument, "null buffer");
  if (root < 0 || root >= comm->nranks) return fail(hlInvalidArgument, "root %d out of range", root);
  if (comm->rank == root && !send) return fail(hlInvalidArgument, "null send buffer on the root");
  Resolved r;
  HL_CHECK(resolve(t, opts, &r));
  if (count == 0) return hlSuccess;
  const size_t bytes = count * hlTypeSize(t);
  std::lock_guard<std::mutex> lk(comm->mu);
  {
    hlResult_t one;
    if (singleRankIdentity(comm, r, send ? send : recv, recv, bytes, stream, &one)) return one;
  }
  const hlPath_t path = choosePath(comm, r.path == hlPathAuto ? hlPathNvlink : r.path, bytes);
  if (path == hlPathPcie) {
    if (!comm->pcie) return fail(hlUnsupported, "PCIe path not initialised");
    account(comm, bytes, 0, bytes);
    return comm->pcie->broadcast(send, recv, count, t, root, stream);
  }
  NvlBufs b;
  memset(&b, 0, sizeof(b));
  b.in[0] = send ? send : recv;
  b.out[0] = recv;
  NvlCall c;
  c.count = count;
  c.in_dt = r.in_dt;
  c.out_dt = r.out_dt;
  c.wire_dt = r.wire_dt;
  c.root = root;
  c.algo = r.algo;
  c.max_blocks = r.max_blocks;
  account(comm, bytes, bytes, 0);
  return comm->nvl->broadcast(b, c, (cudaStream_t)stream);
}

hlResult_t hlAllToAll(const void* send, void* recv, size_t count, hlDataType_t t, hlComm_t comm, hlStream_t stream) {
  return hlAllToAllEx(send, recv, count, t, nullptr, comm, stream);
}

hlResult_t hlAllToAllEx(const void* send, void* recv, size_t count, hlDataType_t t, const hlCallOpts* opts,
                        hlComm_t comm, hlStream_t stream) {
  HL_CHECK(precheck(comm));
  TraceScope range("collective", "hylink all_to_all", comm->rank);   // also an NVTX range
  if (!send || !recv) return fail(hlInvalidArgument, "null buffer");
  Resolved r;
  HL_CHECK(resolve(t, opts, &r));
  if (count == 0) return hlSuccess;
  const size_t bytes = count * hlTypeSize(t);
  std::lock_guard<std::mutex> lk(comm->mu);
  {
    hlResult_t one;
    if (singleRankIdentity(comm, r, send, recv, bytes, stream, &one)) return one;
  }
  const hlPath_t path = choosePath(comm, r.path, bytes);
  if (path == hlPathPcie) {
    if (!comm->pcie) return fail(hlUnsupported, "PCIe path not initialised");
    account(comm, bytes, 0, bytes);
    return comm->pcie->allToAll(send, recv, count, 0, t, stream);
  }
  if (path == hlPathSplit) return comm->orch->allToAll(send, recv, count, t, stream);
  NvlBufs b;
  memset(&b, 0, sizeof(b));
  b.in[0] = send;
  b.out[0] = recv;
  NvlCall c;
  c.count = count;
  c.in_seg_stride = count;
  c.out_seg_stride = count;
  c.in_dt = r.in_dt;
  c.out_dt = r.out_dt;
  c.wire_dt = r.wire_dt;
  c.max_blocks = r.max_blocks;
  account(comm, bytes, bytes, 0);
  return comm->nvl->allToAll(b, c, (cudaStream_t)stream);
}

// ---- collectives with explicit segment strides (dedicated-link path) -----------------------------------------------
// The segments of the gathered / scattered buffer need not be adjacent: `stride` elements lie between their starts
// (>= count). This is what the V-variants of the NCCL surface map to when every rank contributes the same count.
static hlResult_t segCall(int which, const void* send, void* recv, size_t count, size_t in_stride, size_t out_stride, hlDataType_t t,
                          hlRedOp_t op, hlComm_t comm, hlStream_t stream) {
  HL_CHECK(precheck(comm));
  if (!send || !recv) return fail(hlInvalidArgument, "null buffer");
  if (!hlTypeSize(t)) return fail(hlInvalidArgument, "unknown data type %d", (int)t);
  if ((in_stride && in_stride < count) || (out_stride && out_stride < count)) return fail(hlInvalidArgument, "segment stride smaller than the segment");
  if (count == 0) return hlSuccess;
  if (comm->host_device || !comm->nvl) return fail(hlUnsupported, "strided segments need the dedicated-link path");
  std::lock_guard<std::mutex> lk(comm->mu);
  NvlBufs b;
  memset(&b, 0, sizeof(b));
  b.in[0] = send;
  b.out[0] = recv;
  NvlCall c;
  c.count = count;
  c.in_seg_stride = in_stride;
  c.out_seg_stride = out_stride;
  c.in_dt = c.out_dt = c.wire_dt = t;
  c.op = op;
  const size_t bytes = count * hlTypeSize(t);
  account(comm, bytes, bytes, 0);
  if (which == 0) return comm->nvl->allGather(b, c, (cudaStream_t)stream);
  if (which == 1) return comm->nvl->reduceScatter(b, c, (cudaStream_t)stream);
  return comm->nvl->allToAll(b, c, (cudaStream_t)stream);
}
hlResult_t hlAllGatherSeg(const void* send, void* recv, size_t count, size_t recv_stride, hlDataType_t t, hlComm_t comm, hlStream_t stream) {
  return segCall(0, send, recv, count, 0, recv_stride, t, hlSum, comm, stream);
}
hlResult_t hlReduceScatterSeg(const void* send, void* recv, size_t count, size_t send_stride, hlDataType_t t, hlRedOp_t op, hlComm_t comm,
                              hlStream_t stream) {
  return segCall(1, send, recv, count, send_stride, 0, t, op, comm, stream);
}
hlResult_t hlAllToAllSeg(const void* send, void* recv, size_t count, size_t send_stride, size_t recv_stride, hlDataType_t t, hlComm_t comm,
                         hlStream_t stream) {
  return segCall(2, send, recv, count, send_stride, recv_stride, t, hlSum, comm, stream);
}

hlResult_t hlBarrier(hlComm_t comm, hlStream_t stream) {
  HL_CHECK(precheck(comm));
  std::lock_guard<std::mutex> lk(comm->mu);
  if (comm->host_device || !comm->nvl) return comm->bs->barrier(kBarUser);
  return comm->nvl->barrier((cudaStream_t)stream);
}

size_t hlNvlStageBytes(hlComm_t comm) { return (comm && comm->nvl) ? comm->nvl->stageBytes() : 0; }

hlResult_t hlNvlStageAccess(hlComm_t comm, int write, size_t offset, void* host, size_t bytes) {
  HL_CHECK(precheck(comm));
  std::lock_guard<std::mutex> lk(comm->mu);
  if (comm->host_device || !comm->nvl) return fail(hlUnsupported, "stage access needs the NVLink path");
  return comm->nvl->stageAccess(write != 0, offset, host, bytes);
}

hlResult_t hlCommKernelTimeline(hlComm_t comm, uint64_t* out, size_t* words) {
  HL_CHECK(precheck(comm));
  std::lock_guard<std::mutex> lk(comm->mu);
  if (comm->host_device || !comm->nvl) return fail(hlUnsupported, "the kernel timeline needs the NVLink path");
  return comm->nvl->readTimeline(0, out, words);
}

hlResult_t hlNvlLinkProbe(hlComm_t comm, int mode, int blocks, int threads, int unroll, int layout, size_t bytes, hlStream_t stream) {
  HL_CHECK(precheck(comm));
  std::lock_guard<std::mutex> lk(comm->mu);
  if (comm->host_device || !comm->nvl) return fail(hlUnsupported, "link probe needs the NVLink path");
  return comm->nvl->linkProbe(mode, blocks, threads, unroll, layout, bytes, (cudaStream_t)stream);
}

// Registered memory. With an NVLink path of two or more ranks the buffer comes from the communicator's symmetric heap
// (same offset on every rank, mapped by every peer, multicast-bound with NVLS), which lets collectives on it run
// zero-copy; every rank must then allocate and free in the same order. Otherwise (one rank, host device, heap
// exhausted or unavailable) it is ordinary memory.
hlResult_t hlMemAlloc(hlComm_t comm, size_t bytes, void** ptr) {
  if (!comm || !ptr) return hlInvalidArgument;
  if (comm->host_device) {
    *ptr = malloc(bytes);
    return *ptr ? hlSuccess : hlSystemError;
  }
  HL_CUDA(cudaSetDevice(comm->device));
  if (comm->nvl && comm->nranks > 1 && bytes) {
    std::lock_guard<std::mutex> lk(comm->mu);
    void* p[HL_MAX_RANKS] = {nullptr};
    if (comm->nvl->heapAlloc(bytes, p) == hlSuccess) {
      *ptr = p[0];
      return hlSuccess;
    }
  }
  HL_CUDA(cudaMalloc(ptr, bytes));
  return hlSuccess;
}
hlResult_t hlMemFree(hlComm_t comm, void* ptr) {
  if (!comm) return hlInvalidArgument;
  if (comm->host_device) {
    free(ptr);
    return hlSuccess;
  }
  if (!ptr) return hlSuccess;
  if (comm->nvl) {
    std::lock_guard<std::mutex> lk(comm->mu);
    uint64_t off;
    if (comm->nvl->heapOffset(0, ptr, 1, &off)) return comm->nvl->heapFree(ptr);
  }
  HL_CUDA(cudaFree(ptr));
  return hlSuccess;
}
int hlMemIsRegistered(hlComm_t comm, const void* ptr, size_t bytes) {
  if (!comm || !comm->nvl || !ptr) return 0;
  uint64_t off;
  return comm->nvl->heapOffset(0, ptr, bytes ? bytes : 1, &off) ? 1 : 0;
}

// The communicator whose heap serves hlTorchAlloc / hlTorchFree (allocator hooks with the signature PyTorch's
// pluggable CUDA allocator expects). Set by the torch.distributed backend when it creates its communicator.
void hlSetAllocatorComm(hlComm_t comm) {
  if (comm && comm->device >= 0 && comm->device < 64) g_alloc_comm[comm->device].store(comm);
}
hlComm_t hlGetAllocatorComm(int device) { return device >= 0 && device < 64 ? g_alloc_comm[device].load() : nullptr; }
void* hlTorchAlloc(ssize_t size, int device, void* stream) {
  (void)stream;
  hlComm_t c = hlGetAllocatorComm(device);
  void* p = nullptr;
  if (c) {
    if (hlMemAlloc(c, (size_t)size, &p) == hlSuccess) return p;
    return nullptr;
  }
  cudaSetDevice(device);
  if (cudaMalloc(&p, (size_t)size) != cudaSuccess) return nullptr;
  return p;
}
void hlTorchFree(void* ptr, ssize_t size, int device, void* stream) {
  (void)size;
  (void)stream;
  hlComm_t c = hlGetAllocatorComm(device);
  if (c) {
    hlMemFree(c, ptr);
    return;
  }
  cudaSetDevice(device);
  cudaFree(ptr);
}

hlResult_t hlCommGetStats(hlComm_t comm, hlCommStats* out) {
  if (!comm || !out) return hlInvalidArgument;
  std::lock_guard<std::mutex> lk(comm->mu);
  *out = comm->stats;
  out->kernel_launches = comm->stats.kernel_launches + (comm->nvl ? comm->nvl->launches() : 0) + (comm->pcie ? comm->pcie->kernelLaunches() : 0);
  out->copy_engine_ops = comm->pcie ? comm->pcie->copyOps() : 0;
  out->fused_landing_slices = comm->pcie ? comm->pcie->fusedSlices() : 0;
  out->folded_sources = comm->pcie ? comm->pcie->foldedSources() : 0;
  out->registered_bytes = comm->nvl ? comm->nvl->heapInUse() : 0;
  out->small_path_calls = comm->pcie ? comm->pcie->smallCalls() : 0;
  out->h2h_range_jobs = comm->pcie ? comm->pcie->rangeJobs() : 0;
  out->composed_allreduces = comm->pcie ? comm->pcie->composedAllReduces() : 0;
  if (comm->orch) comm->orch->fillStats(out);
  return hlSuccess;
}

hlResult_t hlCommDumpTuning(hlComm_t comm, char* buf, size_t* len) {
  if (!comm || !len) return hlInvalidArgument;
  std::string s = comm->orch ? comm->orch->dumpTuning() : std::string("{\"entries\":[]}");
  const size_t need = s.size() + 1;
  if (buf && *len >= need) memcpy(buf, s.c_str(), need);
  *len = need;
  return hlSuccess;
}
hlResult_t hlCommLoadTuning(hlComm_t comm, const char* json) {
  if (!comm || !json) return hlInvalidArgument;
  if (!comm->orch) return hlSuccess;
  return comm->orch->loadTuning(json);
}

// ------------------------------------------------------------ emulation + low-level ops
struct hlEmu {
  NvlPath* path;
};

hlResult_t hlEmuCreate(int nranks, int device, size_t stage_bytes, int timeout_ms, hlEmu_t* out) {
  if (!out) return hlInvalidArgument;
  if (!cudaAvailable()) return fail(hlDeviceError, "no CUDA device");
  NvlPath* p = nullptr;
  HL_CHECK(NvlPath::createEmu(nranks, device, stage_bytes, timeout_ms, &p));
  *out = new hlEmu{p};
  return hlSuccess;
}
hlResult_t hlEmuDestroy(hlEmu_t e) {
  if (!e) return hlSuccess;
  delete e->path;
  delete e;
  return hlSuccess;
}
hlResult_t hlEmuCollective(hlEmu_t e, int kind, const void* const* ins, void* const* outs, size_t count,
                           size_t in_seg_stride, size_t out_seg_stride, int in_dt, int out_dt, int wire_dt, int op,
                           float scale, int root, int algo, int max_blocks, hlStream_t stream) {
  if (!e) return hlInvalidArgument;
  NvlBufs b;
  memset(&b, 0, sizeof(b));
  for (int i = 0; i < e->path->nranks(); ++i) {
    b.in[i] = ins ? ins[i] : nullptr;
    b.out[i] = outs ? outs[i] : nullptr;
  }
  NvlCall c;
  c.count = count;
  c.in_seg_stride = in_seg_stride;
  c.out_seg_stride = out_seg_stride;
  c.in_dt = in_dt;
  c.out_dt = out_dt;
  c.wire_dt = wire_dt;
  c.op = op;
  c.scale = scale;
  c.root = root;
  c.algo = algo;
  c.max_blocks = max_blocks;
  cudaStream_t s = (cudaStream_t)stream;
  switch (kind) {
    case 0: return e->path->allReduce(b, c, s);
    case 1: return e->path->reduceScatter(b, c, s);
    case 2: return e->path->allGather(b, c, s);
    case 3: return e->path->broadcast(b, c, s);
    case 4: return e->path->allToAll(b, c, s);
    case 5: return e->path->barrier(s);
    default: return fail(hlInvalidArgument, "unknown emulated collective %d", kind);
  }
}
hlResult_t hlEmuHeapAlloc(hlEmu_t e, size_t bytes, void** ptrs) {
  if (!e || !ptrs) return hlInvalidArgument;
  return e->path->heapAlloc(bytes, ptrs);
}
hlResult_t hlEmuHeapFree(hlEmu_t e, void* ptr_rank0) { return e ? e->path->heapFree(ptr_rank0) : hlInvalidArgument; }
hlResult_t hlEmuSetActiveRanks(hlEmu_t e, int k) {
  if (!e || k < 1 || k > e->path->nranks()) return hlInvalidArgument;
  e->path->setEmuActiveRanks(k);
  return hlSuccess;
}
hlResult_t hlEmuStatus(hlEmu_t e, int i, uint64_t* code, uint64_t* detail, uint64_t* block) {
  if (!e || i < 0 || i >= e->path->nranks() || !code) return hlInvalidArgument;
  *code = e->path->deviceStatus(i, detail, block);
  return hlSuccess;
}
hlResult_t hlEmuKernelTimeline(hlEmu_t e, int i, uint64_t* out, size_t* words) {
  if (!e) return hlInvalidArgument;
  return e->path->readTimeline(i, out, words);
}
hlResult_t hlEmuReset(hlEmu_t e) { return e ? e->path->resetAfterError() : hlInvalidArgument; }
hlResult_t hlEmuLaunches(hlEmu_t e, uint64_t* n) {
  if (!e || !n) return hlInvalidArgument;
  *n = e->path->launches();
  return hlSuccess;
}

hlResult_t hlReduceLanding(void* dst, const void* const* srcs, int nsrc, int accumulate, size_t count, hlDataType_t t,
                           hlRedOp_t op, float scale, int blocks, hlStream_t stream) {
  if (!dst || !srcs || nsrc < 1 || nsrc > 8) return fail(hlInvalidArgument, "bad reduce-landing arguments");
  nvl::ReduceLandingArgs a;
  memset(&a, 0, sizeof(a));
  a.dst = dst;
  for (int i = 0; i < nsrc; ++i) a.src[i] = srcs[i];
  a.nsrc = nsrc;
  a.accumulate = accumulate;
  a.count = count;
  a.dtype = t;
  a.op = op;
  a.scale = scale == 0.0f ? 1.0f : scale;
  return nvl::launchReduceLanding(a, blocks, (cudaStream_t)stream);
}

}  // extern "C"
