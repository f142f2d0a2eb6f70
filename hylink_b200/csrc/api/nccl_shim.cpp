// libhylink_nccl.so: drop-in NCCL symbols.
//
// Preload it (LD_PRELOAD) or link against it in place of libnccl: programs keep
// calling ncclCommInitRank / ncclAllReduce / ncclReduceScatter / ncclAllGather /
// ncclBroadcast with unchanged signatures. The real library is opened with
// dlopen and used for everything this layer does not serve: communicator
// bootstrap, ncclSend/ncclRecv (pipeline traffic stays on NCCL p2p), ncclReduce,
// custom reduction operators, communicators that span several nodes.
//
// For every communicator whose ranks all live on this node, a hylink
// communicator is created next to the real one (same rank numbering, unique id
// derived from the NCCL id); the five collectives above then run on this
// library's NVLink kernels — forked onto the PCIe path when the orchestrator is
// enabled (HYLINK_ORCH_ENABLE / AMPCCL_ENABLE). Any failure to set the side
// communicator up degrades to pure pass-through.
//
// Parity: multipath-orchestrator/libampccl/hook/nccl_hook.cc:129-219 (dlopen
// and originals), :244-284 (node-scope gate), :295-462 (init / split / destroy
// hooks), :464-646 (per-collective gates), and the PCIe-only NCCL personality
// of pcie-ccl-cuda/src/api/nccl_compat/nccl_hook.cpp:264-811 (pnccl* aliases
// included).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "core/core.h"
#include "hylink/hylink.h"
#include "hylink/hylink_ext.h"

namespace {

struct Real {
  void* handle = nullptr;
#define HL_REAL(name) decltype(&::name) name = nullptr
  HL_REAL(ncclGetVersion);
  HL_REAL(ncclGetUniqueId);
  HL_REAL(ncclCommInitRank);
  HL_REAL(ncclCommInitRankConfig);
  HL_REAL(ncclCommInitAll);
  HL_REAL(ncclCommFinalize);
  HL_REAL(ncclCommDestroy);
  HL_REAL(ncclCommAbort);
  HL_REAL(ncclCommSplit);
  HL_REAL(ncclCommCount);
  HL_REAL(ncclCommCuDevice);
  HL_REAL(ncclCommUserRank);
  HL_REAL(ncclCommGetAsyncError);
  HL_REAL(ncclAllReduce);
  HL_REAL(ncclReduceScatter);
  HL_REAL(ncclAllGather);
  HL_REAL(ncclBroadcast);
  HL_REAL(ncclBcast);
  HL_REAL(ncclGroupStart);
  HL_REAL(ncclGroupEnd);
#undef HL_REAL
};

Real g_real;
std::once_flag g_once;
bool g_loaded = false;

void loadReal() {
  std::call_once(g_once, [] {
    const char* forced = getenv("HYLINK_REAL_NCCL");
    const char* names[] = {forced, "libnccl.so.2", "libnccl.so", nullptr};
    for (int i = forced ? 0 : 1; names[i] && !g_real.handle; ++i) g_real.handle = dlopen(names[i], RTLD_NOW | RTLD_LOCAL);
    if (!g_real.handle) {
      HL_ERR("libhylink_nccl: cannot open the real NCCL library (%s)", dlerror());
      return;
    }
#define HL_LOAD(name) g_real.name = reinterpret_cast<decltype(g_real.name)>(dlsym(g_real.handle, #name))
    HL_LOAD(ncclGetVersion);
    HL_LOAD(ncclGetUniqueId);
    HL_LOAD(ncclCommInitRank);
    HL_LOAD(ncclCommInitRankConfig);
    HL_LOAD(ncclCommInitAll);
    HL_LOAD(ncclCommFinalize);
    HL_LOAD(ncclCommDestroy);
    HL_LOAD(ncclCommAbort);
    HL_LOAD(ncclCommSplit);
    HL_LOAD(ncclCommCount);
    HL_LOAD(ncclCommCuDevice);
    HL_LOAD(ncclCommUserRank);
    HL_LOAD(ncclCommGetAsyncError);
    HL_LOAD(ncclAllReduce);
    HL_LOAD(ncclReduceScatter);
    HL_LOAD(ncclAllGather);
    HL_LOAD(ncclBroadcast);
    HL_LOAD(ncclBcast);
    HL_LOAD(ncclGroupStart);
    HL_LOAD(ncclGroupEnd);
#undef HL_LOAD
    g_loaded = g_real.ncclCommInitRank && g_real.ncclAllReduce;
  });
}

struct Side {
  hlComm_t comm = nullptr;
  int rank = 0, nranks = 1;
  uint64_t id_hash = 0;
  int splits = 0;
};
std::mutex g_mu;
std::map<ncclComm_t, Side> g_side;
std::atomic<uint64_t> g_intercepted{0}, g_passed{0};

bool enabled() {
  static const bool on = hl::envBool({"HYLINK_NCCL_INTERCEPT"}, true);
  return on;
}
size_t minBytes() {
  static const size_t v = (size_t)hl::envInt({"HYLINK_NCCL_MIN_BYTES"}, 0);
  return v;
}

uint64_t fnv(const void* p, size_t n, uint64_t h = 0xcbf29ce484222325ull) {
  const unsigned char* b = (const unsigned char*)p;
  for (size_t i = 0; i < n; ++i) {
    h ^= b[i];
    h *= 0x100000001b3ull;
  }
  return h;
}

hlUniqueId deriveId(uint64_t h) {
  hlUniqueId id;
  memset(&id, 0, sizeof(id));
  snprintf(id.internal, sizeof(id.internal), "nccl-%016llx", (unsigned long long)h);
  return id;
}

// Node scope: the side communicator exists only when every rank of the NCCL
// communicator is a GPU of this machine.
void attachSide(ncclComm_t real, uint64_t id_hash) {
  if (!enabled() || !real) return;
  int n = 0, r = 0, dev = -1;
  if (g_real.ncclCommCount(real, &n) != ncclSuccess || g_real.ncclCommUserRank(real, &r) != ncclSuccess ||
      g_real.ncclCommCuDevice(real, &dev) != ncclSuccess)
    return;
  int local = 0;
  if (cudaGetDeviceCount(&local) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  if (n < 1 || n > 8 || (n > local && !hl::envBool({"HYLINK_NCCL_ASSUME_SINGLE_NODE"}, false))) {
    HL_INFO("libhylink_nccl: communicator of %d ranks is not confined to this node (%d GPUs): pass-through", n, local);
    return;
  }
  // Ranks leave the real init within moments of each other, so a short wait
  // distinguishes "all here" from "some ranks are elsewhere".
  hlSetRendezvousTimeoutMs((int)std::max<long long>(2000, hl::Config::get().node_scope_wait_ms));
  hlComm_t side = nullptr;
  int prev = -1;
  cudaGetDevice(&prev);
  hlResult_t rc = hlCommInitRankDevice(&side, n, deriveId(id_hash), r, dev);
  if (prev >= 0) cudaSetDevice(prev);
  if (rc != hlSuccess) {
    HL_WARN("libhylink_nccl: side communicator not created (%s): pass-through", hlGetLastError());
    return;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  Side s;
  s.comm = side;
  s.rank = r;
  s.nranks = n;
  s.id_hash = id_hash;
  g_side[real] = s;
}

hlComm_t sideOf(ncclComm_t real) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_side.find(real);
  return it == g_side.end() ? nullptr : it->second.comm;
}

void dropSide(ncclComm_t real, bool abort) {
  hlComm_t c = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_side.find(real);
    if (it == g_side.end()) return;
    c = it->second.comm;
    g_side.erase(it);
  }
  if (abort) hlCommAbort(c);
  else hlCommDestroy(c);
}

bool typeOk(ncclDataType_t t) { return (int)t >= 0 && (int)t < (int)hlNumTypes && hlTypeSize((hlDataType_t)t) != 0; }
bool opOk(ncclRedOp_t op) { return (int)op >= 0 && (int)op <= (int)ncclAvg; }

ncclResult_t toNccl(hlResult_t r) {
  switch (r) {
    case hlSuccess: return ncclSuccess;
    case hlInvalidArgument: return ncclInvalidArgument;
    case hlSystemError: return ncclSystemError;
    case hlDeviceError: return ncclUnhandledCudaError;
    case hlUnsupported: return ncclInvalidUsage;
    case hlRemoteError: case hlNetworkError: return ncclRemoteError;
    default: return ncclInternalError;
  }
}

#define REQUIRE_REAL()         \
  loadReal();                  \
  if (!g_loaded) return ncclSystemError

}  // namespace

extern "C" {

__attribute__((visibility("default"))) ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
  REQUIRE_REAL();
  ncclResult_t r = g_real.ncclCommInitRank(comm, nranks, id, rank);
  if (r == ncclSuccess && comm) attachSide(*comm, fnv(&id, sizeof(id)));
  return r;
}

__attribute__((visibility("default"))) ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank,
                                                                           ncclConfig_t* config) {
  REQUIRE_REAL();
  if (!g_real.ncclCommInitRankConfig) return ncclInvalidUsage;
  ncclResult_t r = g_real.ncclCommInitRankConfig(comm, nranks, id, rank, config);
  // a non-blocking communicator may still be initialising (ncclInProgress): the side communicator needs the final one
  if (r == ncclSuccess && comm) attachSide(*comm, fnv(&id, sizeof(id)));
  return r;
}

__attribute__((visibility("default"))) ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm,
                                                                  ncclConfig_t* config) {
  REQUIRE_REAL();
  if (!g_real.ncclCommSplit) return ncclInvalidUsage;
  ncclResult_t r = g_real.ncclCommSplit(comm, color, key, newcomm, config);
  if (r != ncclSuccess || !newcomm || !*newcomm || color < 0) return r;
  // Children are pure NCCL unless asked for (same default as the reference: AMPCCL_PCIE_CHILD_COMMS).
  if (!hl::envBool({"HYLINK_NCCL_CHILD_COMMS", "AMPCCL_PCIE_CHILD_COMMS"}, false)) return r;
  uint64_t parent = 0;
  int ordinal = 0;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_side.find(comm);
    if (it == g_side.end()) return r;
    parent = it->second.id_hash;
    ordinal = ++it->second.splits;
  }
  int tuple[2] = {color, ordinal};
  attachSide(*newcomm, fnv(tuple, sizeof(tuple), parent));
  return r;
}

__attribute__((visibility("default"))) ncclResult_t ncclCommDestroy(ncclComm_t comm) {
  REQUIRE_REAL();
  dropSide(comm, false);
  return g_real.ncclCommDestroy(comm);
}
__attribute__((visibility("default"))) ncclResult_t ncclCommFinalize(ncclComm_t comm) {
  REQUIRE_REAL();
  return g_real.ncclCommFinalize ? g_real.ncclCommFinalize(comm) : ncclSuccess;
}
__attribute__((visibility("default"))) ncclResult_t ncclCommAbort(ncclComm_t comm) {
  REQUIRE_REAL();
  dropSide(comm, true);
  return g_real.ncclCommAbort(comm);
}

__attribute__((visibility("default"))) ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* err) {
  REQUIRE_REAL();
  ncclResult_t r = g_real.ncclCommGetAsyncError(comm, err);
  if (r == ncclSuccess && err && *err == ncclSuccess) {
    if (hlComm_t s = sideOf(comm)) {
      hlResult_t e = hlSuccess;
      hlCommGetAsyncError(s, &e);
      if (e != hlSuccess) *err = toNccl(e);
    }
  }
  return r;
}

__attribute__((visibility("default"))) ncclResult_t ncclAllReduce(const void* send, void* recv, size_t count, ncclDataType_t t,
                                                                  ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  REQUIRE_REAL();
  hlComm_t s = sideOf(comm);
  if (s && typeOk(t) && opOk(op) && count * hlTypeSize((hlDataType_t)t) >= minBytes()) {
    g_intercepted++;
    return toNccl(hlAllReduce(send, recv, count, (hlDataType_t)t, (hlRedOp_t)op, s, stream));
  }
  g_passed++;
  return g_real.ncclAllReduce(send, recv, count, t, op, comm, stream);
}

__attribute__((visibility("default"))) ncclResult_t ncclReduceScatter(const void* send, void* recv, size_t recvcount, ncclDataType_t t,
                                                                      ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  REQUIRE_REAL();
  hlComm_t s = sideOf(comm);
  if (s && typeOk(t) && opOk(op) && recvcount * hlTypeSize((hlDataType_t)t) >= minBytes()) {
    g_intercepted++;
    return toNccl(hlReduceScatter(send, recv, recvcount, (hlDataType_t)t, (hlRedOp_t)op, s, stream));
  }
  g_passed++;
  return g_real.ncclReduceScatter(send, recv, recvcount, t, op, comm, stream);
}

__attribute__((visibility("default"))) ncclResult_t ncclAllGather(const void* send, void* recv, size_t sendcount, ncclDataType_t t,
                                                                  ncclComm_t comm, cudaStream_t stream) {
  REQUIRE_REAL();
  hlComm_t s = sideOf(comm);
  if (s && typeOk(t) && sendcount * hlTypeSize((hlDataType_t)t) >= minBytes()) {
    g_intercepted++;
    return toNccl(hlAllGather(send, recv, sendcount, (hlDataType_t)t, s, stream));
  }
  g_passed++;
  return g_real.ncclAllGather(send, recv, sendcount, t, comm, stream);
}

__attribute__((visibility("default"))) ncclResult_t ncclBroadcast(const void* send, void* recv, size_t count, ncclDataType_t t, int root,
                                                                  ncclComm_t comm, cudaStream_t stream) {
  REQUIRE_REAL();
  hlComm_t s = sideOf(comm);
  if (s && typeOk(t) && count * hlTypeSize((hlDataType_t)t) >= minBytes()) {
    g_intercepted++;
    return toNccl(hlBroadcast(send, recv, count, (hlDataType_t)t, root, s, stream));
  }
  g_passed++;
  return g_real.ncclBroadcast(send, recv, count, t, root, comm, stream);
}

__attribute__((visibility("default"))) ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t t, int root, ncclComm_t comm,
                                                              cudaStream_t stream) {
  return ncclBroadcast(buff, buff, count, t, root, comm, stream);
}

// Counters for tests and tools: collectives served here vs passed through.
__attribute__((visibility("default"))) void hlNcclShimCounters(uint64_t* intercepted, uint64_t* passed) {
  if (intercepted) *intercepted = g_intercepted.load();
  if (passed) *passed = g_passed.load();
}

// pnccl* aliases (profiling entry points of the NCCL ABI)
#define HL_ALIAS(name) __attribute__((visibility("default"), alias(#name))) extern decltype(name) p##name
HL_ALIAS(ncclCommInitRank);
HL_ALIAS(ncclCommInitRankConfig);
HL_ALIAS(ncclCommSplit);
HL_ALIAS(ncclCommDestroy);
HL_ALIAS(ncclCommFinalize);
HL_ALIAS(ncclCommAbort);
HL_ALIAS(ncclCommGetAsyncError);
HL_ALIAS(ncclAllReduce);
HL_ALIAS(ncclReduceScatter);
HL_ALIAS(ncclAllGather);
HL_ALIAS(ncclBroadcast);
HL_ALIAS(ncclBcast);
#undef HL_ALIAS

}  // extern "C"
