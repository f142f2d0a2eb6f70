// libhylink_nccl.so: drop-in NCCL symbols, in two personalities.
//
// INTERPOSITION (a real libnccl can be opened). Preload the library (LD_PRELOAD)
// or link against it in place of libnccl: programs keep calling ncclCommInitRank /
// ncclCommInitAll / ncclAllReduce / ncclReduceScatter / ncclAllGather / ncclBroadcast /
// ncclAllToAll with unchanged signatures. The real library is opened with dlopen and
// serves everything this layer does not: communicator bootstrap, ncclSend / ncclRecv
// (pipeline traffic stays on NCCL p2p), ncclReduce, custom reduction operators,
// communicators that span several nodes. For every communicator whose ranks all live
// on this node a hylink communicator is created next to the real one (same rank
// numbering, unique id derived from the NCCL id); the collectives above then run on
// this library's NVLink kernels — forked onto the PCIe path when the orchestrator is
// enabled (HYLINK_ORCH_ENABLE / AMPCCL_ENABLE). Any failure to set the side
// communicator up degrades to pure pass-through.
//
// STAND-ALONE (no real libnccl, or HYLINK_NCCL_STANDALONE=1). The library IS the NCCL
// of the process: ncclGetUniqueId, ncclCommInitRank / InitRankConfig / InitAll / Split,
// the communicator queries, the collectives and ncclReduce all run on this library's
// own two paths; a one-rank communicator copies on the device; ncclSend / ncclRecv are
// refused (point-to-point traffic is NCCL's job).
//
// Both: calls between ncclGroupStart and ncclGroupEnd are collected and launched at the
// outermost ncclGroupEnd (one thread driving several GPUs issues all its ranks' calls
// in one group); the V-variants ncclAllGatherV / ncclReduceScatterV / ncclAllToAllV
// map onto the strided-segment kernels when every rank contributes the same count and
// onto per-root calls otherwise; ncclMemAlloc can hand out registered memory.
//
// Parity: multipath-orchestrator/libampccl/hook/nccl_hook.cc:129-219 (dlopen and
// originals), :244-284 (node-scope gate), :295-462 (init / InitAll / split / destroy
// hooks), :464-646 (per-collective gates, AllToAll, V-variants), and the PCIe-only NCCL
// personality of pcie-ccl-cuda/src/api/nccl_compat/nccl_hook.cpp:264-811 (group waves
// :467-544, InitAll :742, one-rank copies, pnccl* aliases).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

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
  HL_REAL(ncclGetErrorString);
  HL_REAL(ncclGetLastError);
  HL_REAL(ncclAllReduce);
  HL_REAL(ncclReduceScatter);
  HL_REAL(ncclAllGather);
  HL_REAL(ncclBroadcast);
  HL_REAL(ncclBcast);
  HL_REAL(ncclReduce);
  HL_REAL(ncclSend);
  HL_REAL(ncclRecv);
  HL_REAL(ncclGroupStart);
  HL_REAL(ncclGroupEnd);
  HL_REAL(ncclMemAlloc);
  HL_REAL(ncclMemFree);
#undef HL_REAL
  // not in every NCCL release: looked up by name, called through a plain function pointer
  ncclResult_t (*ncclAlltoAll)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
};

Real g_real;
std::once_flag g_once;
bool g_loaded = false;       // a real NCCL is open
bool g_standalone = false;   // this library serves every nccl* call itself

void loadReal() {
  std::call_once(g_once, [] {
    if (hl::envBool({"HYLINK_NCCL_STANDALONE"}, false)) {
      g_standalone = true;
      return;
    }
    const char* forced = getenv("HYLINK_REAL_NCCL");
    const char* names[] = {forced, "libnccl.so.2", "libnccl.so", nullptr};
    for (int i = forced ? 0 : 1; names[i] && !g_real.handle; ++i) g_real.handle = dlopen(names[i], RTLD_NOW | RTLD_LOCAL);
    if (g_real.handle) {
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
      HL_LOAD(ncclGetErrorString);
      HL_LOAD(ncclGetLastError);
      HL_LOAD(ncclAllReduce);
      HL_LOAD(ncclReduceScatter);
      HL_LOAD(ncclAllGather);
      HL_LOAD(ncclBroadcast);
      HL_LOAD(ncclBcast);
      HL_LOAD(ncclReduce);
      HL_LOAD(ncclSend);
      HL_LOAD(ncclRecv);
      HL_LOAD(ncclGroupStart);
      HL_LOAD(ncclGroupEnd);
      HL_LOAD(ncclMemAlloc);
      HL_LOAD(ncclMemFree);
#undef HL_LOAD
      g_real.ncclAlltoAll = reinterpret_cast<decltype(g_real.ncclAlltoAll)>(dlsym(g_real.handle, "ncclAlltoAll"));
      if (!g_real.ncclAlltoAll) g_real.ncclAlltoAll = reinterpret_cast<decltype(g_real.ncclAlltoAll)>(dlsym(g_real.handle, "ncclAllToAll"));
      // a "real" library that is this one (e.g. installed under NCCL's name) would recurse
      Dl_info mine, theirs;
      if (g_real.ncclAllReduce && dladdr((void*)&loadReal, &mine) && dladdr((void*)g_real.ncclAllReduce, &theirs) && mine.dli_fbase == theirs.dli_fbase)
        g_real = Real();
      g_loaded = g_real.ncclCommInitRank && g_real.ncclAllReduce;
    }
    if (!g_loaded) {
      HL_INFO("libhylink_nccl: no real NCCL library (%s): serving every nccl* call stand-alone", forced ? forced : "libnccl.so.2");
      g_standalone = true;
    }
  });
}

// ------------------------------------------------------------------ communicators
// Stand-alone communicators are objects of this layer; an interposed communicator is the real library's, with a
// side communicator of ours looked up by its address.
struct OwnComm {
  hlComm_t hl = nullptr;
  int rank = 0, nranks = 1, dev = -1;
  uint64_t id_hash = 0;
  int splits = 0;
};
struct Side {
  hlComm_t comm = nullptr;
  int rank = 0, nranks = 1;
  uint64_t id_hash = 0;
  int splits = 0;
  bool pending = false;   // the real communicator was still initialising when it was handed out (non-blocking init)
  bool scoped = false;    // has an entry in this machine's node-scope table
};
std::mutex g_mu;
std::map<ncclComm_t, Side> g_side;
std::set<OwnComm*> g_own;
std::atomic<uint64_t> g_intercepted{0}, g_passed{0};
thread_local std::string t_last_error;

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

OwnComm* asOwn(ncclComm_t c) {
  if (!g_standalone || !c) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  OwnComm* o = reinterpret_cast<OwnComm*>(c);
  return g_own.count(o) ? o : nullptr;
}

// Node scope: the side communicator exists only when every rank of the NCCL
// communicator is a GPU of this machine.
void attachSide(ncclComm_t real, uint64_t id_hash, const hlUniqueId* in_process = nullptr) {
  if (!enabled() || !real) return;
  int n = 0, r = 0, dev = -1;
  bool scoped = false;
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
  if (!in_process && n > 1 && !hl::envBool({"HYLINK_NCCL_ASSUME_SINGLE_NODE"}, false)) {
    // every rank registers in this machine's table and looks for the others: ranks on another machine never appear
    int flags = 0;
    const int seen = hlNodeScopeDetect(id_hash, n, r, dev, (int)std::max<long long>(200, hl::Config::get().node_scope_wait_ms), &flags);
    scoped = true;   // the entry stays while the communicator lives (peers may still be looking for it)
    if (!(flags & 1) || !(flags & 2)) {
      hlNodeScopeLeave(id_hash, n, r);
      HL_INFO("libhylink_nccl: %d of %d ranks are on this machine%s: pass-through", seen, n, (flags & 1) ? " (two ranks share a device)" : "");
      return;
    }
  }
  // Ranks leave the real init within moments of each other, so a short wait
  // distinguishes "all here" from "some ranks are elsewhere".
  hlSetRendezvousTimeoutMs((int)std::max<long long>(2000, hl::Config::get().node_scope_wait_ms));
  hlComm_t side = nullptr;
  int prev = -1;
  cudaGetDevice(&prev);
  hlResult_t rc = hlCommInitRankDevice(&side, n, in_process ? *in_process : deriveId(id_hash), r, dev);
  if (prev >= 0) cudaSetDevice(prev);
  if (rc != hlSuccess) {
    HL_WARN("libhylink_nccl: side communicator not created (%s): pass-through", hlGetLastError());
    if (scoped) hlNodeScopeLeave(id_hash, n, r);
    return;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  Side& s = g_side[real];
  s.scoped = scoped;
  s.comm = side;
  s.rank = r;
  s.nranks = n;
  s.id_hash = id_hash;
  s.pending = false;
}

hlComm_t sideOf(ncclComm_t c) {
  if (OwnComm* o = asOwn(c)) return o->hl;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_side.find(c);
  return it == g_side.end() ? nullptr : it->second.comm;
}

void dropSide(ncclComm_t real, bool abort) {
  hlComm_t c = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_side.find(real);
    if (it == g_side.end()) return;
    c = it->second.comm;
    if (it->second.scoped) hlNodeScopeLeave(it->second.id_hash, it->second.nranks, it->second.rank);
    g_side.erase(it);
  }
  if (!c) return;
  if (abort) hlCommAbort(c);
  else hlCommDestroy(c);
}

bool typeOk(ncclDataType_t t) { return (int)t >= 0 && (int)t < (int)hlNumTypes && hlTypeSize((hlDataType_t)t) != 0; }
bool opOk(ncclRedOp_t op) { return (int)op >= 0 && (int)op <= (int)ncclAvg; }
size_t esize(ncclDataType_t t) { return typeOk(t) ? hlTypeSize((hlDataType_t)t) : 0; }

ncclResult_t toNccl(hlResult_t r) {
  if (r != hlSuccess) t_last_error = hlGetLastError();
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

// ------------------------------------------------------------------ group calls
// Between ncclGroupStart and the matching outermost ncclGroupEnd this layer's launches are only recorded; they are
// issued, in call order, at the end. A thread that drives several GPUs puts all its ranks' calls into one group:
// nothing of the group may start before every member is known (NCCL's rule), and although our kernels never block
// the host, a caller is entitled to pass buffers that only become valid at the group end.
struct Deferred {
  int kind;   // 0 AR, 1 RS, 2 AG, 3 Bcast, 4 A2A, 5 reduce, 6 AG-seg, 7 RS-seg, 8 A2A-seg
  const void* send;
  void* recv;
  size_t count, stride_a, stride_b;
  ncclDataType_t t;
  ncclRedOp_t op;
  int root;
  hlComm_t comm;
  cudaStream_t stream;
};
thread_local int t_depth = 0;
thread_local std::vector<Deferred> t_queue;
thread_local ncclResult_t t_group_error = ncclSuccess;

hlResult_t reduceToRoot(const Deferred& d);

ncclResult_t issue(const Deferred& d) {
  const hlDataType_t t = (hlDataType_t)d.t;
  const hlRedOp_t op = (hlRedOp_t)d.op;
  switch (d.kind) {
    case 0: return toNccl(hlAllReduce(d.send, d.recv, d.count, t, op, d.comm, d.stream));
    case 1: return toNccl(hlReduceScatter(d.send, d.recv, d.count, t, op, d.comm, d.stream));
    case 2: return toNccl(hlAllGather(d.send, d.recv, d.count, t, d.comm, d.stream));
    case 3: return toNccl(hlBroadcast(d.send, d.recv, d.count, t, d.root, d.comm, d.stream));
    case 4: return toNccl(hlAllToAll(d.send, d.recv, d.count, t, d.comm, d.stream));
    case 5: return toNccl(reduceToRoot(d));
    case 6: return toNccl(hlAllGatherSeg(d.send, d.recv, d.count, d.stride_b, t, d.comm, d.stream));
    case 7: return toNccl(hlReduceScatterSeg(d.send, d.recv, d.count, d.stride_a, t, op, d.comm, d.stream));
    case 8: return toNccl(hlAllToAllSeg(d.send, d.recv, d.count, d.stride_a, d.stride_b, t, d.comm, d.stream));
    default: return ncclInternalError;
  }
}

ncclResult_t submit(const Deferred& d) {
  g_intercepted++;
  if (t_depth > 0) {
    t_queue.push_back(d);
    return ncclSuccess;
  }
  return issue(d);
}

// Reduce to one root = an all-reduce whose result the other ranks drop into a stream-ordered scratch buffer.
hlResult_t reduceToRoot(const Deferred& d) {
  int rank = 0;
  hlCommRank(d.comm, &rank);
  if (rank == d.root) return hlAllReduce(d.send, d.recv, d.count, (hlDataType_t)d.t, (hlRedOp_t)d.op, d.comm, d.stream);
  void* scratch = nullptr;
  const size_t bytes = d.count * hlTypeSize((hlDataType_t)d.t);
  int dev = -1, prev = -1;
  hlCommDevice(d.comm, &dev);
  cudaGetDevice(&prev);
  if (dev >= 0) cudaSetDevice(dev);
  cudaError_t e = cudaMallocAsync(&scratch, bytes ? bytes : 1, d.stream);
  hlResult_t r = hlDeviceError;
  if (e == cudaSuccess) {
    r = hlAllReduce(d.send, scratch, d.count, (hlDataType_t)d.t, (hlRedOp_t)d.op, d.comm, d.stream);
    cudaFreeAsync(scratch, d.stream);
  } else {
    cudaGetLastError();
  }
  if (prev >= 0) cudaSetDevice(prev);
  return r;
}

bool serve(hlComm_t s, ncclDataType_t t, size_t count) { return s && typeOk(t) && count * esize(t) >= minBytes(); }

#define PREPARE() loadReal()
#define REQUIRE_REAL() \
  if (!g_loaded) return ncclInvalidUsage

}  // namespace

#define HL_EXPORT __attribute__((visibility("default")))

extern "C" {

// ------------------------------------------------------------------ library-level calls
HL_EXPORT ncclResult_t ncclGetVersion(int* version) {
  PREPARE();
  if (!version) return ncclInvalidArgument;
  if (!g_standalone && g_real.ncclGetVersion) return g_real.ncclGetVersion(version);
  *version = NCCL_VERSION_CODE;
  return ncclSuccess;
}

HL_EXPORT ncclResult_t ncclGetUniqueId(ncclUniqueId* id) {
  PREPARE();
  if (!id) return ncclInvalidArgument;
  if (!g_standalone) return g_real.ncclGetUniqueId(id);
  static_assert(sizeof(ncclUniqueId) >= sizeof(hlUniqueId), "the NCCL id must be able to carry ours");
  hlUniqueId u;
  hlResult_t r = hlGetUniqueId(&u);
  memset(id, 0, sizeof(*id));
  memcpy(id, &u, sizeof(u));
  return toNccl(r);
}

HL_EXPORT const char* ncclGetErrorString(ncclResult_t r) {
  PREPARE();
  if (!g_standalone && g_real.ncclGetErrorString) return g_real.ncclGetErrorString(r);
  switch (r) {
    case ncclSuccess: return "no error";
    case ncclUnhandledCudaError: return "unhandled cuda error";
    case ncclSystemError: return "unhandled system error";
    case ncclInternalError: return "internal error";
    case ncclInvalidArgument: return "invalid argument";
    case ncclInvalidUsage: return "invalid usage";
    case ncclRemoteError: return "remote process exited or there was a network error";
    case ncclInProgress: return "operation in progress";
    default: return "unknown result code";
  }
}

HL_EXPORT const char* ncclGetLastError(ncclComm_t comm) {
  PREPARE();
  if (!t_last_error.empty() || g_standalone || !g_real.ncclGetLastError) return t_last_error.c_str();
  return g_real.ncclGetLastError(comm);
}

// ------------------------------------------------------------------ communicator lifetime
static ncclResult_t ownInit(ncclComm_t* comm, int nranks, const hlUniqueId& id, int rank, int dev, uint64_t id_hash) {
  if (!comm || nranks < 1 || rank < 0 || rank >= nranks) return ncclInvalidArgument;
  if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return ncclUnhandledCudaError;
  }
  hlComm_t h = nullptr;
  int prev = -1;
  cudaGetDevice(&prev);
  hlResult_t rc = hlCommInitRankDevice(&h, nranks, id, rank, dev);
  if (prev >= 0) cudaSetDevice(prev);
  if (rc != hlSuccess) return toNccl(rc);
  OwnComm* o = new OwnComm();
  o->hl = h;
  o->rank = rank;
  o->nranks = nranks;
  o->dev = dev;
  o->id_hash = id_hash;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_own.insert(o);
  }
  // ncclMemAlloc names no communicator: it serves from the first one of each device that is still alive
  if (!hlGetAllocatorComm(dev) && hl::envBool({"HYLINK_NCCL_REGISTERED_ALLOC"}, true)) hlSetAllocatorComm(h);
  *comm = reinterpret_cast<ncclComm_t>(o);
  return ncclSuccess;
}

HL_EXPORT ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
  PREPARE();
  if (g_standalone) {
    hlUniqueId u;
    memcpy(&u, &id, sizeof(u));
    return ownInit(comm, nranks, u, rank, -1, fnv(&id, sizeof(id)));
  }
  ncclResult_t r = g_real.ncclCommInitRank(comm, nranks, id, rank);
  if (r == ncclSuccess && comm) attachSide(*comm, fnv(&id, sizeof(id)));
  return r;
}

HL_EXPORT ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, ncclConfig_t* config) {
  PREPARE();
  if (g_standalone) {
    hlUniqueId u;
    memcpy(&u, &id, sizeof(u));
    return ownInit(comm, nranks, u, rank, -1, fnv(&id, sizeof(id)));   // the options concern the real library's transports
  }
  if (!g_real.ncclCommInitRankConfig) return ncclInvalidUsage;
  ncclResult_t r = g_real.ncclCommInitRankConfig(comm, nranks, id, rank, config);
  if (r == ncclSuccess && comm) {
    attachSide(*comm, fnv(&id, sizeof(id)));
  } else if (r == ncclInProgress && comm && *comm) {
    // Non-blocking initialisation: the communicator is handed out before it is complete. Remember it; the side
    // communicator is created when the caller's polling of ncclCommGetAsyncError first sees ncclSuccess.
    std::lock_guard<std::mutex> lk(g_mu);
    Side& s = g_side[*comm];
    s.pending = true;
    s.id_hash = fnv(&id, sizeof(id));
  }
  return r;
}

// One thread creates a communicator for each of `ndev` GPUs (devlist == nullptr: devices 0..ndev-1).
HL_EXPORT ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist) {
  PREPARE();
  if (!comms || ndev < 1) return ncclInvalidArgument;
  if (g_standalone) {
    hlUniqueId u;   // the ranks are threads of this process: they meet in process memory
    if (hlGetInProcessId(&u) != hlSuccess) return ncclSystemError;
    const uint64_t h = fnv(&u, sizeof(u));
    std::vector<ncclResult_t> res((size_t)ndev, ncclSuccess);
    std::vector<std::thread> th;
    // every rank's set-up meets the others at a rendezvous: they have to run side by side
    for (int r = 0; r < ndev; ++r) th.emplace_back([&, r] { res[(size_t)r] = ownInit(&comms[r], ndev, u, r, devlist ? devlist[r] : r, h); });
    for (auto& t : th) t.join();
    for (auto r : res)
      if (r != ncclSuccess) return r;
    return ncclSuccess;
  }
  if (!g_real.ncclCommInitAll) return ncclInvalidUsage;
  ncclResult_t r = g_real.ncclCommInitAll(comms, ndev, devlist);
  if (r != ncclSuccess || !enabled()) return r;
  static std::atomic<uint64_t> nonce{0};
  struct { uint64_t pid, n, first; } key = {(uint64_t)getpid(), nonce.fetch_add(1), (uint64_t)(uintptr_t)comms[0]};
  const uint64_t h = fnv(&key, sizeof(key));
  hlUniqueId u;
  if (hlGetInProcessId(&u) != hlSuccess) return r;
  std::vector<std::thread> th;
  for (int i = 0; i < ndev; ++i) th.emplace_back([&, i] { attachSide(comms[i], h, &u); });
  for (auto& t : th) t.join();
  return r;
}

HL_EXPORT ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* config) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) {
    // Stand-alone: every rank of the parent learns all (color, key) pairs through an all-gather on the parent, then
    // the members of one colour build a communicator ordered by (key, parent rank).
    if (!newcomm) return ncclInvalidArgument;
    const int n = o->nranks;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(o->dev);
    int* dbuf = nullptr;
    std::vector<int> all((size_t)n * 2);
    int mine[2] = {color, key};
    cudaError_t e = cudaMalloc((void**)&dbuf, sizeof(int) * 2 * (size_t)(n + 1));
    if (e != cudaSuccess) {
      cudaGetLastError();
      return ncclUnhandledCudaError;
    }
    cudaMemcpy(dbuf, mine, sizeof(mine), cudaMemcpyHostToDevice);
    hlResult_t rc = hlAllGather(dbuf, dbuf + 2, 2, hlInt32, o->hl, nullptr);
    if (rc == hlSuccess && cudaMemcpy(all.data(), dbuf + 2, sizeof(int) * 2 * (size_t)n, cudaMemcpyDeviceToHost) != cudaSuccess) rc = hlDeviceError;
    cudaFree(dbuf);
    if (prev >= 0) cudaSetDevice(prev);
    if (rc != hlSuccess) return toNccl(rc);
    int ordinal;
    {
      std::lock_guard<std::mutex> lk(g_mu);
      ordinal = ++o->splits;
    }
    if (color < 0) {   // NCCL_SPLIT_NOCOLOR: this rank joins no child
      *newcomm = nullptr;
      return ncclSuccess;
    }
    std::vector<std::pair<int, int>> members;   // (key, parent rank)
    for (int q = 0; q < n; ++q)
      if (all[(size_t)q * 2] == color) members.emplace_back(all[(size_t)q * 2 + 1], q);
    std::sort(members.begin(), members.end());
    int child_rank = 0;
    for (size_t i = 0; i < members.size(); ++i)
      if (members[i].second == o->rank) child_rank = (int)i;
    int tuple[2] = {color, ordinal};
    const uint64_t h = fnv(tuple, sizeof(tuple), o->id_hash);
    return ownInit(newcomm, (int)members.size(), deriveId(h), child_rank, o->dev, h);
  }
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

static ncclResult_t ownDestroy(OwnComm* o, bool abort) {
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_own.erase(o);
  }
  hlResult_t r = abort ? hlCommAbort(o->hl) : hlCommDestroy(o->hl);
  delete o;
  return toNccl(r);
}

HL_EXPORT ncclResult_t ncclCommDestroy(ncclComm_t comm) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) return ownDestroy(o, false);
  REQUIRE_REAL();
  dropSide(comm, false);
  return g_real.ncclCommDestroy(comm);
}
HL_EXPORT ncclResult_t ncclCommFinalize(ncclComm_t comm) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) return toNccl(hlCommDrain(o->hl));
  REQUIRE_REAL();
  return g_real.ncclCommFinalize ? g_real.ncclCommFinalize(comm) : ncclSuccess;
}
HL_EXPORT ncclResult_t ncclCommAbort(ncclComm_t comm) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) return ownDestroy(o, true);
  REQUIRE_REAL();
  dropSide(comm, true);
  return g_real.ncclCommAbort(comm);
}

HL_EXPORT ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) {
    if (!count) return ncclInvalidArgument;
    *count = o->nranks;
    return ncclSuccess;
  }
  REQUIRE_REAL();
  return g_real.ncclCommCount(comm, count);
}
HL_EXPORT ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) {
    if (!rank) return ncclInvalidArgument;
    *rank = o->rank;
    return ncclSuccess;
  }
  REQUIRE_REAL();
  return g_real.ncclCommUserRank(comm, rank);
}
HL_EXPORT ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) {
    if (!device) return ncclInvalidArgument;
    *device = o->dev;
    return ncclSuccess;
  }
  REQUIRE_REAL();
  return g_real.ncclCommCuDevice(comm, device);
}

HL_EXPORT ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* err) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) {
    if (!err) return ncclInvalidArgument;
    hlResult_t e = hlSuccess;
    hlCommGetAsyncError(o->hl, &e);
    *err = toNccl(e);
    return ncclSuccess;
  }
  REQUIRE_REAL();
  ncclResult_t r = g_real.ncclCommGetAsyncError(comm, err);
  if (r == ncclSuccess && err && *err == ncclSuccess) {
    bool pending = false;
    uint64_t h = 0;
    {
      std::lock_guard<std::mutex> lk(g_mu);
      auto it = g_side.find(comm);
      if (it != g_side.end() && it->second.pending) {
        pending = true;
        h = it->second.id_hash;
        it->second.pending = false;   // one attempt: a failure means pass-through for good
      }
    }
    if (pending) attachSide(comm, h);   // the non-blocking initialisation has just completed
    if (hlComm_t s = sideOf(comm)) {
      hlResult_t e = hlSuccess;
      hlCommGetAsyncError(s, &e);
      if (e != hlSuccess) *err = toNccl(e);
    }
  }
  return r;
}

// ------------------------------------------------------------------ groups
HL_EXPORT ncclResult_t ncclGroupStart() {
  PREPARE();
  if (t_depth++ == 0) t_group_error = ncclSuccess;
  if (!g_standalone && g_real.ncclGroupStart) return g_real.ncclGroupStart();
  return ncclSuccess;
}

HL_EXPORT ncclResult_t ncclGroupEnd() {
  PREPARE();
  if (t_depth <= 0) return ncclInvalidUsage;
  ncclResult_t mine = ncclSuccess;
  if (--t_depth == 0) {
    std::vector<Deferred> q;
    q.swap(t_queue);
    for (const Deferred& d : q) {
      ncclResult_t r = issue(d);
      if (r != ncclSuccess && mine == ncclSuccess) mine = r;
    }
    if (t_group_error != ncclSuccess && mine == ncclSuccess) mine = t_group_error;
  }
  if (!g_standalone && g_real.ncclGroupEnd) {
    ncclResult_t r = g_real.ncclGroupEnd();
    if (r != ncclSuccess) return r;
  }
  return mine;
}

// ------------------------------------------------------------------ collectives
HL_EXPORT ncclResult_t ncclAllReduce(const void* send, void* recv, size_t count, ncclDataType_t t, ncclRedOp_t op, ncclComm_t comm,
                                     cudaStream_t stream) {
  PREPARE();
  hlComm_t s = sideOf(comm);
  if (serve(s, t, count) && opOk(op)) return submit({0, send, recv, count, 0, 0, t, op, 0, s, stream});
  if (g_standalone) return ncclInvalidArgument;
  g_passed++;
  return g_real.ncclAllReduce(send, recv, count, t, op, comm, stream);
}

HL_EXPORT ncclResult_t ncclReduceScatter(const void* send, void* recv, size_t recvcount, ncclDataType_t t, ncclRedOp_t op, ncclComm_t comm,
                                         cudaStream_t stream) {
  PREPARE();
  hlComm_t s = sideOf(comm);
  if (serve(s, t, recvcount) && opOk(op)) return submit({1, send, recv, recvcount, 0, 0, t, op, 0, s, stream});
  if (g_standalone) return ncclInvalidArgument;
  g_passed++;
  return g_real.ncclReduceScatter(send, recv, recvcount, t, op, comm, stream);
}

HL_EXPORT ncclResult_t ncclAllGather(const void* send, void* recv, size_t sendcount, ncclDataType_t t, ncclComm_t comm, cudaStream_t stream) {
  PREPARE();
  hlComm_t s = sideOf(comm);
  if (serve(s, t, sendcount)) return submit({2, send, recv, sendcount, 0, 0, t, ncclSum, 0, s, stream});
  if (g_standalone) return ncclInvalidArgument;
  g_passed++;
  return g_real.ncclAllGather(send, recv, sendcount, t, comm, stream);
}

HL_EXPORT ncclResult_t ncclBroadcast(const void* send, void* recv, size_t count, ncclDataType_t t, int root, ncclComm_t comm,
                                     cudaStream_t stream) {
  PREPARE();
  hlComm_t s = sideOf(comm);
  if (serve(s, t, count)) return submit({3, send, recv, count, 0, 0, t, ncclSum, root, s, stream});
  if (g_standalone) return ncclInvalidArgument;
  g_passed++;
  return g_real.ncclBroadcast(send, recv, count, t, root, comm, stream);
}

HL_EXPORT ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t t, int root, ncclComm_t comm, cudaStream_t stream) {
  return ncclBroadcast(buff, buff, count, t, root, comm, stream);
}

// `count` elements go to (and come from) every peer.
HL_EXPORT ncclResult_t ncclAllToAll(const void* send, void* recv, size_t count, ncclDataType_t t, ncclComm_t comm, cudaStream_t stream) {
  PREPARE();
  hlComm_t s = sideOf(comm);
  if (serve(s, t, count)) return submit({4, send, recv, count, 0, 0, t, ncclSum, 0, s, stream});
  if (g_standalone) return ncclInvalidArgument;
  g_passed++;
  if (g_real.ncclAlltoAll) return g_real.ncclAlltoAll(send, recv, count, t, comm, stream);
  // older NCCL releases have no all-to-all: the documented grouped send / receive form
  int n = 0;
  if (g_real.ncclCommCount(comm, &n) != ncclSuccess || !g_real.ncclSend || !g_real.ncclRecv) return ncclInvalidUsage;
  const size_t es = esize(t);
  g_real.ncclGroupStart();
  for (int q = 0; q < n; ++q) {
    g_real.ncclSend((const char*)send + (size_t)q * count * es, count, t, q, comm, stream);
    g_real.ncclRecv((char*)recv + (size_t)q * count * es, count, t, q, comm, stream);
  }
  return g_real.ncclGroupEnd();
}
HL_EXPORT ncclResult_t ncclAlltoAll(const void* send, void* recv, size_t count, ncclDataType_t t, ncclComm_t comm, cudaStream_t stream) {
  return ncclAllToAll(send, recv, count, t, comm, stream);
}

HL_EXPORT ncclResult_t ncclReduce(const void* send, void* recv, size_t count, ncclDataType_t t, ncclRedOp_t op, int root, ncclComm_t comm,
                                  cudaStream_t stream) {
  PREPARE();
  if (OwnComm* o = asOwn(comm)) {
    if (!typeOk(t) || !opOk(op) || root < 0 || root >= o->nranks) return ncclInvalidArgument;
    return submit({5, send, recv, count, 0, 0, t, op, root, o->hl, stream});
  }
  REQUIRE_REAL();
  g_passed++;
  return g_real.ncclReduce ? g_real.ncclReduce(send, recv, count, t, op, root, comm, stream) : ncclInvalidUsage;
}

// Point-to-point traffic is the real library's: pipeline stages keep using NCCL p2p beside these collectives.
HL_EXPORT ncclResult_t ncclSend(const void* send, size_t count, ncclDataType_t t, int peer, ncclComm_t comm, cudaStream_t stream) {
  PREPARE();
  if (asOwn(comm) || !g_real.ncclSend) {
    t_last_error = "ncclSend: point-to-point transfers need a real NCCL library beside this one";
    return ncclInvalidUsage;
  }
  return g_real.ncclSend(send, count, t, peer, comm, stream);
}
HL_EXPORT ncclResult_t ncclRecv(void* recv, size_t count, ncclDataType_t t, int peer, ncclComm_t comm, cudaStream_t stream) {
  PREPARE();
  if (asOwn(comm) || !g_real.ncclRecv) {
    t_last_error = "ncclRecv: point-to-point transfers need a real NCCL library beside this one";
    return ncclInvalidUsage;
  }
  return g_real.ncclRecv(recv, count, t, peer, comm, stream);
}

// ------------------------------------------------------------------ V-variants
// Rank q contributes recvcounts[q] elements, placed at element rdispls[q] of every receive buffer.
HL_EXPORT ncclResult_t ncclAllGatherV(const void* send, size_t sendcount, void* recv, const size_t* recvcounts, const size_t* rdispls,
                                      ncclDataType_t t, ncclComm_t comm, cudaStream_t stream) {
  PREPARE();
  hlComm_t s = sideOf(comm);
  int n = 0, me = 0;
  if (!s || !typeOk(t) || !recvcounts || !rdispls || hlCommSize(s, &n) != hlSuccess || hlCommRank(s, &me) != hlSuccess) {
    t_last_error = "ncclAllGatherV: needs a communicator served by this library";
    return ncclInvalidUsage;
  }
  const size_t es = esize(t);
  bool uniform = n > 1;
  const size_t stride = n > 1 ? rdispls[1] - rdispls[0] : sendcount;
  for (int q = 0; q < n; ++q) uniform = uniform && recvcounts[q] == sendcount && rdispls[q] == rdispls[0] + (size_t)q * stride;
  if (uniform && stride >= sendcount)
    return submit({6, send, (char*)recv + rdispls[0] * es, sendcount, 0, stride, t, ncclSum, 0, s, stream});
  ncclResult_t out = ncclSuccess;
  for (int q = 0; q < n; ++q) {   // one broadcast per contributor
    if (recvcounts[q] == 0) continue;
    ncclResult_t r = submit({3, q == me ? send : nullptr, (char*)recv + rdispls[q] * es, recvcounts[q], 0, 0, t, ncclSum, q, s, stream});
    if (r != ncclSuccess) out = r;
  }
  return out;
}

// Segment q of `send` (sendcounts[q] elements at element sdispls[q]) is reduced over all ranks and lands on rank q.
HL_EXPORT ncclResult_t ncclReduceScatterV(const void* send, const size_t* sendcounts, const size_t* sdispls, void* recv, size_t recvcount,
                                          ncclDataType_t t, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  PREPARE();
  hlComm_t s = sideOf(comm);
  int n = 0, me = 0;
  if (!s || !typeOk(t) || !opOk(op) || !sendcounts || !sdispls || hlCommSize(s, &n) != hlSuccess || hlCommRank(s, &me) != hlSuccess) {
    t_last_error = "ncclReduceScatterV: needs a communicator served by this library";
    return ncclInvalidUsage;
  }
  const size_t es = esize(t);
  bool uniform = n > 1;
  const size_t stride = n > 1 ? sdispls[1] - sdispls[0] : recvcount;
  for (int q = 0; q < n; ++q) uniform = uniform && sendcounts[q] == recvcount && sdispls[q] == sdispls[0] + (size_t)q * stride;
  if (uniform && stride >= recvcount)
    return submit({7, (const char*)send + sdispls[0] * es, recv, recvcount, stride, 0, t, op, 0, s, stream});
  ncclResult_t out = ncclSuccess;
  for (int q = 0; q < n; ++q) {   // one reduce per owner
    if (sendcounts[q] == 0) continue;
    ncclResult_t r = submit({5, (const char*)send + sdispls[q] * es, recv, sendcounts[q], 0, 0, t, op, q, s, stream});
    if (r != ncclSuccess) out = r;
  }
  return out;
}

HL_EXPORT ncclResult_t ncclAllToAllV(const void* send, const size_t* sendcounts, const size_t* sdispls, void* recv, const size_t* recvcounts,
                                     const size_t* rdispls, ncclDataType_t t, ncclComm_t comm, cudaStream_t stream) {
  PREPARE();
  hlComm_t s = sideOf(comm);
  int n = 0;
  const size_t es = esize(t);
  if (s && es && sendcounts && sdispls && recvcounts && rdispls && hlCommSize(s, &n) == hlSuccess && n > 1) {
    const size_t count = sendcounts[0], ss = sdispls[1] - sdispls[0], rs = rdispls[1] - rdispls[0];
    bool uniform = true;
    for (int q = 0; q < n; ++q)
      uniform = uniform && sendcounts[q] == count && recvcounts[q] == count && sdispls[q] == sdispls[0] + (size_t)q * ss &&
                rdispls[q] == rdispls[0] + (size_t)q * rs;
    if (uniform && ss >= count && rs >= count)
      return submit({8, (const char*)send + sdispls[0] * es, (char*)recv + rdispls[0] * es, count, ss, rs, t, ncclSum, 0, s, stream});
  }
  // ragged exchanges: grouped sends and receives of the real library
  if (g_standalone || !g_real.ncclSend || !g_real.ncclRecv || !es) {
    t_last_error = "ncclAllToAllV: ragged counts need a real NCCL library beside this one";
    return ncclInvalidUsage;
  }
  if (g_real.ncclCommCount(comm, &n) != ncclSuccess) return ncclInvalidArgument;
  g_passed++;
  g_real.ncclGroupStart();
  for (int q = 0; q < n; ++q) {
    if (sendcounts[q]) g_real.ncclSend((const char*)send + sdispls[q] * es, sendcounts[q], t, q, comm, stream);
    if (recvcounts[q]) g_real.ncclRecv((char*)recv + rdispls[q] * es, recvcounts[q], t, q, comm, stream);
  }
  return g_real.ncclGroupEnd();
}

// ------------------------------------------------------------------ memory
// Registered memory of the most recently created communicator of this layer (zero-copy collectives); the real
// library's allocator when interposing, unless HYLINK_NCCL_REGISTERED_ALLOC=1 asks for ours.
HL_EXPORT ncclResult_t ncclMemAlloc(void** ptr, size_t size) {
  PREPARE();
  if (!ptr) return ncclInvalidArgument;
  const bool ours = g_standalone || hl::envBool({"HYLINK_NCCL_REGISTERED_ALLOC"}, false);
  if (!ours && g_real.ncclMemAlloc) return g_real.ncclMemAlloc(ptr, size);
  int dev = 0;
  cudaGetDevice(&dev);
  *ptr = hlTorchAlloc((ssize_t)size, dev, nullptr);
  return *ptr ? ncclSuccess : ncclUnhandledCudaError;
}
HL_EXPORT ncclResult_t ncclMemFree(void* ptr) {
  PREPARE();
  const bool ours = g_standalone || hl::envBool({"HYLINK_NCCL_REGISTERED_ALLOC"}, false);
  if (!ours && g_real.ncclMemFree) return g_real.ncclMemFree(ptr);
  int dev = 0;
  cudaGetDevice(&dev);
  hlTorchFree(ptr, 0, dev, nullptr);
  return ncclSuccess;
}

// Counters for tests and tools: collectives served here vs passed through.
HL_EXPORT void hlNcclShimCounters(uint64_t* intercepted, uint64_t* passed) {
  if (intercepted) *intercepted = g_intercepted.load();
  if (passed) *passed = g_passed.load();
}
HL_EXPORT int hlNcclShimStandalone() {
  loadReal();
  return g_standalone ? 1 : 0;
}

// pnccl* aliases (profiling entry points of the NCCL ABI)
#define HL_ALIAS(name) __attribute__((visibility("default"), alias(#name))) extern decltype(name) p##name
HL_ALIAS(ncclGetVersion);
HL_ALIAS(ncclGetUniqueId);
HL_ALIAS(ncclGetErrorString);
HL_ALIAS(ncclGetLastError);
HL_ALIAS(ncclCommInitRank);
HL_ALIAS(ncclCommInitRankConfig);
HL_ALIAS(ncclCommInitAll);
HL_ALIAS(ncclCommSplit);
HL_ALIAS(ncclCommDestroy);
HL_ALIAS(ncclCommFinalize);
HL_ALIAS(ncclCommAbort);
HL_ALIAS(ncclCommCount);
HL_ALIAS(ncclCommUserRank);
HL_ALIAS(ncclCommCuDevice);
HL_ALIAS(ncclCommGetAsyncError);
HL_ALIAS(ncclGroupStart);
HL_ALIAS(ncclGroupEnd);
HL_ALIAS(ncclAllReduce);
HL_ALIAS(ncclReduceScatter);
HL_ALIAS(ncclAllGather);
HL_ALIAS(ncclBroadcast);
HL_ALIAS(ncclBcast);
HL_ALIAS(ncclReduce);
HL_ALIAS(ncclSend);
HL_ALIAS(ncclRecv);
HL_ALIAS(ncclMemAlloc);
HL_ALIAS(ncclMemFree);
#undef HL_ALIAS

}  // extern "C"
