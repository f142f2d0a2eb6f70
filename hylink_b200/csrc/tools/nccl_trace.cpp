// libhylink_nccltrace.so: an LD_PRELOAD tracer that writes one JSON line per
// NCCL call (name, wall time, duration of the host call, element count, type,
// operator, root/peer, communicator and stream handles, and whether the stream
// was being captured into a CUDA graph) and forwards the call to the next
// provider of the symbol — the real library, or this project's symbol layer
// when both are preloaded. Output: HYLINK_NCCL_TRACE_FILE ("%p" = pid), default
// nccl_trace.<pid>.jsonl. The companion parser is
// hylink_b200/utils/nccl_trace_parse.py.
//
// Parity: pcie-ccl-cuda/tools/nccl_full_trace_intercept.c:66-605.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace {
std::mutex g_mu;
FILE* g_out = nullptr;
std::atomic<uint64_t> g_seq{0};

double wallSeconds() {
  return std::chrono::duration<double>(std::chrono::system_clock::now().time_since_epoch()).count();
}

FILE* out() {
  if (g_out) return g_out;
  std::string path = getenv("HYLINK_NCCL_TRACE_FILE") ? getenv("HYLINK_NCCL_TRACE_FILE") : "nccl_trace.%p.jsonl";
  size_t k = path.find("%p");
  if (k != std::string::npos) path.replace(k, 2, std::to_string((int)getpid()));
  g_out = fopen(path.c_str(), "a");
  if (!g_out) g_out = stderr;
  return g_out;
}

int capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return st == cudaStreamCaptureStatusActive ? 1 : 0;
}

template <typename F> F nextSym(const char* name) {
  void* p = dlsym(RTLD_NEXT, name);
  if (!p) {
    static void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (h) p = dlsym(h, name);
  }
  return reinterpret_cast<F>(p);
}

void record(const char* name, double t0, double dur, long long count, int dtype, int op, int peer, const void* comm,
            const void* stream, int cap, int rc) {
  std::lock_guard<std::mutex> lk(g_mu);
  fprintf(out(),
          "{\"seq\":%llu,\"pid\":%d,\"call\":\"%s\",\"t\":%.6f,\"host_us\":%.2f,\"count\":%lld,\"dtype\":%d,\"op\":%d,\"peer\":%d,"
          "\"comm\":\"%p\",\"stream\":\"%p\",\"capturing\":%d,\"rc\":%d}\n",
          (unsigned long long)g_seq++, (int)getpid(), name, t0, dur * 1e6, count, dtype, op, peer, comm, stream, cap, rc);
  fflush(out());
}
}  // namespace

#define TRACE_COLL(NAME, COUNT, DTYPE, OP, PEER, COMM, STREAM, CALL)                         \
  static auto fn = nextSym<decltype(&::NAME)>(#NAME);                                        \
  if (!fn) return ncclSystemError;                                                           \
  const int cap = capturing(STREAM);                                                         \
  const double t0 = wallSeconds();                                                           \
  ncclResult_t rc = CALL;                                                                    \
  record(#NAME, t0, wallSeconds() - t0, (long long)(COUNT), (int)(DTYPE), (int)(OP), PEER, COMM, STREAM, cap, (int)rc); \
  return rc

extern "C" {
#define EXPORT __attribute__((visibility("default")))

EXPORT ncclResult_t ncclAllReduce(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  TRACE_COLL(ncclAllReduce, n, t, op, -1, c, st, fn(s, r, n, t, op, c, st));
}
EXPORT ncclResult_t ncclReduceScatter(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  TRACE_COLL(ncclReduceScatter, n, t, op, -1, c, st, fn(s, r, n, t, op, c, st));
}
EXPORT ncclResult_t ncclAllGather(const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st) {
  TRACE_COLL(ncclAllGather, n, t, -1, -1, c, st, fn(s, r, n, t, c, st));
}
EXPORT ncclResult_t ncclBroadcast(const void* s, void* r, size_t n, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st) {
  TRACE_COLL(ncclBroadcast, n, t, -1, root, c, st, fn(s, r, n, t, root, c, st));
}
EXPORT ncclResult_t ncclReduce(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, int root, ncclComm_t c, cudaStream_t st) {
  TRACE_COLL(ncclReduce, n, t, op, root, c, st, fn(s, r, n, t, op, root, c, st));
}
EXPORT ncclResult_t ncclSend(const void* s, size_t n, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t st) {
  TRACE_COLL(ncclSend, n, t, -1, peer, c, st, fn(s, n, t, peer, c, st));
}
EXPORT ncclResult_t ncclRecv(void* r, size_t n, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t st) {
  TRACE_COLL(ncclRecv, n, t, -1, peer, c, st, fn(r, n, t, peer, c, st));
}
EXPORT ncclResult_t ncclGroupStart(void) {
  static auto fn = nextSym<decltype(&::ncclGroupStart)>("ncclGroupStart");
  if (!fn) return ncclSystemError;
  const double t0 = wallSeconds();
  ncclResult_t rc = fn();
  record("ncclGroupStart", t0, wallSeconds() - t0, 0, -1, -1, -1, nullptr, nullptr, -1, (int)rc);
  return rc;
}
EXPORT ncclResult_t ncclGroupEnd(void) {
  static auto fn = nextSym<decltype(&::ncclGroupEnd)>("ncclGroupEnd");
  if (!fn) return ncclSystemError;
  const double t0 = wallSeconds();
  ncclResult_t rc = fn();
  record("ncclGroupEnd", t0, wallSeconds() - t0, 0, -1, -1, -1, nullptr, nullptr, -1, (int)rc);
  return rc;
}
EXPORT ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
  static auto fn = nextSym<decltype(&::ncclCommInitRank)>("ncclCommInitRank");
  if (!fn) return ncclSystemError;
  const double t0 = wallSeconds();
  ncclResult_t rc = fn(comm, nranks, id, rank);
  record("ncclCommInitRank", t0, wallSeconds() - t0, nranks, -1, -1, rank, comm ? *comm : nullptr, nullptr, -1, (int)rc);
  return rc;
}
EXPORT ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, ncclConfig_t* cfg) {
  static auto fn = nextSym<decltype(&::ncclCommInitRankConfig)>("ncclCommInitRankConfig");
  if (!fn) return ncclSystemError;
  const double t0 = wallSeconds();
  ncclResult_t rc = fn(comm, nranks, id, rank, cfg);
  record("ncclCommInitRankConfig", t0, wallSeconds() - t0, nranks, -1, -1, rank, comm ? *comm : nullptr, nullptr, -1, (int)rc);
  return rc;
}
EXPORT ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* cfg) {
  static auto fn = nextSym<decltype(&::ncclCommSplit)>("ncclCommSplit");
  if (!fn) return ncclSystemError;
  const double t0 = wallSeconds();
  ncclResult_t rc = fn(comm, color, key, newcomm, cfg);
  record("ncclCommSplit", t0, wallSeconds() - t0, color, -1, -1, key, comm, nullptr, -1, (int)rc);
  return rc;
}
EXPORT ncclResult_t ncclCommDestroy(ncclComm_t comm) {
  static auto fn = nextSym<decltype(&::ncclCommDestroy)>("ncclCommDestroy");
  if (!fn) return ncclSystemError;
  const double t0 = wallSeconds();
  ncclResult_t rc = fn(comm);
  record("ncclCommDestroy", t0, wallSeconds() - t0, 0, -1, -1, -1, comm, nullptr, -1, (int)rc);
  return rc;
}
EXPORT ncclResult_t ncclCommAbort(ncclComm_t comm) {
  static auto fn = nextSym<decltype(&::ncclCommAbort)>("ncclCommAbort");
  if (!fn) return ncclSystemError;
  const double t0 = wallSeconds();
  ncclResult_t rc = fn(comm);
  record("ncclCommAbort", t0, wallSeconds() - t0, 0, -1, -1, -1, comm, nullptr, -1, (int)rc);
  return rc;
}
}  // extern "C"
