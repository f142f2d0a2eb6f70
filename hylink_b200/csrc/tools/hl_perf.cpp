// hl_perf: stand-alone correctness + bandwidth test of the collectives, in the
// style of the reference's test executables (no test framework, exit code 0 on
// success).
//
//   hl_perf --coll allreduce --ranks 4 --mode threads --device gpu --path nvlink
//   hl_perf --coll reducescatter --ranks 2 --mode fork --device host --strided
//
// Ranks are threads of this process (zeroed unique id, one thread per device)
// or forked children (one process per rank). `--device host` runs the same
// schedules on the host-memory stand-in device, so the tool also works on a
// machine without a GPU.
//
// Rank r fills its input with r+1; a reduction must give n(n+1)/2, gathered
// segment q must hold q+1. Output lines and tables keep the reference's wording
// so that its log post-processors keep working:
//   pcie-ccl-cuda/tests/common/test_common.hpp:127-136,210-220 (size table, percentile table),
//   pcie-ccl-cuda/tests/coll/test_allreduce.cpp:52-113 (fill, expectation, 2 warm-up + 10 timed iterations),
//   pcie-ccl-cuda/tests/common/test_common.hpp:310-315 (strided configurations 75/50/25/0 % on the other transport),
//   multipath-orchestrator/tests/nccl_test/allreduce/allreduce_param.cc:114-154,248-251 (per-iteration lines, verdict).
#include <cuda_runtime.h>
#include <pthread.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "hylink/hylink.h"
#include "pccl/pccl.h"

namespace {

enum Coll { kAllReduce, kAllGather, kReduceScatter, kAllToAll, kBroadcast };
constexpr int kMaxRanks = 8;
constexpr int kMaxIters = 4096;

struct Options {
  Coll coll = kAllReduce;
  int ranks = 2;
  bool fork_mode = false;
  bool host = false;
  hlPath_t path = hlPathAuto;
  size_t lo = 1 << 10, hi = 64 << 20;
  int factor = 2;
  int iters = 10, warmup = 2;
  hlDataType_t dtype = hlFloat32;
  hlRedOp_t op = hlSum;
  bool strided = false;
  bool per_iter = false;
  int root = 0;
};

struct Shared {
  pthread_barrier_t bar;
  hlUniqueId id;
  double ms[kMaxRanks][kMaxIters];
  int ok[kMaxRanks];
  int failed_init[kMaxRanks];
};

size_t parseSize(const char* s) {
  char* end = nullptr;
  double v = strtod(s, &end);
  switch (*end) {
    case 'k': case 'K': v *= 1024.0; break;
    case 'm': case 'M': v *= 1024.0 * 1024; break;
    case 'g': case 'G': v *= 1024.0 * 1024 * 1024; break;
    default: break;
  }
  return (size_t)v;
}

const char* collName(Coll c) {
  static const char* n[] = {"allreduce", "allgather", "reducescatter", "alltoall", "broadcast"};
  return n[c];
}

// ---- element encoding (values are small integers, exact in every type) ----
uint16_t toHalf(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t e = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  const uint32_t m = x & 0x7fffffu;
  if (f == 0.0f) return (uint16_t)sign;
  if (e <= 0) return (uint16_t)sign;
  if (e >= 31) return (uint16_t)(sign | 0x7c00u);
  return (uint16_t)(sign | ((uint32_t)e << 10) | (m >> 13));
}
float fromHalf(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1f, m = h & 0x3ffu;
  uint32_t x;
  if (e == 0) x = sign;  // zero (subnormals are never produced here)
  else if (e == 31) x = sign | 0x7f800000u | (m << 13);
  else x = sign | ((e - 15 + 127) << 23) | (m << 13);
  float f;
  memcpy(&f, &x, 4);
  return f;
}
void put(void* base, size_t i, double v, hlDataType_t t) {
  switch (t) {
    case hlInt8: ((int8_t*)base)[i] = (int8_t)v; break;
    case hlUint8: ((uint8_t*)base)[i] = (uint8_t)v; break;
    case hlInt32: ((int32_t*)base)[i] = (int32_t)v; break;
    case hlUint32: ((uint32_t*)base)[i] = (uint32_t)v; break;
    case hlInt64: ((int64_t*)base)[i] = (int64_t)v; break;
    case hlUint64: ((uint64_t*)base)[i] = (uint64_t)v; break;
    case hlFloat16: ((uint16_t*)base)[i] = toHalf((float)v); break;
    case hlFloat32: ((float*)base)[i] = (float)v; break;
    case hlFloat64: ((double*)base)[i] = v; break;
    case hlBfloat16: {
      float f = (float)v;
      uint32_t x;
      memcpy(&x, &f, 4);
      ((uint16_t*)base)[i] = (uint16_t)(x >> 16);
    } break;
    default: break;
  }
}
double get(const void* base, size_t i, hlDataType_t t) {
  switch (t) {
    case hlInt8: return ((const int8_t*)base)[i];
    case hlUint8: return ((const uint8_t*)base)[i];
    case hlInt32: return ((const int32_t*)base)[i];
    case hlUint32: return ((const uint32_t*)base)[i];
    case hlInt64: return (double)((const int64_t*)base)[i];
    case hlUint64: return (double)((const uint64_t*)base)[i];
    case hlFloat16: return fromHalf(((const uint16_t*)base)[i]);
    case hlFloat32: return ((const float*)base)[i];
    case hlFloat64: return ((const double*)base)[i];
    case hlBfloat16: {
      uint32_t x = (uint32_t)((const uint16_t*)base)[i] << 16;
      float f;
      memcpy(&f, &x, 4);
      return f;
    }
    default: return 0;
  }
}
void fill(void* base, size_t first, size_t n, double v, hlDataType_t t) {
  for (size_t i = 0; i < n; ++i) put(base, first + i, v, t);
}

double reduced(int n, hlRedOp_t op) {
  switch (op) {
    case hlMax: return n;
    case hlMin: return 1;
    case hlAvg: return (n + 1) / 2.0;
    default: return n * (n + 1) / 2.0;
  }
}

// Element counts of the two buffers for a message of `bytes` (the nccl-tests convention: the larger buffer).
void shape(const Options& o, size_t bytes, size_t* per_seg, size_t* send_elems, size_t* recv_elems) {
  const size_t es = hlTypeSize(o.dtype);
  size_t total = std::max<size_t>(bytes / es, (size_t)o.ranks);
  size_t seg = total / (size_t)o.ranks;
  if (seg == 0) seg = 1;
  switch (o.coll) {
    case kAllReduce: case kBroadcast: *per_seg = total; *send_elems = total; *recv_elems = total; break;
    case kAllGather: *per_seg = seg; *send_elems = seg; *recv_elems = seg * o.ranks; break;
    case kReduceScatter: *per_seg = seg; *send_elems = seg * o.ranks; *recv_elems = seg; break;
    case kAllToAll: *per_seg = seg; *send_elems = seg * o.ranks; *recv_elems = seg * o.ranks; break;
  }
}

double busFactor(Coll c, int n) {
  switch (c) {
    case kAllReduce: return 2.0 * (n - 1) / n;
    case kBroadcast: return 1.0;
    default: return (double)(n - 1) / n;
  }
}

struct RankCtx {
  Options o;
  Shared* sh;
  int rank;
  hlComm_t comm = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
};

// An error on one rank leaves the others waiting at the next barrier: end the process at once (threads mode: all
// ranks; fork mode: this child, and the parent then ends the other children).
[[noreturn]] void die() {
  fflush(stdout);
  fflush(stderr);
  _exit(1);
}

#define CK(x)                                                                                  \
  do {                                                                                         \
    hlResult_t _r = (x);                                                                       \
    if (_r != hlSuccess) {                                                                     \
      fprintf(stderr, "rank %d: %s failed: %s (%s)\n", c.rank, #x, hlGetErrorString(_r), hlGetLastError()); \
      die();                                                                                   \
    }                                                                                          \
  } while (0)
#define CKCUDA(x)                                                                              \
  do {                                                                                         \
    cudaError_t _e = (x);                                                                      \
    if (_e != cudaSuccess) {                                                                   \
      fprintf(stderr, "rank %d: %s failed: %s\n", c.rank, #x, cudaGetErrorString(_e));         \
      die();                                                                                   \
    }                                                                                          \
  } while (0)

bool issue(RankCtx& c, const void* send, void* recv, size_t per_seg, size_t stride) {
  const Options& o = c.o;
  hlCallOpts opts;
  memset(&opts, 0, sizeof(opts));
  opts.path = o.path;
  hlStream_t s = (hlStream_t)c.stream;
  if (o.strided) {
    // The first `stride` elements of every segment belong to the other transport: nothing may touch them here.
    pcclComm_t pc = reinterpret_cast<pcclComm_t>(c.comm);
    pcclResult_t r = pcclSuccess;
    const pcclDataType_t dt = (pcclDataType_t)o.dtype;
    const pcclReduceOp_t rop = o.op == hlMax ? pcclReduceMax : (o.op == hlMin ? pcclReduceMin : pcclReduceSum);
    switch (o.coll) {
      case kAllGather: r = pcclAllGatherStridedTyped(send, recv, per_seg, stride, dt, pc, s); break;
      case kReduceScatter: r = pcclReduceScatterStridedTyped(send, recv, per_seg * o.ranks, stride, dt, rop, pc, s); break;
      case kAllToAll: r = pcclAllToAllStridedTyped(send, recv, per_seg * o.ranks, stride, dt, pc, s); break;
      default: fprintf(stderr, "--strided applies to allgather, reducescatter and alltoall\n"); die();
    }
    if (r != pcclSuccess) {
      fprintf(stderr, "rank %d: strided call failed: %s (%s)\n", c.rank, pcclGetErrorString(r), hlGetLastError());
      die();
    }
    return true;
  }
  switch (o.coll) {
    case kAllReduce: CK(hlAllReduceEx(send, recv, per_seg, o.dtype, o.op, &opts, c.comm, s)); break;
    case kAllGather: CK(hlAllGatherEx(send, recv, per_seg, o.dtype, &opts, c.comm, s)); break;
    case kReduceScatter: CK(hlReduceScatterEx(send, recv, per_seg, o.dtype, o.op, &opts, c.comm, s)); break;
    case kAllToAll: CK(hlAllToAllEx(send, recv, per_seg, o.dtype, &opts, c.comm, s)); break;
    case kBroadcast: CK(hlBroadcastEx(send, recv, per_seg, o.dtype, o.root, &opts, c.comm, s)); break;
  }
  return true;
}

bool finish(RankCtx& c) {
  if (!c.o.host) CKCUDA(cudaStreamSynchronize(c.stream));
  CK(hlCommDrain(c.comm));
  return true;
}

// Expected value of element i of the receive buffer (NAN = must be untouched, i.e. still the sentinel).
double expected(const Options& o, int rank, size_t per_seg, size_t stride, size_t i) {
  const int n = o.ranks;
  const size_t seg = i / per_seg, off = i % per_seg;
  switch (o.coll) {
    case kAllReduce: return reduced(n, o.op);
    case kBroadcast: return o.root + 1;
    case kAllGather: return off < stride ? NAN : (double)(seg + 1);
    case kReduceScatter: return off < stride ? NAN : reduced(n, o.op);
    case kAllToAll: return off < stride ? NAN : (double)(seg + 1);
  }
  return 0;
}

bool runRank(RankCtx& c) {
  const Options& o = c.o;
  const size_t es = hlTypeSize(o.dtype);
  const int n = o.ranks;
  if (!o.host) {
    CKCUDA(cudaSetDevice(c.rank));
    CKCUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
    CKCUDA(cudaEventCreate(&c.e0));
    CKCUDA(cudaEventCreate(&c.e1));
  }
  CK(hlCommInitRankDevice(&c.comm, n, c.sh->id, c.rank, o.host ? -2 : c.rank));
  bool all_ok = true;
  std::vector<size_t> sizes;
  for (size_t b = o.lo; b <= o.hi; b *= (size_t)o.factor) sizes.push_back(b);
  // strided runs: share of every segment that the other transport would carry
  const double shares[4] = {0.75, 0.5, 0.25, 0.0};
  const int configs = o.strided ? 4 : 1;
  if (c.rank == 0) {
    printf("# %s ranks=%d mode=%s device=%s dtype=%d iters=%d warmup=%d%s\n", collName(o.coll), n, o.fork_mode ? "fork" : "threads",
           o.host ? "host" : "gpu", (int)o.dtype, o.iters, o.warmup, o.strided ? " strided" : "");
    printf("%12s | %11s | %13s | %13s | %7s\n", "Size", "Avg Lat(ms)", "Alg BW(GB/s)", "Bus BW(GB/s)", "Correct");
  }
  std::vector<std::string> pct_rows;
  for (int cfg = 0; cfg < configs; ++cfg) {
    for (size_t bytes : sizes) {
      size_t per_seg, send_elems, recv_elems;
      shape(o, bytes, &per_seg, &send_elems, &recv_elems);
      size_t stride = 0;
      if (o.strided) stride = std::min(per_seg, (size_t)(per_seg * shares[cfg]) / 32 * 32);
      std::vector<unsigned char> hsend(send_elems * es), hrecv(recv_elems * es);
      fill(hsend.data(), 0, send_elems, c.rank + 1, o.dtype);
      const double sentinel = 99;  // never a legal result for n <= 8
      fill(hrecv.data(), 0, recv_elems, sentinel, o.dtype);
      void *dsend = hsend.data(), *drecv = hrecv.data();
      if (!o.host) {
        CKCUDA(cudaMalloc(&dsend, send_elems * es));
        CKCUDA(cudaMalloc(&drecv, recv_elems * es));
        CKCUDA(cudaMemcpy(dsend, hsend.data(), send_elems * es, cudaMemcpyHostToDevice));
        CKCUDA(cudaMemcpy(drecv, hrecv.data(), recv_elems * es, cudaMemcpyHostToDevice));
      }
      pthread_barrier_wait(&c.sh->bar);
      for (int w = 0; w < o.warmup; ++w) {
        if (!issue(c, dsend, drecv, per_seg, stride) || !finish(c)) return false;
      }
      if (c.rank == 0 && o.per_iter) printf("Warmup done (%u iters)\n", (unsigned)o.warmup);
      // correctness is judged on the state after the warm-up calls (every call rewrites the same result)
      if (!o.host) CKCUDA(cudaMemcpy(hrecv.data(), drecv, recv_elems * es, cudaMemcpyDeviceToHost));
      bool ok = true;
      const size_t step = recv_elems > (16u << 20) ? 61 : 1;
      for (size_t i = 0; i < recv_elems && ok; i += step) {
        const double want = expected(o, c.rank, per_seg, stride, i), got = get(hrecv.data(), i, o.dtype);
        const double ref = std::isnan(want) ? sentinel : want;
        if (std::fabs(got - ref) > 1e-5) {
          fprintf(stderr, "rank %d: size %zu element %zu: got %g, expected %g%s\n", c.rank, bytes, i, got, ref,
                  std::isnan(want) ? " (prefix owned by the other transport was overwritten)" : "");
          ok = false;
        }
      }
      c.sh->ok[c.rank] = ok ? 1 : 0;
      for (int it = 0; it < o.iters; ++it) {
        pthread_barrier_wait(&c.sh->bar);
        double ms = 0;
        if (o.host) {
          const auto t0 = std::chrono::steady_clock::now();
          if (!issue(c, dsend, drecv, per_seg, stride) || !finish(c)) return false;
          ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        } else {
          CKCUDA(cudaEventRecord(c.e0, c.stream));
          if (!issue(c, dsend, drecv, per_seg, stride)) return false;
          CKCUDA(cudaEventRecord(c.e1, c.stream));
          if (!finish(c)) return false;
          float f = 0;
          CKCUDA(cudaEventElapsedTime(&f, c.e0, c.e1));
          ms = f;
        }
        c.sh->ms[c.rank][it] = ms;
      }
      pthread_barrier_wait(&c.sh->bar);
      if (c.rank == 0) {
        std::vector<double> lat(o.iters);
        bool okall = true;
        for (int q = 0; q < n; ++q) okall = okall && c.sh->ok[q];
        for (int it = 0; it < o.iters; ++it) {
          double m = 0;
          for (int q = 0; q < n; ++q) m = std::max(m, c.sh->ms[q][it]);  // a collective is as slow as its slowest rank
          lat[it] = m;
        }
        const size_t moved = std::max(send_elems, recv_elems) * es;
        const size_t active = o.strided ? (size_t)((double)moved * (double)(per_seg - stride) / (double)per_seg) : moved;
        double sum = 0;
        for (int it = 0; it < o.iters; ++it) {
          sum += lat[it];
          if (o.per_iter) printf("iter %u: %.3f ms (%s), bandwidth: %.3f GB/s\n", (unsigned)it, lat[it], o.host ? "host" : "event", active / lat[it] / 1e6);
        }
        const double avg = sum / o.iters, alg = active / avg / 1e6;
        if (o.per_iter) printf("Average bandwidth over %u iters (%s): %.3f GB/s\n", (unsigned)o.iters, o.host ? "host" : "event", alg);
        char tag[32] = "";
        if (o.strided) snprintf(tag, sizeof(tag), " [%d%% other]", (int)(shares[cfg] * 100));
        printf("%12zu | %11.4f | %13.3f | %13.3f | %7s%s\n", bytes, avg, alg, alg * busFactor(o.coll, n), okall ? "yes" : "NO", tag);
        std::sort(lat.begin(), lat.end());
        auto p = [&](double q) { return lat[std::min<size_t>(lat.size() - 1, (size_t)(q * (lat.size() - 1) + 0.5))]; };
        char row[256];
        snprintf(row, sizeof(row), "%12zu | %9.4f | %9.4f | %9.4f | %9.4f | %9.4f | %9.4f%s", bytes, p(0), p(0.5), p(0.9), p(0.95), p(0.99), p(1.0), tag);
        pct_rows.push_back(row);
        all_ok = all_ok && okall;
      }
      pthread_barrier_wait(&c.sh->bar);
      if (!c.sh->ok[c.rank]) all_ok = false;
      if (!o.host) {
        cudaFree(dsend);
        cudaFree(drecv);
      }
    }
  }
  if (c.rank == 0) {
    printf("\nLatency percentiles (ms)\n%12s | %9s | %9s | %9s | %9s | %9s | %9s\n", "Size", "P0", "P50", "P90", "P95", "P99", "P100");
    for (auto& r : pct_rows) printf("%s\n", r.c_str());
  }
  printf("rank %d: %s\n", c.rank, all_ok ? "PASSED" : "FAILED");
  fflush(stdout);
  hlCommDestroy(c.comm);
  if (!o.host) {
    cudaEventDestroy(c.e0);
    cudaEventDestroy(c.e1);
    cudaStreamDestroy(c.stream);
  }
  // rank 0 carries the verdict over all ranks, the others their own
  return all_ok;
}

void usage() {
  fprintf(stderr,
          "usage: hl_perf [--coll allreduce|allgather|reducescatter|alltoall|broadcast] [--ranks N] [--mode threads|fork]\n"
          "               [--device gpu|host] [--path auto|nvlink|pcie|split] [--bytes-from S] [--bytes-to S] [--factor F]\n"
          "               [--iters K] [--warmup W] [--dtype fp32|fp16|bf16|fp64|int8|uint8|int32|uint32|int64|uint64]\n"
          "               [--op sum|max|min|avg] [--root R] [--strided] [--per-iter]\n");
}

bool parse(int argc, char** argv, Options* o) {
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto val = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--coll") {
      std::string v = val();
      if (v == "allreduce") o->coll = kAllReduce;
      else if (v == "allgather") o->coll = kAllGather;
      else if (v == "reducescatter") o->coll = kReduceScatter;
      else if (v == "alltoall") o->coll = kAllToAll;
      else if (v == "broadcast") o->coll = kBroadcast;
      else return false;
    } else if (a == "--ranks") o->ranks = atoi(val());
    else if (a == "--mode") o->fork_mode = std::string(val()) == "fork";
    else if (a == "--device") o->host = std::string(val()) == "host";
    else if (a == "--path") {
      std::string v = val();
      o->path = v == "nvlink" ? hlPathNvlink : v == "pcie" ? hlPathPcie : v == "split" ? hlPathSplit : hlPathAuto;
    } else if (a == "--bytes-from") o->lo = parseSize(val());
    else if (a == "--bytes-to") o->hi = parseSize(val());
    else if (a == "--factor") o->factor = std::max(2, atoi(val()));
    else if (a == "--iters") o->iters = std::min(kMaxIters, std::max(1, atoi(val())));
    else if (a == "--warmup") o->warmup = std::max(1, atoi(val()));
    else if (a == "--root") o->root = atoi(val());
    else if (a == "--strided") o->strided = true;
    else if (a == "--per-iter") o->per_iter = true;
    else if (a == "--dtype") {
      std::string v = val();
      const char* names[] = {"int8", "uint8", "int32", "uint32", "int64", "uint64", "fp16", "fp32", "fp64", "bf16"};
      bool found = false;
      for (int k = 0; k < 10; ++k)
        if (v == names[k]) {
          o->dtype = (hlDataType_t)k;
          found = true;
        }
      if (!found) return false;
    } else if (a == "--op") {
      std::string v = val();
      o->op = v == "max" ? hlMax : v == "min" ? hlMin : v == "avg" ? hlAvg : hlSum;
    } else return false;
  }
  return o->ranks >= 1 && o->ranks <= kMaxRanks && o->lo > 0 && o->hi >= o->lo && o->root >= 0 && o->root < o->ranks;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  if (!parse(argc, argv, &o)) {
    usage();
    return 2;
  }
  Shared* sh = (Shared*)mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
  if (sh == MAP_FAILED) {
    perror("mmap");
    return 2;
  }
  memset(sh, 0, sizeof(*sh));
  pthread_barrierattr_t at;
  pthread_barrierattr_init(&at);
  pthread_barrierattr_setpshared(&at, PTHREAD_PROCESS_SHARED);
  pthread_barrier_init(&sh->bar, &at, (unsigned)o.ranks);
  bool pass = true;
  if (o.fork_mode) {
    if (hlGetUniqueId(&sh->id) != hlSuccess) {
      fprintf(stderr, "hlGetUniqueId failed: %s\n", hlGetLastError());
      return 2;
    }
    std::vector<pid_t> kids;
    for (int r = 0; r < o.ranks; ++r) {
      fflush(stdout);
      pid_t p = fork();
      if (p == 0) {
        RankCtx c;
        c.o = o;
        c.sh = sh;
        c.rank = r;
        const bool ok = runRank(c);
        fflush(stdout);
        _exit(ok ? 0 : 1);
      }
      kids.push_back(p);
    }
    for (size_t left = kids.size(); left > 0; --left) {
      int st = 0;
      const pid_t p = wait(&st);
      if (p < 0) break;
      kids.erase(std::remove(kids.begin(), kids.end(), p), kids.end());
      if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) {
        pass = false;
        for (pid_t q : kids) kill(q, SIGKILL);  // the others would wait for the failed rank at the next barrier
      }
    }
  } else {
    // zeroed id: the ranks are threads of this process
    std::vector<std::thread> th;
    std::vector<int> res(o.ranks, 0);
    for (int r = 0; r < o.ranks; ++r)
      th.emplace_back([&, r] {
        RankCtx c;
        c.o = o;
        c.sh = sh;
        c.rank = r;
        res[r] = runRank(c) ? 1 : 0;
      });
    for (auto& t : th) t.join();
    for (int r = 0; r < o.ranks; ++r) pass = pass && res[r];
  }
  printf(pass ? "Test PASSED.\n" : "Test FAILED.\n");
  return pass ? 0 : 1;
}
