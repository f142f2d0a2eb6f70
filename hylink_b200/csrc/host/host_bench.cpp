// Host copy / reduce micro-benchmark through the NUMA worker pool: how the
// rate of a staging-buffer copy (or a three-address reduction) scales with the
// number of workers, inside one NUMA node and across two.
//
// Parity: pcie-ccl-cuda/tests/dev/test_h2h.cpp (1-16 threads, intra / cross
// NUMA, copy and reduce). Here the measured code is the pool the executor
// itself uses, not a separate test harness.
#include <sys/mman.h>

#include <chrono>
#include <cstring>
#include <memory>
#include <thread>

#include "core/core.h"
#include "host/topology.h"
#include "host/worker_pool.h"
#include "hylink/hylink_ext.h"

using namespace hl;

extern "C" hlResult_t hlHostBench(int reduce, size_t bytes, int threads, int src_numa, int dst_numa, int iters, int non_temporal,
                                  int dtype, double* gbs, double* best_gbs) {
  if (!gbs || bytes < 4096 || threads < 1 || threads > 64 || iters < 1) return fail(hlInvalidArgument, "hlHostBench: bad arguments");
  const size_t es = hlTypeSize((hlDataType_t)dtype);
  if (!es) return fail(hlInvalidArgument, "hlHostBench: unknown data type");
  bytes = bytes / 4096 * 4096;
  auto map = [&](int node) -> void* {
    void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (p == MAP_FAILED) return nullptr;
    if (node >= 0) bindMemoryToNumaNode(p, bytes, node);  // best effort: containers may refuse
    memset(p, 1, bytes);                                   // touch: pages are placed now
    return p;
  };
  void* a = map(src_numa);
  void* b = reduce ? map(src_numa) : nullptr;
  void* d = map(dst_numa);
  if (!a || !d || (reduce && !b)) {
    if (a) munmap(a, bytes);
    if (b) munmap(b, bytes);
    if (d) munmap(d, bytes);
    return fail(hlSystemError, "hlHostBench: cannot map %zu bytes", bytes);
  }
  double sum = 0, best = 0;
  {
    WorkerPool pool(std::vector<int>{dst_numa}, threads);  // workers sit next to the destination, as in the executor
    HostJob job;
    job.kind = reduce ? HostJob::Reduce : HostJob::Copy;
    job.dst = d;
    job.a = a;
    job.b = b;
    job.bytes = bytes;
    job.dtype = (hlDataType_t)dtype;
    job.op = hlSum;
    job.non_temporal = non_temporal != 0;
    job.numa = 0;
    for (int it = -1; it < iters; ++it) {  // iteration -1 warms the pool up
      auto ticket = std::make_shared<HostTicket>();
      const auto t0 = std::chrono::steady_clock::now();
      pool.submit(job, ticket);
      while (!ticket->done()) std::this_thread::yield();
      const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
      if (it < 0) continue;
      const double r = (double)bytes / s / 1e9;
      sum += r;
      if (r > best) best = r;
    }
  }
  munmap(a, bytes);
  if (b) munmap(b, bytes);
  munmap(d, bytes);
  *gbs = sum / iters;
  if (best_gbs) *best_gbs = best;
  return hlSuccess;
}

extern "C" int hlHostNumaNodes(void) { return numaNodeCount(); }
