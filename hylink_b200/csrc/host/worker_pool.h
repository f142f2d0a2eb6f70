// NUMA-pinned worker threads for host-side copies and reductions.
//
// The executor hands a slice of an H2H / H2HReduce node (or, with the
// host-memory device, any copy) to the pool as one job; the job is cut into
// shards that the workers of the destination's NUMA node pick up; a ticket
// counts the shards still running so the executor can poll for completion
// without blocking.
//
// Parity: pcie-ccl-cuda/src/executor/h2h_engine.cpp:170-301 (16 lazily spawned
// workers per destination NUMA node, 16 shards per sub-chunk, shared atomic
// completion counter) and the Ascend port's range jobs
// (pcie-ccl-ascend/src/executor/h2h_engine.hpp:22-148).
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "hylink/hylink.h"

namespace hl {

struct HostTicket {
  std::atomic<int> remaining{0};
  std::atomic<int> failed{0};
  bool done() const { return remaining.load(std::memory_order_acquire) == 0; }
};

struct HostJob {
  enum Kind { Copy, Reduce } kind = Copy;
  void* dst = nullptr;
  const void* a = nullptr;
  const void* b = nullptr;   // Reduce: dst = op(a, b)
  size_t bytes = 0;
  hlDataType_t dtype = hlFloat32;
  hlRedOp_t op = hlSum;
  bool non_temporal = true;
  int numa = 0;              // logical NUMA node whose workers should run it
};

class WorkerPool {
 public:
  // physical_of_logical[i]: machine NUMA node to pin the workers of logical node i to (-1: no pinning)
  WorkerPool(const std::vector<int>& physical_of_logical, int workers_per_node);
  ~WorkerPool();
  // Splits the job into shards of at least 64 KiB; ticket->remaining is raised
  // before the shards become visible to workers.
  void submit(const HostJob& job, const std::shared_ptr<HostTicket>& ticket);
  int workersPerNode() const { return per_node_; }
  uint64_t shardsRun() const { return shards_run_.load(); }

 private:
  struct Shard {
    HostJob job;
    std::shared_ptr<HostTicket> ticket;
  };
  struct NodeQueue {
    std::mutex mu;
    std::condition_variable cv;
    std::deque<Shard> q;
    std::vector<std::thread> threads;
    bool started = false;
  };
  void ensureStarted(int node);
  void loop(int node);
  std::vector<int> phys_;
  int per_node_;
  std::vector<std::unique_ptr<NodeQueue>> nodes_;
  std::atomic<bool> stop_{false};
  std::atomic<uint64_t> shards_run_{0};
};

}  // namespace hl
