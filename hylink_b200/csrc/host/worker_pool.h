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
// completion counter) and the Ascend port's range jobs with worker-side
// progress (pcie-ccl-ascend/src/executor/h2h_engine.hpp:22-148): submitRange.
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

// A whole H2H / H2HReduce node handed to the workers at once. A team of `team` workers walks the node slice by slice;
// every member waits by itself until the inputs of slice k are there (the progress words of the nodes it depends on),
// moves its share of the slice, and the member that finishes a slice last publishes the node's own progress word, so
// consumers on other ranks see the slice without the executor thread in between.
// Progress words hold (seq << seq_shift) | slices_done; a word of a later seq counts as complete.
struct RangeJob {
  HostJob::Kind kind = HostJob::Copy;
  char* dst = nullptr;
  const char* a = nullptr;
  const char* b = nullptr;          // Reduce: dst = op(a, b)
  size_t bytes = 0;                 // payload of the node
  size_t slice_bytes = 0;
  int nslices = 1;
  hlDataType_t dtype = hlFloat32;
  hlRedOp_t op = hlSum;
  bool non_temporal = true;
  int numa = 0;
  int team = 1;
  std::atomic<uint64_t>* out = nullptr;
  std::vector<std::atomic<uint64_t>*> deps;
  uint64_t seq = 0;
  int seq_shift = 32;
  const std::atomic<uint32_t>* abort = nullptr;   // non-zero: somebody failed, give up
  uint64_t deadline_ns = 0;                       // steady-clock time after which a wait gives up (0: never)
};

class WorkerPool {
 public:
  // ticket->remaining counts the team members still at work; ticket->failed is set when a wait ran out, the abort
  // word was raised or the reduction is not supported. The node's progress word is the completion record.
  void submitRange(const RangeJob& job, const std::shared_ptr<HostTicket>& ticket);
  uint64_t rangeJobsRun() const { return range_jobs_.load(); }

  // physical_of_logical[i]: machine NUMA node to pin the workers of logical node i to (-1: no pinning)
  WorkerPool(const std::vector<int>& physical_of_logical, int workers_per_node);
  ~WorkerPool();
  // Splits the job into shards of at least 64 KiB; ticket->remaining is raised
  // before the shards become visible to workers.
  void submit(const HostJob& job, const std::shared_ptr<HostTicket>& ticket);
  int workersPerNode() const { return per_node_; }
  uint64_t shardsRun() const { return shards_run_.load(); }

 private:
  struct RangeState {
    RangeJob job;
    std::unique_ptr<std::atomic<int>[]> arrived;   // per slice: members through with it
  };
  struct Shard {
    HostJob job;
    std::shared_ptr<HostTicket> ticket;
    std::shared_ptr<RangeState> range;   // set: this queue entry is one member of a range job
    int member = 0;
  };
  void runRange(RangeState& st, int member, HostTicket& ticket, int node);
  void runShard(Shard& s);
  bool helpWhileWaiting(int node);
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
  std::atomic<uint64_t> range_jobs_{0};
};

}  // namespace hl
