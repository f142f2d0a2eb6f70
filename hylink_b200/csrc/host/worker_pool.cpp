#include "host/worker_pool.h"

#include <algorithm>

#include "core/core.h"
#include "host/host_simd.h"
#include "host/topology.h"

namespace hl {

WorkerPool::WorkerPool(const std::vector<int>& physical_of_logical, int workers_per_node) : phys_(physical_of_logical) {
  if (phys_.empty()) phys_.push_back(-1);
  int hw = (int)std::thread::hardware_concurrency();
  if (hw < 1) hw = 4;
  per_node_ = workers_per_node > 0 ? workers_per_node : std::max(2, std::min(16, hw / (2 * (int)phys_.size())));
  for (size_t i = 0; i < phys_.size(); ++i) nodes_.emplace_back(new NodeQueue());
}

WorkerPool::~WorkerPool() {
  stop_.store(true);
  for (auto& n : nodes_) {
    {
      std::lock_guard<std::mutex> lk(n->mu);
    }
    n->cv.notify_all();
    for (auto& t : n->threads) t.join();
  }
}

void WorkerPool::ensureStarted(int node) {
  NodeQueue& n = *nodes_[(size_t)node];
  if (n.started) return;
  n.started = true;  // caller holds n.mu
  for (int i = 0; i < per_node_; ++i) n.threads.emplace_back([this, node] { loop(node); });
}

void WorkerPool::submit(const HostJob& job, const std::shared_ptr<HostTicket>& ticket) {
  const int node = (job.numa >= 0 && job.numa < (int)nodes_.size()) ? job.numa : 0;
  const size_t es = job.kind == HostJob::Reduce ? hlTypeSize(job.dtype) : 1;
  const size_t min_shard = 64u << 10;
  size_t shards = std::min<size_t>((size_t)per_node_, std::max<size_t>(1, job.bytes / min_shard));
  size_t per = ((job.bytes / shards) + 255) & ~(size_t)255;  // 256-byte multiples keep every element type whole
  if (per == 0) per = job.bytes;
  std::vector<Shard> cut;
  for (size_t off = 0; off < job.bytes; off += per) {
    Shard s;
    s.job = job;
    s.job.dst = (char*)job.dst + off;
    s.job.a = (const char*)job.a + off;
    if (job.b) s.job.b = (const char*)job.b + off;
    s.job.bytes = std::min(per, job.bytes - off);
    s.ticket = ticket;
    cut.push_back(std::move(s));
  }
  (void)es;
  if (cut.empty()) return;
  ticket->remaining.fetch_add((int)cut.size(), std::memory_order_acq_rel);
  NodeQueue& n = *nodes_[(size_t)node];
  {
    std::lock_guard<std::mutex> lk(n.mu);
    ensureStarted(node);
    for (auto& s : cut) n.q.push_back(std::move(s));
  }
  if (cut.size() > 1) n.cv.notify_all();
  else n.cv.notify_one();
}

void WorkerPool::loop(int node) {
  if (phys_[(size_t)node] >= 0) pinThreadToNumaNode(phys_[(size_t)node]);
  NodeQueue& n = *nodes_[(size_t)node];
  for (;;) {
    Shard s;
    {
      std::unique_lock<std::mutex> lk(n.mu);
      n.cv.wait(lk, [&] { return stop_.load() || !n.q.empty(); });
      if (n.q.empty()) {
        if (stop_.load()) return;
        continue;
      }
      s = std::move(n.q.front());
      n.q.pop_front();
    }
    if (s.job.kind == HostJob::Copy) {
      hostCopy(s.job.dst, s.job.a, s.job.bytes, s.job.non_temporal);
    } else {
      const size_t es = hlTypeSize(s.job.dtype);
      if (!es || !hostReduce(s.job.dst, s.job.a, s.job.b, s.job.bytes / es, s.job.dtype, s.job.op)) s.ticket->failed.store(1);
    }
    shards_run_.fetch_add(1, std::memory_order_relaxed);
    s.ticket->remaining.fetch_sub(1, std::memory_order_acq_rel);
  }
}

}  // namespace hl
