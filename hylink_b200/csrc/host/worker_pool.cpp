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

void WorkerPool::submitRange(const RangeJob& job, const std::shared_ptr<HostTicket>& ticket) {
  const int node = (job.numa >= 0 && job.numa < (int)nodes_.size()) ? job.numa : 0;
  auto st = std::make_shared<RangeState>();
  st->job = job;
  st->job.team = std::max(1, std::min(job.team, per_node_));
  st->job.nslices = std::max(1, job.nslices);
  st->arrived.reset(new std::atomic<int>[(size_t)st->job.nslices]);
  for (int k = 0; k < st->job.nslices; ++k) st->arrived[(size_t)k].store(0, std::memory_order_relaxed);
  ticket->remaining.fetch_add(st->job.team, std::memory_order_acq_rel);
  range_jobs_.fetch_add(1, std::memory_order_relaxed);
  NodeQueue& n = *nodes_[(size_t)node];
  {
    std::lock_guard<std::mutex> lk(n.mu);
    ensureStarted(node);
    for (int m = 0; m < st->job.team; ++m) {
      Shard s;
      s.ticket = ticket;
      s.range = st;
      s.member = m;
      n.q.push_back(std::move(s));
    }
  }
  n.cv.notify_all();
}

void WorkerPool::runRange(RangeState& st, int member, HostTicket& ticket, int node) {
  const RangeJob& j = st.job;
  const uint64_t mask = ((uint64_t)1 << j.seq_shift) - 1;
  auto slicesOf = [&](const std::atomic<uint64_t>* w) -> int {
    const uint64_t v = w->load(std::memory_order_acquire);
    const uint64_t t = v >> j.seq_shift;
    if (t == j.seq) return (int)(v & mask);
    return t > j.seq ? j.nslices : 0;
  };
  const size_t es = j.kind == HostJob::Reduce ? hlTypeSize(j.dtype) : 1;
  for (int k = 0; k < j.nslices; ++k) {
    // inputs of slice k
    uint32_t spins = 0;
    for (;;) {
      bool ready = true;
      for (const std::atomic<uint64_t>* d : j.deps)
        if (slicesOf(d) < k + 1) {
          ready = false;
          break;
        }
      if (ready) break;
      if ((++spins & 15u) == 0 && helpWhileWaiting(node)) continue;
      if ((spins & 255u) == 0) {
        if ((j.abort && j.abort->load(std::memory_order_relaxed)) || (j.deadline_ns && nowNs() > j.deadline_ns) || stop_.load()) {
          ticket.failed.store(1);
          return;
        }
        if (spins > 8192) std::this_thread::yield();
      } else {
        cpuRelax();
      }
    }
    const size_t off = (size_t)k * j.slice_bytes;
    const size_t len = off >= j.bytes ? 0 : std::min(j.slice_bytes, j.bytes - off);
    if (len) {
      // this member's share: 256-byte multiples keep every element type whole
      const size_t part = (((len + (size_t)j.team - 1) / (size_t)j.team) + 255) & ~(size_t)255;
      const size_t lo = std::min(len, (size_t)member * part), hi = std::min(len, lo + part);
      if (hi > lo) {
        if (j.kind == HostJob::Copy) hostCopy(j.dst + off + lo, j.a + off + lo, hi - lo, j.non_temporal);
        else if (!es || !hostReduce(j.dst + off + lo, j.a + off + lo, j.b + off + lo, (hi - lo) / es, j.dtype, j.op)) {
          ticket.failed.store(1);
          return;
        }
        shards_run_.fetch_add(1, std::memory_order_relaxed);
      }
    }
    // the member that completes the slice publishes it; members may be slices apart, so the word only ever grows
    if (st.arrived[(size_t)k].fetch_add(1, std::memory_order_acq_rel) + 1 == j.team) {
      const uint64_t want = (j.seq << j.seq_shift) | (uint64_t)(k + 1);
      uint64_t cur = j.out->load(std::memory_order_relaxed);
      while (cur < want && !j.out->compare_exchange_weak(cur, want, std::memory_order_release, std::memory_order_relaxed)) {
      }
    }
  }
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
    if (s.range) {
      runRange(*s.range, s.member, *s.ticket, node);
      s.ticket->remaining.fetch_sub(1, std::memory_order_acq_rel);
      continue;
    }
    runShard(s);
  }
}

void WorkerPool::runShard(Shard& s) {
  if (s.job.kind == HostJob::Copy) {
    hostCopy(s.job.dst, s.job.a, s.job.bytes, s.job.non_temporal);
  } else {
    const size_t es = hlTypeSize(s.job.dtype);
    if (!es || !hostReduce(s.job.dst, s.job.a, s.job.b, s.job.bytes / es, s.job.dtype, s.job.op)) s.ticket->failed.store(1);
  }
  shards_run_.fetch_add(1, std::memory_order_relaxed);
  s.ticket->remaining.fetch_sub(1, std::memory_order_acq_rel);
}

// A range member that waits for its inputs keeps the queue moving: plain shards never block, and one of them may be
// the very input it waits for (host-memory device: the D2H in front of an H2H runs on the same workers).
bool WorkerPool::helpWhileWaiting(int node) {
  NodeQueue& n = *nodes_[(size_t)node];
  Shard s;
  {
    std::lock_guard<std::mutex> lk(n.mu);
    auto it = n.q.begin();
    while (it != n.q.end() && it->range) ++it;
    if (it == n.q.end()) return false;
    s = std::move(*it);
    n.q.erase(it);
  }
  runShard(s);
  return true;
}

}  // namespace hl
