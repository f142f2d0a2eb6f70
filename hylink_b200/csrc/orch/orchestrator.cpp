// Multipath orchestrator: fork / join of one collective over both transports
// and the feedback loop that retunes the split.
//
// Launch path of a forked call (no host synchronisation, no cross-rank
// rendezvous in steady state):
//   user stream:  ev_fork | t0 | NVLink kernel on the prefix | t1 | wait(ev_join) | host callback
//   pcie stream:  wait(ev_fork) | t2 | doorbell + CPU-driven schedule on the suffix | t3 | ev_join
// The NVLink kernels take segment strides and a prefix length natively and the
// PCIe schedules take the complementary stride, so neither side packs, stages
// or merges anything.
//
// Feedback without a barrier: every forked call has an index that is the same
// on all ranks. When call c completes, each rank's timer thread writes
// (fast time, PCIe time, bytes, ok) into slot c of its ring in the shared
// control block. Before launching call j every rank folds in — in call order —
// the statistics of all calls up to j - LAG, taking the maximum over ranks,
// and feeds its own copy of the controller. All ranks therefore apply the
// same updates at the same call index and compute the same split for call j,
// which is what keeps the two halves of the collective aligned across ranks.
// A rank only blocks when it runs more than LAG forked calls ahead of the
// slowest rank's completions.
//
// Parity: multipath-orchestrator/libampccl/core/virtual_collective.h:66-146,
// 187-848 (prepare, fork, join, per-op splits), core/shm_store.cc:282-461
// (cross-rank aggregation: max over ranks; there rank 0 decides and all ranks
// rendezvous twice per call), core/stream_sync.cc:108-299 and
// stream_host_callback.cc:16-43 (completion callback, timers queried off the
// callback thread), core/domain.h:22-182 (per-communicator state).
#include "orch/orchestrator.h"

#include <cuda_runtime.h>

#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>

#include "api/comm.h"
#include "core/trace.h"
#include "hal/cuda_driver.h"
#include "orch/controller.h"
#include "pcie/pcie_path.h"

namespace hl {

namespace {
constexpr int kRing = 64;

struct StatSlot {
  std::atomic<uint64_t> call_idx;  // published last (release)
  double fast_s, pcie_s;
  uint64_t fast_bytes, pcie_bytes;
  uint32_t fast_ok, pcie_ok;
  char pad[16];
};
struct OrchShared {
  StatSlot slots[kMaxRanks][kRing];
};

struct CallRecord {
  uint64_t idx = 0;
  orch::OpKey key;
  orch::Plan plan;
  size_t key_bytes = 0;   // bytes the op key was built from
  size_t alg_bytes = 0;   // bytes of the whole collective for algbw
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};  // fast start/end, pcie start/end
  bool timed = false;
};
}  // namespace

class OrchImpl {
 public:
  OrchImpl(hlComm* c, void* area) : comm_(c), shared_((OrchShared*)area), ctl_(Config::get().algo, c->nranks) {}
  ~OrchImpl();
  hlResult_t init();
  bool shouldSplit(size_t bytes) const;

  struct Split {
    uint64_t idx;
    orch::Plan plan;
    CallRecord* rec;
  };
  hlResult_t begin(int op, size_t key_bytes, size_t alg_bytes, int dtype, size_t elem, Split* out);
  hlResult_t fork(const Split& s, cudaStream_t user);
  hlResult_t join(const Split& s, cudaStream_t user, bool fast_ok, bool pcie_ok);
  cudaStream_t pcieStream() const { return pcie_stream_; }
  void fillStats(hlCommStats* out) const;
  std::string dumpTuning() const { return ctl_.dumpJson(); }
  hlResult_t loadTuning(const char* json) { return ctl_.loadJson(json) ? hlSuccess : fail(hlInvalidArgument, "tuning table: malformed JSON"); }
  void publishImmediate(uint64_t idx, const orch::Plan& plan);
  hlComm* comm() const { return comm_; }

 private:
  hlResult_t applyStatsUpTo(int64_t upto);
  void timerMain();
  static void CUDART_CB hostCallback(void* p);
  struct Done {
    OrchImpl* self;
    uint64_t idx;
    bool fast_ok, pcie_ok;
  };
  hlComm* comm_;
  OrchShared* shared_;
  orch::AdaptiveController ctl_;
  orch::PlannerLimits lim_;
  int lag_ = 2;
  uint64_t next_idx_ = 1;
  int64_t applied_ = 0;
  CallRecord ring_[kRing];
  cudaStream_t pcie_stream_ = nullptr;
  cudaStream_t notify_stream_ = nullptr;  // carries the completion callbacks, so that they never sit in the caller's stream
  cudaEvent_t ev_fork_[kRing] = {nullptr}, ev_join_[kRing] = {nullptr};
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Done*> done_q_;
  bool stop_ = false;
  std::thread timer_;
  double last_alpha_ = 0, last_fast_ms_ = 0, last_pcie_ms_ = 0;
  bool bw_log_ = false;
  uint64_t logged_ = 0;
  double sum_busbw_ = 0;
};

hlResult_t OrchImpl::init() {
  const Config& cfg = Config::get();
  lim_.min_msg_bytes = comm_->nranks >= 8 ? cfg.min_msg_bytes_8 : cfg.min_msg_bytes;
  lim_.min_part_bytes = cfg.min_chunk_bytes;
  lag_ = (int)std::min<long long>(kRing / 2, std::max<long long>(1, envInt({"HYLINK_ORCH_LAG"}, 2)));
  bw_log_ = cfg.avg_bw_log || logLevel() >= kLogInfo;
  HL_CUDA(cudaSetDevice(comm_->device));
  int lo = 0, hi = 0;
  HL_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  HL_CUDA(cudaStreamCreateWithPriority(&pcie_stream_, cudaStreamNonBlocking, hi));
  HL_CUDA(cudaStreamCreateWithFlags(&notify_stream_, cudaStreamNonBlocking));
  for (int i = 0; i < kRing; ++i) {
    for (int k = 0; k < 4; ++k) HL_CUDA(cudaEventCreate(&ring_[i].ev[k]));
    HL_CUDA(cudaEventCreateWithFlags(&ev_fork_[i], cudaEventDisableTiming));
    HL_CUDA(cudaEventCreateWithFlags(&ev_join_[i], cudaEventDisableTiming));
  }
  for (int s = 0; s < kRing; ++s) shared_->slots[comm_->rank][s].call_idx.store(0);
  timer_ = std::thread([this] { timerMain(); });
  return hlSuccess;
}

OrchImpl::~OrchImpl() {
  cudaSetDevice(comm_->device);
  cudaDeviceSynchronize();
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (timer_.joinable()) timer_.join();
  for (int i = 0; i < kRing; ++i) {
    for (int k = 0; k < 4; ++k)
      if (ring_[i].ev[k]) cudaEventDestroy(ring_[i].ev[k]);
    if (ev_fork_[i]) cudaEventDestroy(ev_fork_[i]);
    if (ev_join_[i]) cudaEventDestroy(ev_join_[i]);
  }
  if (pcie_stream_) cudaStreamDestroy(pcie_stream_);
  if (notify_stream_) cudaStreamDestroy(notify_stream_);
  if (Config::get().avg_bw_log && comm_->rank == 0 && logged_)
    logAlways("average busbw over %llu forked collectives: %.3f GB/s", (unsigned long long)logged_, sum_busbw_ / (double)logged_);
}

bool OrchImpl::shouldSplit(size_t bytes) const { return bytes >= lim_.min_msg_bytes; }

hlResult_t OrchImpl::applyStatsUpTo(int64_t upto) {
  const int n = comm_->nranks;
  const uint64_t limit = (uint64_t)Config::get().executor_timeout_ms * 1000000ull;
  while (applied_ < upto) {
    const uint64_t c = (uint64_t)(applied_ + 1);
    const int slot = (int)(c % kRing);
    orch::ExecStat agg;
    const uint64_t t0 = nowNs();
    for (int q = 0; q < n; ++q) {
      StatSlot& s = shared_->slots[q][slot];
      uint32_t spins = 0;
      while (s.call_idx.load(std::memory_order_acquire) < c) {
        if ((++spins & 1023u) == 0) {
          if (comm_->bs->anyFailed()) return fail(hlRemoteError, "orchestrator: a peer failed while call %llu was in flight", (unsigned long long)c);
          if (nowNs() - t0 > limit) return fail(hlTimeout, "orchestrator: statistics of call %llu from rank %d never arrived", (unsigned long long)c, q);
          std::this_thread::yield();
        } else {
          cpuRelax();
        }
      }
      agg.fast_time = std::max(agg.fast_time, s.fast_s);
      agg.pcie_time = std::max(agg.pcie_time, s.pcie_s);
      agg.fast_bytes = s.fast_bytes;
      agg.pcie_bytes = s.pcie_bytes;
      agg.fast_ok = agg.fast_ok && s.fast_ok;
      agg.pcie_ok = agg.pcie_ok && s.pcie_ok;
    }
    CallRecord& rec = ring_[slot];
    ctl_.update(rec.key, agg);
    if (agg.pcie_bytes) {
      last_fast_ms_ = agg.fast_time * 1e3;
      last_pcie_ms_ = agg.pcie_time * 1e3;
    }
    if (bw_log_ && comm_->rank == 0 && agg.pcie_bytes) {
      const double t = std::max(agg.fast_time, agg.pcie_time);
      const double total = (double)(agg.fast_bytes + agg.pcie_bytes);
      const double factor = orch::busFactor(rec.key.op, n);
      const double algbw = t > 0 ? (double)rec.alg_bytes / t / 1e9 : 0;
      logAlways("(max) fast_time=%lfs", agg.fast_time);
      logAlways("(max) pcie_time=%lfs", agg.pcie_time);
      logAlways("aggregate op=%s op_key_bytes=%zu base_bytes=%zu alg_bytes=%.0f n=%d | fast_bytes=%zu pcie_bytes=%zu split_fast=%.4f split_pcie=%.4f | "
                "fast_bw(GB/s,decimal)=%.3f pcie_bw(GB/s,decimal)=%.3f | algbw(GB/s,decimal)=%.3f busbw(GB/s,decimal)=%.3f bus_factor=%.4f",
                orch::opKindName(rec.key.op), rec.key_bytes, rec.key_bytes, (double)rec.alg_bytes, n, (size_t)agg.fast_bytes,
                (size_t)agg.pcie_bytes, total > 0 ? agg.fast_bytes / total : 0, total > 0 ? agg.pcie_bytes / total : 0,
                agg.fastBw() / 1e9, agg.pcieBw() / 1e9, algbw, algbw * factor, factor);
      logAlways("Total bw is %lf GB/s", algbw * factor);
      sum_busbw_ += algbw * factor;
      ++logged_;
    }
    ++applied_;
  }
  return hlSuccess;
}

hlResult_t OrchImpl::begin(int op, size_t key_bytes, size_t alg_bytes, int dtype, size_t elem, Split* out) {
  const uint64_t idx = next_idx_++;
  HL_CHECK(applyStatsUpTo((int64_t)idx - lag_));
  CallRecord& rec = ring_[idx % kRing];
  rec.idx = idx;
  rec.key = orch::makeOpKey(op, key_bytes, dtype, comm_->nranks, 0);
  rec.key_bytes = key_bytes;
  rec.alg_bytes = alg_bytes;
  const double alpha = ctl_.suggestAlpha(rec.key);
  rec.plan = orch::createPlan(key_bytes, alpha, ctl_.usePcie(rec.key), elem, lim_);
  rec.timed = false;
  last_alpha_ = key_bytes ? (double)rec.plan.pcie_bytes / (double)key_bytes : 0;
  comm_->stats.last_alpha = last_alpha_;
  HL_DBG("[Rank %d] Before %s, bytes=%zu bucket=%d dtype=%d nranks=%d alpha=%.4f, plan.use_pcie=%d plan.pcie_bytes=%zu plan.fast_bytes=%zu",
         comm_->rank, orch::opKindName(op), key_bytes, rec.key.bucket, dtype, comm_->nranks, alpha, (int)rec.plan.use_pcie,
         rec.plan.pcie_bytes, rec.plan.fast_bytes);
  out->idx = idx;
  out->plan = rec.plan;
  out->rec = &rec;
  return hlSuccess;
}

void OrchImpl::publishImmediate(uint64_t idx, const orch::Plan& plan) {
  StatSlot& s = shared_->slots[comm_->rank][idx % kRing];
  s.fast_s = 0;
  s.pcie_s = 0;
  s.fast_bytes = plan.fast_bytes;
  s.pcie_bytes = 0;
  s.fast_ok = 1;
  s.pcie_ok = 1;
  s.call_idx.store(idx, std::memory_order_release);
}

hlResult_t OrchImpl::fork(const Split& s, cudaStream_t user) {
  TraceScope range("orch", "fork", comm_->rank);
  const int slot = (int)(s.idx % kRing);
  HL_CUDA(cudaEventRecord(ev_fork_[slot], user));
  HL_CUDA(cudaStreamWaitEvent(pcie_stream_, ev_fork_[slot], 0));
  HL_CUDA(cudaEventRecord(s.rec->ev[0], user));
  HL_CUDA(cudaEventRecord(s.rec->ev[2], pcie_stream_));
  return hlSuccess;
}

void CUDART_CB OrchImpl::hostCallback(void* p) {
  // Runs on a driver thread: no CUDA calls here, hand over to the timer thread.
  Done* d = (Done*)p;
  {
    std::lock_guard<std::mutex> lk(d->self->mu_);
    d->self->done_q_.push_back(d);
  }
  d->self->cv_.notify_one();
}

hlResult_t OrchImpl::join(const Split& s, cudaStream_t user, bool fast_ok, bool pcie_ok) {
  TraceScope range("orch", "join", comm_->rank);
  const int slot = (int)(s.idx % kRing);
  HL_CUDA(cudaEventRecord(s.rec->ev[1], user));
  HL_CUDA(cudaEventRecord(s.rec->ev[3], pcie_stream_));
  HL_CUDA(cudaEventRecord(ev_join_[slot], pcie_stream_));
  HL_CUDA(cudaStreamWaitEvent(user, ev_join_[slot], 0));
  // The callback runs in a stream of its own behind both halves: a host function in the caller's stream would
  // hold back the caller's next kernel until the driver thread has run it.
  HL_CUDA(cudaStreamWaitEvent(notify_stream_, s.rec->ev[1], 0));
  HL_CUDA(cudaStreamWaitEvent(notify_stream_, ev_join_[slot], 0));
  Done* d = new Done{this, s.idx, fast_ok, pcie_ok};
  HL_CUDA(cudaLaunchHostFunc(notify_stream_, hostCallback, d));
  comm_->stats.calls++;
  comm_->stats.bytes += s.rec->alg_bytes;
  comm_->stats.nvl_bytes += s.plan.fast_bytes;
  comm_->stats.pcie_bytes += s.plan.pcie_bytes;
  return hlSuccess;
}

void OrchImpl::timerMain() {
  cudaSetDevice(comm_->device);
  for (;;) {
    Done* d = nullptr;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [&] { return stop_ || !done_q_.empty(); });
      if (done_q_.empty()) {
        if (stop_) return;
        continue;
      }
      d = done_q_.front();
      done_q_.pop_front();
    }
    CallRecord& rec = ring_[d->idx % kRing];
    float fast_ms = 0, pcie_ms = 0;
    // the callback ran after the join, so all four events have completed
    if (cudaEventElapsedTime(&fast_ms, rec.ev[0], rec.ev[1]) != cudaSuccess) fast_ms = 0;
    if (cudaEventElapsedTime(&pcie_ms, rec.ev[2], rec.ev[3]) != cudaSuccess) pcie_ms = 0;
    cudaGetLastError();
    StatSlot& s = shared_->slots[comm_->rank][d->idx % kRing];
    s.fast_s = fast_ms * 1e-3;
    s.pcie_s = pcie_ms * 1e-3;
    s.fast_bytes = rec.plan.fast_bytes;
    s.pcie_bytes = rec.plan.pcie_bytes;
    s.fast_ok = d->fast_ok ? 1 : 0;
    s.pcie_ok = d->pcie_ok ? 1 : 0;
    s.call_idx.store(d->idx, std::memory_order_release);
    if (traceEnabled()) {
      traceCounter("alpha", 900, rec.key_bytes ? (double)rec.plan.pcie_bytes / (double)rec.key_bytes : 0);
      traceCounter("fast_ms", 901, fast_ms);
      traceCounter("pcie_ms", 902, pcie_ms);
    }
    delete d;
  }
}

void OrchImpl::fillStats(hlCommStats* out) const {
  out->last_alpha = last_alpha_;
  out->last_fast_ms = last_fast_ms_;
  out->last_pcie_ms = last_pcie_ms_;
}

// ====================================================================== facade
Orchestrator::~Orchestrator() { delete impl_; }
size_t Orchestrator::ctrlBytes(int) { return (sizeof(OrchShared) + 4095) & ~(size_t)4095; }

hlResult_t Orchestrator::create(hlComm* comm, void* area, Orchestrator** out) {
  std::unique_ptr<Orchestrator> o(new Orchestrator());
  o->impl_ = new OrchImpl(comm, area);
  HL_CHECK(o->impl_->init());
  *out = o.release();
  return hlSuccess;
}
bool Orchestrator::shouldSplit(size_t bytes) const { return impl_->shouldSplit(bytes); }
void Orchestrator::fillStats(hlCommStats* out) const { impl_->fillStats(out); }
std::string Orchestrator::dumpTuning() const { return impl_->dumpTuning(); }
hlResult_t Orchestrator::loadTuning(const char* json) { return impl_->loadTuning(json); }

namespace {
// One forked call: `fast` runs the NVLink kernel on `fast_elems` leading
// elements (per segment), `slow` runs the PCIe schedule on the rest.
template <typename Fast, typename Slow>
hlResult_t forked(OrchImpl* o, hlComm* comm, int op, size_t key_bytes, size_t alg_bytes, hlDataType_t t, cudaStream_t user,
                  Fast&& fast, Slow&& slow) {
  const size_t es = hlTypeSize(t);
  OrchImpl::Split s;
  HL_CHECK(o->begin(op, key_bytes, alg_bytes, (int)t, es, &s));
  const size_t fast_elems = s.plan.fast_bytes / es, total_elems = key_bytes / es;
  if (!s.plan.use_pcie || s.plan.pcie_bytes == 0) {
    o->publishImmediate(s.idx, s.plan);
    comm->stats.calls++;
    comm->stats.bytes += alg_bytes;
    comm->stats.nvl_bytes += key_bytes;
    return fast(total_elems, user);
  }
  HL_CHECK(o->fork(s, user));
  hlResult_t fr = hlSuccess, pr = hlSuccess;
  if (fast_elems) fr = fast(fast_elems, user);
  pr = slow(fast_elems, (hlStream_t)o->pcieStream());
  HL_CHECK(o->join(s, user, fr == hlSuccess, pr == hlSuccess));
  return fr != hlSuccess ? fr : pr;
}
}  // namespace

hlResult_t Orchestrator::allReduce(const void* send, void* recv, size_t count, hlDataType_t t, hlRedOp_t op, float scale, int algo,
                                   hlStream_t stream) {
  hlComm* c = impl_->comm();
  const size_t es = hlTypeSize(t);
  return forked(
      impl_, c, orch::kOpAllReduce, count * es, count * es, t, (cudaStream_t)stream,
      [&](size_t elems, cudaStream_t s) {
        NvlBufs b;
        memset(&b, 0, sizeof(b));
        b.in[0] = send;
        b.out[0] = recv;
        NvlCall k;
        k.count = elems;
        k.in_dt = k.out_dt = k.wire_dt = t;
        k.op = op;
        k.scale = scale;
        k.algo = algo;
        return c->nvl->allReduce(b, k, s);
      },
      [&](size_t skip, hlStream_t s) {
        return c->pcie->allReduce((const char*)send + skip * es, (char*)recv + skip * es, count - skip, t, op, scale, s);
      });
}

hlResult_t Orchestrator::reduceScatter(const void* send, void* recv, size_t recvcount, hlDataType_t t, hlRedOp_t op, float scale,
                                       hlStream_t stream) {
  hlComm* c = impl_->comm();
  const size_t es = hlTypeSize(t);
  return forked(
      impl_, c, orch::kOpReduceScatter, recvcount * es, recvcount * es * (size_t)c->nranks, t, (cudaStream_t)stream,
      [&](size_t elems, cudaStream_t s) {
        NvlBufs b;
        memset(&b, 0, sizeof(b));
        b.in[0] = send;
        b.out[0] = recv;
        NvlCall k;
        k.count = elems;
        k.in_seg_stride = recvcount;
        k.in_dt = k.out_dt = k.wire_dt = t;
        k.op = op;
        k.scale = scale;
        return c->nvl->reduceScatter(b, k, s);
      },
      [&](size_t skip, hlStream_t s) { return c->pcie->reduceScatter(send, recv, recvcount, skip, t, op, scale, s); });
}

hlResult_t Orchestrator::allGather(const void* send, void* recv, size_t sendcount, hlDataType_t t, hlStream_t stream) {
  hlComm* c = impl_->comm();
  const size_t es = hlTypeSize(t);
  return forked(
      impl_, c, orch::kOpAllGather, sendcount * es, sendcount * es * (size_t)c->nranks, t, (cudaStream_t)stream,
      [&](size_t elems, cudaStream_t s) {
        NvlBufs b;
        memset(&b, 0, sizeof(b));
        b.in[0] = send;
        b.out[0] = recv;
        NvlCall k;
        k.count = elems;
        k.out_seg_stride = sendcount;
        k.in_dt = k.out_dt = k.wire_dt = t;
        return c->nvl->allGather(b, k, s);
      },
      [&](size_t skip, hlStream_t s) { return c->pcie->allGather(send, recv, sendcount, skip, t, s); });
}

hlResult_t Orchestrator::allToAll(const void* send, void* recv, size_t count, hlDataType_t t, hlStream_t stream) {
  hlComm* c = impl_->comm();
  const size_t es = hlTypeSize(t);
  return forked(
      impl_, c, orch::kOpAllToAll, count * es, count * es * (size_t)c->nranks, t, (cudaStream_t)stream,
      [&](size_t elems, cudaStream_t s) {
        NvlBufs b;
        memset(&b, 0, sizeof(b));
        b.in[0] = send;
        b.out[0] = recv;
        NvlCall k;
        k.count = elems;
        k.in_seg_stride = count;
        k.out_seg_stride = count;
        k.in_dt = k.out_dt = k.wire_dt = t;
        return c->nvl->allToAll(b, k, s);
      },
      [&](size_t skip, hlStream_t s) { return c->pcie->allToAll(send, recv, count, skip, t, s); });
}

}  // namespace hl
