// torch.distributed backend ("hylink"): a c10d::Backend whose collectives run
// on this library's communicator.
//
// * One communicator per device kind, created lazily on the first collective;
//   the unique id travels through the c10d Store (rank 0 sets, others get).
// * CUDA tensors: every collective is launched on the backend's own
//   high-priority stream, which first waits for the caller's current stream;
//   the returned Work carries a CUDA event — wait() makes the caller's stream
//   wait for it (no host synchronisation), getFuture() gives DDP a CUDA-aware
//   future, so gradient buckets overlap with the backward pass.
// * CPU tensors: served by the host-memory device of the schedule-IR path
//   (no GPU needed), synchronously.
// * send/recv are not implemented here: pipeline point-to-point traffic stays
//   on NCCL (see hylink_b200.parallel.p2p).
//
// Parity: the reference has no c10d backend; PyTorch reaches it only through
// LD_PRELOAD of NCCL symbols (pcie-ccl-cuda/torch_dist_smoke/
// collectives_smoke.py:38-44, ddp_mlp_smoke.py:58-60).
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/chrono.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/python.h>

#include <atomic>
#include <cstring>
#include <mutex>

#include "hylink/hylink.h"

namespace {

using c10d::OpType;

void hlCheck(hlResult_t r, const char* what) {
  if (r != hlSuccess) {
    TORCH_CHECK(false, "hylink ", what, ": ", hlGetErrorString(r), " (", hlGetLastError(), ")");
  }
}

hlDataType_t toHl(at::ScalarType t) {
  switch (t) {
    case at::kChar: return hlInt8;
    case at::kByte: return hlUint8;
    case at::kBool: return hlUint8;
    case at::kInt: return hlInt32;
    case at::kLong: return hlInt64;
    case at::kHalf: return hlFloat16;
    case at::kFloat: return hlFloat32;
    case at::kDouble: return hlFloat64;
    case at::kBFloat16: return hlBfloat16;
    case at::kUInt32: return hlUint32;
    case at::kUInt64: return hlUint64;
    default: TORCH_CHECK(false, "hylink: unsupported dtype ", t);
  }
}

struct OpInfo {
  hlRedOp_t op;
  float scale;
};
OpInfo toHlOp(const c10d::ReduceOp& op) {
  switch (op.op_) {
    case c10d::ReduceOp::SUM: return {hlSum, 1.0f};
    case c10d::ReduceOp::AVG: return {hlAvg, 1.0f};
    case c10d::ReduceOp::PRODUCT: return {hlProd, 1.0f};
    case c10d::ReduceOp::MIN: return {hlMin, 1.0f};
    case c10d::ReduceOp::MAX: return {hlMax, 1.0f};
    default: TORCH_CHECK(false, "hylink: unsupported reduce op");
  }
}

// Events are recycled: creating and destroying two CUDA events per collective
// costs more host time than the rest of the launch path, and in a launch-bound
// training step every microsecond on the autograd thread is step time.
class EventPool {
 public:
  ~EventPool() {
    for (auto e : free_) cudaEventDestroy(e);
  }
  cudaEvent_t acquire() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      if (!free_.empty()) {
        cudaEvent_t e = free_.back();
        free_.pop_back();
        return e;
      }
    }
    cudaEvent_t e = nullptr;
    C10_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    return e;
  }
  void release(cudaEvent_t e) {
    std::lock_guard<std::mutex> lk(mu_);
    free_.push_back(e);
  }

 private:
  std::mutex mu_;
  std::vector<cudaEvent_t> free_;
};

class HylinkWork : public c10d::Work {
 public:
  HylinkWork(int rank, OpType op, std::vector<at::Tensor> outputs, std::vector<at::Tensor> keep)
      : c10d::Work(rank, op), outputs_(std::move(outputs)), keep_(std::move(keep)) {}

  ~HylinkWork() override {
    if (event_ && pool_) pool_->release(event_);
  }

  // CUDA flavour: call with the communication stream current.
  void armCuda(c10::cuda::CUDAStream comm_stream, const std::shared_ptr<EventPool>& pool) {
    cuda_ = true;
    device_ = comm_stream.device();
    pool_ = pool;
    event_ = pool->acquire();
    C10_CUDA_CHECK(cudaEventRecord(event_, comm_stream.stream()));
    future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                       std::vector<c10::Device>{device_});
    c10::cuda::CUDAStreamGuard g(comm_stream);
    future_->markCompleted(at::IValue(outputs_));
  }
  // One-rank groups: the work ran on the caller's own stream, so there is nothing to wait for on that stream and
  // no event is recorded (an event pair per call is most of the cost of a collective that moves nothing).
  void armInline(c10::cuda::CUDAStream stream, const std::shared_ptr<EventPool>& pool) {
    cuda_ = true;
    inline_ = true;
    device_ = stream.device();
    pool_ = pool;
    inline_stream_ = stream.stream();
  }
  void armCpu() {
    future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
    future_->markCompleted(at::IValue(outputs_));
  }

  bool isCompleted() override {
    if (!cuda_ || (inline_ && !event_)) return true;
    const cudaError_t e = cudaEventQuery(event_);
    if (e == cudaErrorNotReady) {
      (void)cudaGetLastError();
      return false;
    }
    return true;
  }
  bool isSuccess() const override { return true; }
  void synchronize() override {
    if (!cuda_) return;
    cudaStream_t cur = c10::cuda::getCurrentCUDAStream(device_.index()).stream();
    if (inline_) {
      if (cur == inline_stream_) return;   // stream order already covers it
      if (!event_) {                       // recorded late: covers the work and whatever followed it on that stream
        event_ = pool_->acquire();
        C10_CUDA_CHECK(cudaEventRecord(event_, inline_stream_));
      }
    }
    C10_CUDA_CHECK(cudaStreamWaitEvent(cur, event_, 0));
  }
  bool wait(std::chrono::milliseconds /*timeout*/) override {
    synchronize();
    keep_.clear();
    return true;
  }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override {
    if (!future_ && inline_) {
      future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), std::vector<c10::Device>{device_});
      c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(inline_stream_, device_.index()));
      future_->markCompleted(at::IValue(outputs_));
    }
    return future_;
  }
  std::vector<at::Tensor> result() override { return outputs_; }

 private:
  std::vector<at::Tensor> outputs_;
  std::vector<at::Tensor> keep_;  // inputs kept alive until the caller has waited
  bool cuda_ = false;
  bool inline_ = false;
  cudaStream_t inline_stream_ = nullptr;
  c10::Device device_{c10::kCPU};
  cudaEvent_t event_ = nullptr;
  std::shared_ptr<EventPool> pool_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

class HylinkBackend : public c10d::Backend {
 public:
  HylinkBackend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout)
      : c10d::Backend(rank, size), store_(store), timeout_(timeout) {
    // CTA budget of a collective (0 = the library's table, up to one CTA per SM for large messages). A caller
    // whose collectives overlap with compute lowers it (setCtaBudget, as DDPTrainer does): a grid on every SM
    // finishes each gradient bucket sooner but stalls the GEMMs beside it for longer than it saves (GPT-2-medium
    // DDP on 2 GPUs: 55.4 ms per step with 148 CTAs, 54.5 ms with 48 to 96). Stand-alone collectives keep the table.
    if (const char* e = getenv("HYLINK_TORCH_MAX_BLOCKS")) max_blocks_ = atoi(e);
    if (const char* e = getenv("HYLINK_TORCH_SYNC_INLINE")) sync_inline_ = atoi(e) != 0;
  }
  ~HylinkBackend() override { shutdown(); }

  const std::string getBackendName() const override { return "hylink"; }

  void shutdown() override {
    std::lock_guard<std::mutex> lk(mu_);
    alive_->store(false);   // registered tensors that outlive the group must not reach into a destroyed communicator
    if (cuda_comm_) {
      hlCommDestroy(cuda_comm_);
      cuda_comm_ = nullptr;
    }
    if (cpu_comm_) {
      hlCommDestroy(cpu_comm_);
      cpu_comm_ = nullptr;
    }
  }
  void abort() override { shutdown(); }

  // ---- helpers -----------------------------------------------------------
  hlComm_t commFor(const at::Tensor& t) {
    std::lock_guard<std::mutex> lk(mu_);
    const bool cuda = t.is_cuda();
    hlComm_t& slot = cuda ? cuda_comm_ : cpu_comm_;
    if (slot) return slot;
    hlUniqueId id;
    const std::string key = std::string("hylink/uid/") + (cuda ? "cuda" : "cpu") + "/" + std::to_string(generation_);
    if (getRank() == 0) {
      hlCheck(hlGetUniqueId(&id), "hlGetUniqueId");
      std::vector<uint8_t> v(sizeof(id));
      memcpy(v.data(), &id, sizeof(id));
      store_->set(key, v);
    } else {
      std::vector<uint8_t> v = store_->get(key);
      TORCH_CHECK(v.size() == sizeof(id), "hylink: bad unique id in the store");
      memcpy(&id, v.data(), sizeof(id));
    }
    int device = -2;
    if (cuda) {
      device = t.device().index();
      cuda_device_ = device;
      // Normal priority by default: a high-priority collective grabs SMs ahead of the backward pass it overlaps with.
      const char* hp = getenv("HYLINK_TORCH_HIGH_PRIORITY");
      comm_stream_ = std::make_unique<c10::cuda::CUDAStream>(c10::cuda::getStreamFromPool(/*isHighPriority=*/hp && atoi(hp) != 0, device));
    }
    hlCheck(hlCommInitRankDevice(&slot, getSize(), id, getRank(), device), "hlCommInitRankDevice");
    if (cuda) hlSetAllocatorComm(slot);   // the registered-memory allocator hooks serve from this communicator's heap
    if (cuda && ready_ring_.empty()) {
      c10::cuda::CUDAGuard dg(t.device());
      ready_ring_.resize(64);
      for (auto& e : ready_ring_) C10_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    return slot;
  }

  // `async_op` is the caller's async_op flag (c10d passes it in every options struct). A synchronous call is waited
  // for on the caller's stream right after it returns, so it CAN run on that stream (HYLINK_TORCH_SYNC_INLINE=1): no
  // ready event, no hop to the communication stream and back. Off by default, by measurement on 4 GPUs: a call
  // queued behind other work is 1-3 us shorter inline, but a sequence of collectives that are each bracketed by
  // timing events is 2-3 us per call LONGER inline (geometric mean of the 1 MiB-1 GiB table 278.8 against 289.8 GB/s):
  // on its own stream the kernel is set up while the caller's stream is still busy with the events around it.
  template <typename F>
  c10::intrusive_ptr<c10d::Work> run(bool async_op, OpType type, const at::Tensor& probe, std::vector<at::Tensor> outputs,
                                     std::vector<at::Tensor> keep, F&& body) {
    hlComm_t comm = commFor(probe);
    auto work = c10::make_intrusive<HylinkWork>(getRank(), type, std::move(outputs), std::move(keep));
    if (probe.is_cuda() && (getSize() == 1 || (!async_op && sync_inline_))) {
      // one rank: every collective is local work; it runs on the caller's stream, with no hop to another stream
      c10::cuda::CUDAGuard dg(probe.device());
      auto cur = c10::cuda::getCurrentCUDAStream(probe.device().index());
      body(comm, (hlStream_t)cur.stream());
      work->armInline(cur, events_);
      ++collectives_;
    } else if (probe.is_cuda()) {
      c10::cuda::CUDAGuard dg(probe.device());
      auto cur = c10::cuda::getCurrentCUDAStream(probe.device().index());
      cudaEvent_t ready = ready_ring_[ready_next_++ % ready_ring_.size()];
      C10_CUDA_CHECK(cudaEventRecord(ready, cur.stream()));
      C10_CUDA_CHECK(cudaStreamWaitEvent(comm_stream_->stream(), ready, 0));
      body(comm, (hlStream_t)comm_stream_->stream());
      work->armCuda(*comm_stream_, events_);
      ++collectives_;
    } else {
      body(comm, nullptr);
      hlCheck(hlCommDrain(comm), "hlCommDrain");
      work->armCpu();
    }
    return work;
  }

  static void checkContig(const at::Tensor& t) { TORCH_CHECK(t.is_contiguous(), "hylink: tensors must be contiguous"); }

  // ---- collectives ---------------------------------------------------------
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) override {
    TORCH_CHECK(tensors.size() == 1, "hylink: one tensor per allreduce");
    at::Tensor t = tensors[0];
    checkContig(t);
    const OpInfo oi = toHlOp(opts.reduceOp);
    return run(opts.asyncOp, OpType::ALLREDUCE, t, {t}, {t}, [&](hlComm_t c, hlStream_t s) {
      hlCallOpts o;
      memset(&o, 0, sizeof(o));
      o.scale = fused_scale_ != 0.0f ? fused_scale_ : oi.scale;
      o.max_blocks = max_blocks_;
      hlCheck(hlAllReduceEx(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), toHl(t.scalar_type()), oi.op, &o, c, s), "allreduce");
    });
  }

  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                     const c10d::AllreduceCoalescedOptions& opts) override {
    TORCH_CHECK(!tensors.empty(), "hylink: empty tensor list");
    const OpInfo oi = toHlOp(opts.reduceOp);
    std::vector<at::Tensor> ts = tensors;
    return run(opts.asyncOp, OpType::ALLREDUCE_COALESCED, ts[0], ts, ts, [&](hlComm_t c, hlStream_t s) {
      for (auto& t : ts) {
        checkContig(t);
        hlCheck(hlAllReduce(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), toHl(t.scalar_type()), oi.op, c, s), "allreduce_coalesced");
      }
    });
  }

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) override {
    TORCH_CHECK(tensors.size() == 1, "hylink: one tensor per broadcast");
    at::Tensor t = tensors[0];
    checkContig(t);
    const int root = (int)opts.rootRank;
    return run(opts.asyncOp, OpType::BROADCAST, t, {t}, {t}, [&](hlComm_t c, hlStream_t s) {
      hlCheck(hlBroadcast(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), toHl(t.scalar_type()), root, c, s), "broadcast");
    });
  }

  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& out, at::Tensor& in, const c10d::AllgatherOptions& opts) override {
    checkContig(out);
    checkContig(in);
    TORCH_CHECK(out.numel() == in.numel() * getSize(), "hylink: all_gather_into_tensor size mismatch");
    at::Tensor o = out, i = in;
    return run(opts.asyncOp, OpType::_ALLGATHER_BASE, i, {o}, {i, o}, [&](hlComm_t c, hlStream_t s) {
      hlCallOpts co;
      memset(&co, 0, sizeof(co));
      co.max_blocks = max_blocks_;
      hlCheck(hlAllGatherEx(i.data_ptr(), o.data_ptr(), (size_t)i.numel(), toHl(i.scalar_type()), &co, c, s), "allgather");
    });
  }

  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins,
                                           const c10d::AllgatherOptions& opts) override {
    TORCH_CHECK(ins.size() == 1 && outs.size() == 1, "hylink: one input per allgather");
    at::Tensor in = ins[0].contiguous();
    std::vector<at::Tensor> dst = outs[0];
    TORCH_CHECK((int)dst.size() == getSize(), "hylink: allgather output list must have world_size entries");
    at::Tensor flat = at::empty({(int64_t)getSize() * in.numel()}, in.options());
    return run(opts.asyncOp, OpType::ALLGATHER, in, dst, {in, flat}, [&](hlComm_t c, hlStream_t s) {
      hlCheck(hlAllGather(in.data_ptr(), flat.data_ptr(), (size_t)in.numel(), toHl(in.scalar_type()), c, s), "allgather");
      c10::OptionalStreamGuard sg;
      if (in.is_cuda()) sg.reset_stream(c10::cuda::getStreamFromExternal((cudaStream_t)s, in.device().index()));
      else hlCheck(hlCommDrain(c), "hlCommDrain");  // host path: the gather must have landed before it is split up
      for (int q = 0; q < getSize(); ++q) dst[q].copy_(flat.narrow(0, (int64_t)q * in.numel(), in.numel()).view_as(dst[q]), true);
    });
  }

  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins,
                                                                 const c10d::AllgatherOptions& opts) override {
    TORCH_CHECK(outs.size() == ins.size() && !ins.empty(), "hylink: list size mismatch");
    std::vector<at::Tensor> o = outs, i = ins, keep = ins;
    keep.insert(keep.end(), o.begin(), o.end());
    return run(opts.asyncOp, OpType::ALLGATHER_COALESCED, i[0], o, keep, [&](hlComm_t c, hlStream_t s) {
      for (size_t k = 0; k < i.size(); ++k) {
        checkContig(i[k]);
        checkContig(o[k]);
        hlCheck(hlAllGather(i[k].data_ptr(), o[k].data_ptr(), (size_t)i[k].numel(), toHl(i[k].scalar_type()), c, s), "allgather_coalesced");
      }
    });
  }

  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& out, at::Tensor& in, const c10d::ReduceScatterOptions& opts) override {
    checkContig(out);
    checkContig(in);
    TORCH_CHECK(in.numel() == out.numel() * getSize(), "hylink: reduce_scatter_tensor size mismatch");
    const OpInfo oi = toHlOp(opts.reduceOp);
    at::Tensor o = out, i = in;
    return run(opts.asyncOp, OpType::_REDUCE_SCATTER_BASE, i, {o}, {i, o}, [&](hlComm_t c, hlStream_t s) {
      hlCallOpts co;
      memset(&co, 0, sizeof(co));
      co.max_blocks = max_blocks_;
      hlCheck(hlReduceScatterEx(i.data_ptr(), o.data_ptr(), (size_t)o.numel(), toHl(i.scalar_type()), oi.op, &co, c, s), "reduce_scatter");
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins,
                                                const c10d::ReduceScatterOptions& opts) override {
    TORCH_CHECK(outs.size() == 1 && ins.size() == 1 && (int)ins[0].size() == getSize(), "hylink: bad reduce_scatter lists");
    at::Tensor out = outs[0];
    checkContig(out);
    const OpInfo oi = toHlOp(opts.reduceOp);
    std::vector<at::Tensor> parts = ins[0];
    at::Tensor probe = out;
    return run(opts.asyncOp, OpType::REDUCE_SCATTER, probe, {out}, parts, [&](hlComm_t c, hlStream_t s) {
      c10::OptionalStreamGuard sg;
      if (out.is_cuda()) sg.reset_stream(c10::cuda::getStreamFromExternal((cudaStream_t)s, out.device().index()));
      std::vector<at::Tensor> flat_parts;
      for (auto& p : parts) flat_parts.push_back(p.reshape({-1}));
      at::Tensor flat = at::cat(flat_parts);
      hlCheck(hlReduceScatter(flat.data_ptr(), out.data_ptr(), (size_t)out.numel(), toHl(out.scalar_type()), oi.op, c, s), "reduce_scatter");
      if (out.is_cuda())
        c10::cuda::CUDACachingAllocator::recordStream(flat.storage().data_ptr(), c10::cuda::getStreamFromExternal((cudaStream_t)s, out.device().index()));
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins,
                                                                 const c10d::ReduceScatterOptions& opts) override {
    TORCH_CHECK(outs.size() == ins.size() && !ins.empty(), "hylink: list size mismatch");
    const OpInfo oi = toHlOp(opts.reduceOp);
    std::vector<at::Tensor> o = outs, i = ins, keep = ins;
    keep.insert(keep.end(), o.begin(), o.end());
    return run(opts.asyncOp, OpType::COALESCED, i[0], o, keep, [&](hlComm_t c, hlStream_t s) {
      for (size_t k = 0; k < i.size(); ++k) {
        checkContig(i[k]);
        checkContig(o[k]);
        hlCheck(hlReduceScatter(i[k].data_ptr(), o[k].data_ptr(), (size_t)o[k].numel(), toHl(i[k].scalar_type()), oi.op, c, s), "reduce_scatter_coalesced");
      }
    });
  }

  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& out, at::Tensor& in, std::vector<int64_t>& outSplit,
                                               std::vector<int64_t>& inSplit, const c10d::AllToAllOptions& opts) override {
    TORCH_CHECK(outSplit.empty() && inSplit.empty(), "hylink: only equal splits are supported by all_to_all_single");
    checkContig(out);
    checkContig(in);
    TORCH_CHECK(out.numel() == in.numel() && in.numel() % getSize() == 0, "hylink: all_to_all_single size mismatch");
    at::Tensor o = out, i = in;
    return run(opts.asyncOp, OpType::ALLTOALL_BASE, i, {o}, {i, o}, [&](hlComm_t c, hlStream_t s) {
      hlCheck(hlAllToAll(i.data_ptr(), o.data_ptr(), (size_t)i.numel() / getSize(), toHl(i.scalar_type()), c, s), "all_to_all");
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) override {
    // Reduce to one root = all-reduce whose result the other ranks discard
    // into a scratch buffer (keeps their tensors untouched).
    TORCH_CHECK(tensors.size() == 1, "hylink: one tensor per reduce");
    at::Tensor t = tensors[0];
    checkContig(t);
    const OpInfo oi = toHlOp(opts.reduceOp);
    const bool root = (int)opts.rootRank == getRank();
    at::Tensor dst = root ? t : at::empty_like(t);
    return run(opts.asyncOp, OpType::REDUCE, t, {t}, {t, dst}, [&](hlComm_t c, hlStream_t s) {
      hlCheck(hlAllReduce(t.data_ptr(), dst.data_ptr(), (size_t)t.numel(), toHl(t.scalar_type()), oi.op, c, s), "reduce");
    });
  }

  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts) override {
    at::Tensor probe;
    if (cuda_comm_ || !cpu_comm_) {
      int dev = cuda_device_ >= 0 ? cuda_device_ : (opts.device_ids.empty() ? -1 : (int)opts.device_ids[0]);
      if (dev < 0 && at::hasCUDA()) dev = c10::cuda::current_device();
      if (dev >= 0) probe = at::empty({1}, at::TensorOptions().device(at::kCUDA, dev).dtype(at::kFloat));
    }
    if (!probe.defined()) probe = at::empty({1}, at::TensorOptions().dtype(at::kFloat));
    return run(opts.asyncOp, OpType::BARRIER, probe, {}, {probe}, [&](hlComm_t c, hlStream_t s) { hlCheck(hlBarrier(c, s), "barrier"); });
  }

  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>&, int, int) override {
    TORCH_CHECK(false, "hylink: point-to-point traffic stays on NCCL; use hylink_b200.parallel.p2p");
  }
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>&, int, int) override {
    TORCH_CHECK(false, "hylink: point-to-point traffic stays on NCCL; use hylink_b200.parallel.p2p");
  }

  // ---- extras exposed to Python -------------------------------------------
  // A tensor in registered memory (same heap offset on every rank): collectives on it run zero-copy. Every rank
  // must call this in the same order with the same sizes. Falls back to ordinary device memory when the heap is full.
  at::Tensor symmetricEmpty(std::vector<int64_t> sizes, at::ScalarType dtype, int device) {
    at::Tensor probe = at::empty({1}, at::TensorOptions().device(at::kCUDA, device).dtype(at::kFloat));
    hlComm_t comm = commFor(probe);
    int64_t numel = 1;
    for (auto d : sizes) numel *= d;
    const size_t bytes = (size_t)std::max<int64_t>(numel, 1) * c10::elementSize(dtype);
    void* ptr = nullptr;
    hlCheck(hlMemAlloc(comm, bytes, &ptr), "hlMemAlloc");
    std::shared_ptr<std::atomic<bool>> alive = alive_;
    // (after the group is gone its heap is gone with it: nothing left to release)
    return at::from_blob(ptr, sizes, [comm, alive](void* p) { if (alive->load()) hlMemFree(comm, p); },
                         at::TensorOptions().device(at::kCUDA, device).dtype(dtype));
  }
  bool isRegistered(const at::Tensor& t) {
    std::lock_guard<std::mutex> lk(mu_);
    return cuda_comm_ && t.is_cuda() && hlMemIsRegistered(cuda_comm_, t.data_ptr(), t.nbytes()) != 0;
  }
  void setFusedScale(float s) { fused_scale_ = s; }
  void setCtaBudget(int b) { max_blocks_ = b < 0 ? 0 : b; }
  int ctaBudget() const { return max_blocks_; }
  py::dict stats() {
    py::dict d;
    hlComm_t c = cuda_comm_ ? cuda_comm_ : cpu_comm_;
    d["collectives"] = collectives_;
    if (c) {
      hlCommStats st;
      memset(&st, 0, sizeof(st));
      hlCommGetStats(c, &st);
      d["calls"] = st.calls;
      d["bytes"] = st.bytes;
      d["nvl_bytes"] = st.nvl_bytes;
      d["pcie_bytes"] = st.pcie_bytes;
      d["kernel_launches"] = st.kernel_launches;
      d["copy_engine_ops"] = st.copy_engine_ops;
      d["last_alpha"] = st.last_alpha;
      d["last_fast_ms"] = st.last_fast_ms;
      d["last_pcie_ms"] = st.last_pcie_ms;
      d["nvls"] = st.nvls;
      d["symm_mode"] = st.symm_mode;
      d["fused_landing_slices"] = st.fused_landing_slices;
      d["folded_sources"] = st.folded_sources;
      d["registered_bytes"] = st.registered_bytes;
      d["small_path_calls"] = st.small_path_calls;
      d["h2h_range_jobs"] = st.h2h_range_jobs;
      d["composed_allreduces"] = st.composed_allreduces;
    }
    return d;
  }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
  std::chrono::milliseconds timeout_;
  std::mutex mu_;
  hlComm_t cuda_comm_ = nullptr;
  hlComm_t cpu_comm_ = nullptr;
  int cuda_device_ = -1;
  int generation_ = 0;
  std::unique_ptr<c10::cuda::CUDAStream> comm_stream_;
  uint64_t collectives_ = 0;
  std::vector<cudaEvent_t> ready_ring_;   // "inputs are ready" markers; a slot is reused 64 collectives later
  size_t ready_next_ = 0;
  std::shared_ptr<EventPool> events_ = std::make_shared<EventPool>();
  float fused_scale_ = 0.0f;
  int max_blocks_ = 0;
  bool sync_inline_ = false;  // HYLINK_TORCH_SYNC_INLINE=1: synchronous calls run on the caller's stream instead of the communication stream
  std::shared_ptr<std::atomic<bool>> alive_ = std::make_shared<std::atomic<bool>>(true);
};

c10::intrusive_ptr<c10d::Backend> createHylinkBackend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                                      const std::chrono::duration<float>& timeout) {
  return c10::make_intrusive<HylinkBackend>(store, rank, size, std::chrono::duration_cast<std::chrono::milliseconds>(timeout));
}

HylinkBackend* asHylink(const c10::intrusive_ptr<c10d::Backend>& b) {
  auto* p = dynamic_cast<HylinkBackend*>(b.get());
  TORCH_CHECK(p, "not a hylink backend");
  return p;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("create_backend", &createHylinkBackend, py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"));
  m.def("backend_stats", [](const c10::intrusive_ptr<c10d::Backend>& b) { return asHylink(b)->stats(); });
  // Multiplies every all-reduce result by `scale` inside the kernel (0 = off):
  // lets a DDP wrapper fold its gradient pre-division into the collective.
  m.def("set_fused_scale", [](const c10::intrusive_ptr<c10d::Backend>& b, float s) { asHylink(b)->setFusedScale(s); });
  m.def("symmetric_empty", [](const c10::intrusive_ptr<c10d::Backend>& b, std::vector<int64_t> sizes, py::object dtype, int device) {
    return asHylink(b)->symmetricEmpty(std::move(sizes), torch::python::detail::py_object_to_dtype(dtype), device);
  });
  m.def("is_registered", [](const c10::intrusive_ptr<c10d::Backend>& b, const at::Tensor& t) { return asHylink(b)->isRegistered(t); });
  // CTAs a collective of this group may occupy (0 = the library's size table). Returns the previous budget.
  m.def("set_cta_budget", [](const c10::intrusive_ptr<c10d::Backend>& b, int n) {
    const int old = asHylink(b)->ctaBudget();
    asHylink(b)->setCtaBudget(n);
    return old;
  });
}
