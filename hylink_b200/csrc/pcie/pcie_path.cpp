// PCIe path: a CPU-driven executor that runs compiled schedule graphs.
//
// Per communicator: one executor thread, a bounded work queue, shared pinned
// staging pools (one per logical NUMA node, created by the node's lowest rank,
// mapped and registered by every rank), a device scratch buffer, DMA lanes
// (dedicated high-priority streams for D2H, H2D, local D2D and the landing
// reduce kernel) and the NUMA-pinned worker pool for host-to-host work.
//
// A collective is cut into rounds that fit the staging pools; a round is cut
// into pipelined slices. Slice k of a node is issued as soon as slice k of all
// nodes it waits for is complete — completion is published in a per-node
// counter inside the communicator's shared control block, tagged with the
// work sequence number, so peers' executors observe each other's progress
// without any call into the driver. The caller's stream is parked on a
// doorbell: cuStreamWriteValue64 tells the executor that prior work on the
// stream is done (inputs valid), cuStreamWaitValue64 holds the stream until the
// executor's plain CPU store releases it. With the host-memory device (no
// GPU) "device" buffers are host memory and every copy runs on the worker
// pool; the same graphs, protocol and tests apply.
//
// Parity: pcie-ccl-cuda/src/executor/graph_executor.cpp:192-319,353-441,
// 804-879,1006-1465 (submit, thread, doorbell wait, node issue loop, drain,
// barrier), src/memory/completion_flag.cpp:263-438 (doorbell),
// src/memory/host_pool.cpp:95-385 (shared pinned pools),
// src/memory/shared_state.hpp:153-325 (cross-rank progress),
// src/api/pccl_api.cpp:389-629 (plan cache, IR selection, in-place handling).
#include "pcie/pcie_path.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <thread>

#include "core/trace.h"
#include "hal/cuda_driver.h"
#include "host/host_simd.h"
#include "host/topology.h"
#include "host/worker_pool.h"
#include "ir/compiler.h"
#include "nvl/nvl_launch.h"

namespace hl {

namespace {

constexpr int kSeqShift = 20;
constexpr uint64_t kSliceMask = (1ull << kSeqShift) - 1;
constexpr int kLaneDepth = 32;
constexpr uint64_t kReleaseAll = ~0ull >> 1;

struct SharedArea {
  std::atomic<uint64_t> progress[ir::kMaxNodes];
  std::atomic<uint64_t> ready_seq[kMaxRanks];
  std::atomic<uint64_t> ptrs[kMaxRanks][4];  // input, output, scratch, internal bases (single-process mode)
  std::atomic<uint32_t> failed;
};

struct Plan {
  ir::Program program;
  ir::CompiledGraph graph;
  std::string source;  // file path or "generated"
};

struct Work {
  uint64_t seq = 0;
  std::shared_ptr<const Plan> plan;
  ir::Geometry geo;
  const char* send = nullptr;
  char* recv = nullptr;
  hlDataType_t dtype = hlFloat32;
  hlRedOp_t op = hlSum;
  bool first_round = true, last_round = true;
  uint64_t door_seq = 0;     // doorbell value of the whole collective
  double host_scale = 1.0;   // host device only: applied to the output after the last round
  size_t scale_off = 0, scale_count = 0;
  int scale_segs = 0;
  size_t scale_seg_stride = 0;
  std::string name;
  int dma_lanes = 2;         // copy-engine lanes per direction this collective uses (dmaLanePolicy)
  int prev_nslices = 0;      // slices per node of the previous round of the same message (0: this is the first round)
};

constexpr int kMaxDmaLanes = 8;

enum LaneId { kLaneD2H = 0, kLaneH2D = 1, kLaneD2D = 2, kLaneReduce = 3, kLaneHost = 4, kNumLaneKinds = 5 };

struct InFlight {
  int node_slot = -1;     // index into the round's local node table
  cudaEvent_t ev = nullptr;
  std::shared_ptr<HostTicket> ticket;
  uint64_t t0_ns = 0;
  size_t bytes = 0;       // payload of the slice (trace)
  std::vector<int> also;  // further local nodes whose slice finishes with this one (fused H2D nodes, folded reduces)
};

struct Lane {
  cudaStream_t stream = nullptr;
  std::deque<InFlight> inflight;
  std::vector<cudaEvent_t> free_events;
};

}  // namespace

class PcieImpl {
 public:
  PcieImpl(Bootstrap* bs, int device, void* area) : bs_(bs), device_(device), cuda_(device >= 0), shared_((SharedArea*)area) {
    rank_ = bs->rank();
    n_ = bs->nranks();
  }
  ~PcieImpl();
  hlResult_t init();
  hlResult_t submit(const std::string& collective, const std::string& forced_xml, const void* send, void* recv,
                    size_t seg_count, size_t stride, int send_segs, int recv_segs, hlDataType_t t, hlRedOp_t op,
                    float scale, int root, hlStream_t stream);
  hlResult_t drain();
  void drainHostSide() { (void)drain(); }
  hlResult_t lastResult() const { return (hlResult_t)last_result_.load(); }
  uint64_t kernelLaunches() const { return kernel_launches_.load(); }
  uint64_t copyOps() const { return copy_ops_.load(); }
  uint64_t smallCalls() const { return small_calls_.load(); }
  uint64_t fusedSlices() const { return fused_slices_.load(); }
  uint64_t rangeJobs() const { return range_jobs_.load(); }
  uint64_t foldedSources() const { return folded_sources_.load(); }
  const std::vector<int>& rankNuma() const { return numa_; }

 private:
  hlResult_t createHostPools();
  hlResult_t getPlan(const std::string& collective, const std::string& forced_xml, int root, ir::InPlace ip, int send_segs,
                     int recv_segs, size_t bytes, std::shared_ptr<const Plan>* out);
  void threadMain();
  hlResult_t runWork(const Work& w);
  // Returns hlSuccess with *handled = false when the call does not qualify (the ordinary executor then runs it).
  hlResult_t submitSmall(const std::string& collective, const void* send, void* recv, size_t seg_count, int send_segs, int recv_segs,
                         hlDataType_t t, hlRedOp_t op, float scale, int root, cudaStream_t us, bool* handled);
  volatile uint64_t* smallFlag(bool done, int parity, int rank, bool device) const {
    char* base = device ? small_dev_ : small_host_;
    return reinterpret_cast<volatile uint64_t*>(base) + ((done ? 2 : 0) + parity) * kMaxRanks + rank;
  }
  void watchSmallCalls();
  hlResult_t waitReady(const Work& w);
  void releaseDoorbell(uint64_t value);
  void failAll(hlResult_t r);
  char* resolve(const Work& w, const ir::Loc& l, size_t* len_bytes, bool* remote_pending);
  Lane& laneFor(ir::Op op, int salt, int active);
  cudaEvent_t getEvent(Lane& l);

  Bootstrap* bs_;
  int device_;
  bool cuda_;
  SharedArea* shared_;
  int rank_ = 0, n_ = 1;
  std::vector<int> numa_, phys_of_logical_;
  PairTopology pairs_;                 // which GPU pairs share a PCIe switch / an NVLink / peer access
  int numa_nodes_ = 1;
  std::vector<char*> host_base_;
  std::vector<char*> host_dev_base_;   // the same pools as the device addresses them (mapped pinned memory)
  bool fuse_landing_ = true;           // reduce kernels read landed host chunks themselves (HYLINK_PCIE_FUSE_LANDING)
  std::atomic<uint64_t> fused_slices_{0}, folded_sources_{0}, range_jobs_{0};
  std::vector<size_t> host_map_bytes_;
  std::vector<bool> host_registered_, host_cuda_alloc_;
  size_t host_bytes_ = 0;        // size of every pool
  size_t sched_host_bytes_ = 0;  // the part of a pool that schedules use (the small-message area sits behind it in pool 0)
  // ---- small-message path: stream-ordered one-shot exchange through pinned host memory (submitSmall)
  char* small_host_ = nullptr;   // the area as the CPU sees it: 4 KiB of flag words, then [parity][rank] slots
  char* small_dev_ = nullptr;    // ... and as this device addresses it
  size_t small_slot_bytes_ = 0;
  uint64_t small_seq_ = 0;
  struct SmallPending {
    uint64_t seq;
    uint64_t t_ns;
  };
  std::deque<SmallPending> small_pending_;   // under mu_: calls whose completion the watchdog still has to see
  cudaEvent_t small_ev_ = nullptr;
  bool small_used_ = false;
  std::atomic<uint64_t> small_calls_{0};
  char* internal_ = nullptr;
  size_t internal_bytes_ = 0;
  char* inplace_stage_ = nullptr;
  size_t inplace_stage_bytes_ = 0;
  // doorbell words (host memory the GPU can write / poll)
  volatile uint64_t* door_host_ = nullptr;  // [0] ready, [1] complete, [2] status
  uint64_t* door_dev_ = nullptr;
  bool stream_mem_ops_ = true;
  std::unique_ptr<WorkerPool> pool_;
  std::vector<Lane> lanes_[kNumLaneKinds];
  int lanes_per_dir_ = 1;
  // queue
  std::mutex mu_;
  std::condition_variable cv_, cv_done_;
  std::deque<Work> queue_;
  bool stop_ = false;
  std::thread thread_;
  uint64_t next_seq_ = 1, next_door_ = 1;
  std::atomic<uint64_t> completed_door_{0};
  std::atomic<int> last_result_{hlSuccess};
  std::atomic<uint64_t> kernel_launches_{0}, copy_ops_{0};
  long issued_ops_ = 0;  // transfers issued so far (executor thread only; drives host-side fault injection)
  std::map<std::string, std::shared_ptr<const Plan>> plans_;
  cudaEvent_t order_ev_ = nullptr;
  friend class PciePath;
};

// ---------------------------------------------------------------------- init
hlResult_t PcieImpl::init() {
  const Config& cfg = Config::get();
  HL_CHECK(discoverRankNuma(bs_, device_, &numa_, &phys_of_logical_));
  HL_CHECK(discoverPairTopology(bs_, cuda_ ? device_ : -1, &pairs_));
  numa_nodes_ = (int)phys_of_logical_.size();
  bs_->publishSelf(device_, numa_[(size_t)rank_]);
  host_bytes_ = cfg.host_buffer_bytes & ~(size_t)4095;
  // behind the schedules' part of pool 0: flag words + two parities of one slot per rank
  small_slot_bytes_ = (cfg.small_msg_fastpath && cuda_) ? ((cfg.small_msg_threshold_bytes + 4095) & ~(size_t)4095) : 0;
  const size_t small_area = small_slot_bytes_ ? 4096 + 2 * (size_t)n_ * small_slot_bytes_ : 0;
  if (small_area * 2 > host_bytes_) small_slot_bytes_ = 0;   // tiny pools (tests): no small-message area
  sched_host_bytes_ = host_bytes_ - (small_slot_bytes_ ? small_area : 0);
  internal_bytes_ = cfg.internal_buffer_bytes & ~(size_t)4095;
  if (cuda_) {
    HL_CUDA(cudaSetDevice(device_));
    HL_CUDA(cudaMalloc((void**)&internal_, internal_bytes_));
    uint64_t* h = nullptr;
    HL_CUDA(cudaHostAlloc((void**)&h, 64, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(h, 0, 64);
    door_host_ = h;
    HL_CUDA(cudaHostGetDevicePointer((void**)&door_dev_, h, 0));
    const CudaDriver* drv = CudaDriver::get();
    stream_mem_ops_ = drv && !cfg.disable_stream_mem_ops;
    // The executor drives many streams from the CPU while a user stream sits parked on a stream-memory wait: with
    // a single hardware connection the copies queue up behind that wait and nothing moves
    // (pcie-ccl-cuda/README.md:665 asks for 8).
    const long long conns = envInt({"CUDA_DEVICE_MAX_CONNECTIONS"}, 8);
    if (conns < 8 && rank_ == 0)
      HL_WARN("CUDA_DEVICE_MAX_CONNECTIONS=%lld: the PCIe path needs independent hardware queues for its copy streams; use 8 or more", conns);
    int lo = 0, hi = 0;
    HL_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    lanes_per_dir_ = kMaxDmaLanes;   // all created once; each collective uses as many as the lane policy says
    for (int k = 0; k < kNumLaneKinds; ++k) {
      const int count = (k == kLaneD2H || k == kLaneH2D) ? lanes_per_dir_ : 1;
      lanes_[k].resize((size_t)count);
      if (k == kLaneHost) continue;
      for (auto& l : lanes_[k]) HL_CUDA(cudaStreamCreateWithPriority(&l.stream, cudaStreamNonBlocking, hi));
    }
    HL_CUDA(cudaEventCreateWithFlags(&order_ev_, cudaEventDisableTiming));
    if (stream_mem_ops_) {
      // First use of a stream memory operation on a fresh address is slow
      // (pcie-ccl-cuda/src/memory/completion_flag.cpp:231-234): pay it here.
      cudaStream_t s = lanes_[kLaneD2D][0].stream;
      CUresult r = drv->cuStreamWriteValue64((CUstream)s, (CUdeviceptr)(door_dev_ + 3), 1, 0);
      if (r == CUDA_SUCCESS) r = drv->cuStreamWaitValue64((CUstream)s, (CUdeviceptr)(door_dev_ + 3), 1, CU_STREAM_WAIT_VALUE_GEQ);
      if (r != CUDA_SUCCESS) {
        HL_INFO("stream memory operations unavailable (%s): using the doorbell kernel", drv->err(r));
        stream_mem_ops_ = false;
      }
      HL_CUDA(cudaStreamSynchronize(s));
    }
  } else {
    internal_ = (char*)aligned_alloc(4096, internal_bytes_);
    if (!internal_) return fail(hlSystemError, "cannot allocate %zu bytes of scratch", internal_bytes_);
    door_host_ = (volatile uint64_t*)aligned_alloc(64, 64);
    memset((void*)door_host_, 0, 64);
    for (int k = 0; k < kNumLaneKinds; ++k) lanes_[k].resize(1);
  }
  HL_CHECK(createHostPools());
  pool_.reset(new WorkerPool(phys_of_logical_, cfg.h2h_workers));
  thread_ = std::thread([this] { threadMain(); });
  return bs_->barrier(kBarExec);
}

hlResult_t PcieImpl::createHostPools() {
  host_base_.assign((size_t)numa_nodes_, nullptr);
  host_map_bytes_.assign((size_t)numa_nodes_, 0);
  host_registered_.assign((size_t)numa_nodes_, false);
  host_cuda_alloc_.assign((size_t)numa_nodes_, false);
  for (int m = 0; m < numa_nodes_; ++m) {
    int leader = -1;
    for (int q = 0; q < n_; ++q)
      if (numa_[(size_t)q] == m) {
        leader = q;
        break;
      }
    if (leader < 0) leader = 0;
    if (bs_->singleProcess()) {
      // threads share the address space: the leader allocates, the others learn the pointer
      char* p = nullptr;
      if (rank_ == leader) {
        pinThreadToNumaNode(phys_of_logical_[(size_t)m]);
        if (cuda_) {
          HL_CUDA(cudaHostAlloc((void**)&p, host_bytes_, cudaHostAllocPortable | cudaHostAllocMapped));
          host_cuda_alloc_[(size_t)m] = true;
        } else {
          p = (char*)aligned_alloc(4096, host_bytes_);
          if (!p) return fail(hlSystemError, "cannot allocate the host staging pool");
        }
      }
      uint64_t v = (uint64_t)(uintptr_t)p, all[kMaxRanks];
      HL_CHECK(bs_->allGather(&v, sizeof(v), all));
      host_base_[(size_t)m] = (char*)(uintptr_t)all[leader];
      host_map_bytes_[(size_t)m] = rank_ == leader ? host_bytes_ : 0;
      continue;
    }
    int fd = -1;
    if (rank_ == leader) {
      fd = memfd_create("hylink_host_pool", MFD_CLOEXEC);
      if (fd < 0) return fail(hlSystemError, "memfd_create: %s", strerror(errno));
      if (ftruncate(fd, (off_t)host_bytes_) != 0) return fail(hlSystemError, "ftruncate host pool (%zu bytes): %s", host_bytes_, strerror(errno));
    }
    int got = -1;
    HL_CHECK(bs_->broadcastFd(leader, fd, &got));
    void* p = mmap(nullptr, host_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, got, 0);
    if (got != fd && got >= 0) close(got);
    if (fd >= 0) close(fd);
    if (p == MAP_FAILED) return fail(hlSystemError, "mmap host pool: %s", strerror(errno));
    if (rank_ == leader) bindMemoryToNumaNode(p, host_bytes_, phys_of_logical_[(size_t)m]);
    host_base_[(size_t)m] = (char*)p;
    host_map_bytes_[(size_t)m] = host_bytes_;
    if (cuda_) {
      cudaError_t e = cudaHostRegister(p, host_bytes_, cudaHostRegisterPortable | cudaHostRegisterMapped);
      if (e != cudaSuccess) return fail(hlDeviceError, "cudaHostRegister(%zu bytes): %s", host_bytes_, cudaGetErrorString(e));
      host_registered_[(size_t)m] = true;
    }
  }
  host_dev_base_ = host_base_;
  if (cuda_) {
    for (int m = 0; m < numa_nodes_; ++m) {
      void* d = nullptr;
      if (host_base_[(size_t)m] && cudaHostGetDevicePointer(&d, host_base_[(size_t)m], 0) == cudaSuccess && d) host_dev_base_[(size_t)m] = (char*)d;
      else {
        cudaGetLastError();
        fuse_landing_ = false;   // a pool the device cannot address: landed chunks are copied, then reduced
      }
    }
    fuse_landing_ = fuse_landing_ && envBool({"HYLINK_PCIE_FUSE_LANDING"}, true);
  } else {
    fuse_landing_ = false;
  }
  if (small_slot_bytes_ && host_base_[0] && host_dev_base_[0]) {
    small_host_ = host_base_[0] + sched_host_bytes_;
    small_dev_ = host_dev_base_[0] + sched_host_bytes_;
    if (rank_ == 0) memset(small_host_, 0, 4096);   // flag words start at zero before anybody meets at the barrier below
    if (cudaEventCreateWithFlags(&small_ev_, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      small_host_ = small_dev_ = nullptr;
    }
  }
  return bs_->barrier(kBarExec);
}

PcieImpl::~PcieImpl() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
  pool_.reset();
  if (cuda_) {
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    for (int k = 0; k < kNumLaneKinds; ++k)
      for (auto& l : lanes_[k]) {
        for (auto& f : l.inflight)
          if (f.ev) cudaEventDestroy(f.ev);
        for (auto e : l.free_events) cudaEventDestroy(e);
        if (l.stream) cudaStreamDestroy(l.stream);
      }
    if (order_ev_) cudaEventDestroy(order_ev_);
    if (internal_) cudaFree(internal_);
    if (inplace_stage_) cudaFree(inplace_stage_);
    if (door_host_) cudaFreeHost((void*)door_host_);
  } else {
    free(internal_);
    free(inplace_stage_);
    free((void*)door_host_);
  }
  const bool peers_ok = bs_ && !bs_->anyFailed();
  if (peers_ok) bs_->barrier(kBarExec, 10000);  // nobody unmaps while a peer may still read
  for (int m = 0; m < (int)host_base_.size(); ++m) {
    if (!host_base_[(size_t)m]) continue;
    if (bs_->singleProcess()) {
      if (host_map_bytes_[(size_t)m]) {
        if (host_cuda_alloc_[(size_t)m]) cudaFreeHost(host_base_[(size_t)m]);
        else free(host_base_[(size_t)m]);
      }
    } else {
      if (host_registered_[(size_t)m]) cudaHostUnregister(host_base_[(size_t)m]);
      munmap(host_base_[(size_t)m], host_map_bytes_[(size_t)m]);
    }
  }
  if (cuda_) cudaGetLastError();
}

// ---------------------------------------------------------------------- plans
hlResult_t PcieImpl::getPlan(const std::string& collective, const std::string& forced_xml, int root, ir::InPlace ip,
                             int send_segs, int recv_segs, size_t bytes, std::shared_ptr<const Plan>* out) {
  const Config& cfg = Config::get();
  const bool small = bytes <= cfg.small_ir_max_bytes;
  std::string key = collective + "|" + std::to_string(root) + "|" + std::to_string((int)ip) + "|" + std::to_string(send_segs) +
                    "|" + std::to_string(recv_segs) + (small ? "|s" : "|l");
  if (!forced_xml.empty()) key = "xml:" + std::to_string(std::hash<std::string>()(forced_xml)) + key;
  auto it = plans_.find(key);
  if (it != plans_.end()) {
    *out = it->second;
    return hlSuccess;
  }
  std::shared_ptr<Plan> plan(new Plan());
  const std::string pattern = ir::numaPattern(numa_);
  if (!forced_xml.empty()) {
    HL_CHECK(ir::parseProgram(forced_xml, &plan->program));
    plan->source = "caller";
  } else {
    const std::string file_coll = collective == "broadcast" ? "broadcast_root" + std::to_string(root) : collective;
    std::string path;
    // `_direct` schedules copy between GPU pairs under one PCIe switch. They are chosen by topology (never with
    // NVLink between the GPUs) and need the peers' device buffers, which only threads of one process can reach.
    if (directVariantAllowed(file_coll, pattern, pairs_)) {
      if (bs_->singleProcess()) path = ir::findProgramFile(file_coll, pattern, "direct", "");
      else HL_DBG("topology allows %s_%s_direct.xml, but ranks are processes: host-relay schedule", file_coll.c_str(), pattern.c_str());
    }
    // A named variant (HYLINK_IR_VARIANT, e.g. host_reduce or single_d2h) comes from its own file, else from the generator.
    const std::string variant = envStr({"HYLINK_IR_VARIANT"}, "");
    if (path.empty() && !variant.empty()) path = ir::findProgramFile(file_coll, pattern, variant, "");
    if (path.empty() && variant.empty() && small) path = ir::findProgramFile(file_coll, pattern, "small", "");
    if (path.empty() && variant.empty()) path = ir::findProgramFile(file_coll, pattern, "", "");
    if (!path.empty()) {
      hlResult_t r = ir::loadProgramFile(path, &plan->program);
      if (r != hlSuccess) return r;
      plan->source = path;
    } else {
      HL_CHECK(ir::generate(collective, numa_, variant, root, &plan->program));
      plan->source = "generated";
    }
  }
  if (plan->program.nranks != n_) return fail(hlInvalidArgument, "schedule '%s' is for %d ranks, communicator has %d", plan->source.c_str(), plan->program.nranks, n_);
  ir::CompileOptions opt;
  opt.send_segs = send_segs;
  opt.recv_segs = recv_segs;
  opt.in_place = ip;
  opt.gpu_numa = numa_;
  hlResult_t r = ir::compile(plan->program, opt, &plan->graph);
  if (r != hlSuccess) return r;
  if (plan->graph.uses_remote_device && !bs_->singleProcess())
    return fail(hlUnsupported, "schedule '%s' reads a peer's device buffer: only available when ranks are threads of one process", plan->source.c_str());
  if (plan->graph.numa_nodes > numa_nodes_)
    return fail(hlInvalidArgument, "schedule '%s' names NUMA node %d, the communicator spans %d", plan->source.c_str(), plan->graph.numa_nodes - 1, numa_nodes_);
  HL_DBG("plan %s from %s: %zu nodes, %d host chunks", key.c_str(), plan->source.c_str(), plan->graph.nodes.size(), plan->graph.host_chunks);
  plans_[key] = plan;
  *out = plan;
  return hlSuccess;
}

// ---------------------------------------------------------------------- submit
hlResult_t PcieImpl::submit(const std::string& collective, const std::string& forced_xml, const void* send, void* recv,
                            size_t seg_count, size_t stride, int send_segs, int recv_segs, hlDataType_t t, hlRedOp_t op,
                            float scale, int root, hlStream_t stream) {
  if (last_result_.load() != hlSuccess) return fail((hlResult_t)last_result_.load(), "PCIe executor is in an error state");
  const size_t es = hlTypeSize(t);
  if (!es) return fail(hlInvalidArgument, "unknown data type");
  if (stride > seg_count) return fail(hlInvalidArgument, "stride %zu exceeds segment length %zu", stride, seg_count);
  if (stride == seg_count) return hlSuccess;
  const size_t active_total = seg_count - stride;
  if (stride == 0 && forced_xml.empty() && small_dev_) {
    bool handled = false;
    HL_CHECK(submitSmall(collective, send, recv, seg_count, send_segs, recv_segs, t, op, scale, root, (cudaStream_t)stream, &handled));
    if (handled) return hlSuccess;
  }
  // in-place detection by address
  ir::InPlace ip = ir::InPlace::None;
  const char* s = (const char*)send;
  char* r = (char*)recv;
  const size_t seg_bytes = seg_count * es;
  if (s == r) ip = ir::InPlace::Same;
  else if (collective == "allgather" && s == r + (size_t)rank_ * seg_bytes) ip = ir::InPlace::GatherSlot;
  else if (collective == "reducescatter" && r == s + (size_t)rank_ * seg_bytes) ip = ir::InPlace::ScatterSlot;
  else {
    const size_t sb = seg_bytes * (size_t)send_segs, rb = seg_bytes * (size_t)recv_segs;
    if (s < r + rb && r < s + sb) ip = ir::InPlace::Same;  // partial overlap: take the conservative route below
  }
  std::shared_ptr<const Plan> plan;
  hlResult_t pr = getPlan(collective, forced_xml, root, ip, send_segs, recv_segs, active_total * es * (size_t)std::max(send_segs, recv_segs), &plan);
  bool staged = false;
  if (pr == hlUnsupported && ip != ir::InPlace::None && strstr(lastError(), "in-place conflict")) {
    // The schedule would read user input after overwriting it: run it
    // out-of-place on a private copy of the send buffer.
    const size_t need = seg_bytes * (size_t)send_segs;
    if (inplace_stage_bytes_ < need) {
      if (cuda_) {
        if (inplace_stage_) cudaFree(inplace_stage_);
        HL_CUDA(cudaMalloc((void**)&inplace_stage_, need));
      } else {
        free(inplace_stage_);
        inplace_stage_ = (char*)aligned_alloc(4096, (need + 4095) & ~(size_t)4095);
      }
      inplace_stage_bytes_ = need;
    }
    if (cuda_) HL_CUDA(cudaMemcpyAsync(inplace_stage_, send, need, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    else memcpy(inplace_stage_, send, need);
    s = inplace_stage_;
    staged = true;
    HL_CHECK(getPlan(collective, forced_xml, root, ir::InPlace::None, send_segs, recv_segs, active_total * es, &plan));
  } else if (pr != hlSuccess) {
    return pr;
  }
  (void)staged;
  const ir::CompiledGraph& g = plan->graph;
  // rounds: the chunk pitch must fit the staging pools and the device scratch
  const int cps = std::max(1, g.input_chunks ? g.input_chunks / g.send_segs : g.output_chunks / std::max(1, g.recv_segs));
  size_t max_chunk_bytes = (size_t)1 << 40;
  if (g.host_chunks) max_chunk_bytes = std::min(max_chunk_bytes, sched_host_bytes_ / (size_t)g.host_chunks);
  const int dev_chunks = g.internal_chunks + g.scratch_chunks;
  if (dev_chunks) max_chunk_bytes = std::min(max_chunk_bytes, internal_bytes_ / (size_t)dev_chunks);
  max_chunk_bytes &= ~(size_t)255;
  if (max_chunk_bytes < 4096) return fail(hlInvalidArgument, "staging pools too small for schedule '%s' (%d host chunks)", plan->source.c_str(), g.host_chunks);
  const size_t max_active = (max_chunk_bytes / es) * (size_t)cps;

  const uint64_t door = next_door_++;
  cudaStream_t us = (cudaStream_t)stream;
  size_t done = 0;
  std::vector<Work> works;
  while (done < active_total) {
    Work w;
    const size_t act = std::min(max_active, active_total - done);
    HL_CHECK(ir::makeGeometry(g, seg_count, stride + done, act, es, &w.geo));
    w.plan = plan;
    w.send = s;
    w.recv = r;
    w.dtype = t;
    w.op = op == hlAvg ? hlSum : op;
    w.first_round = done == 0;
    w.last_round = done + act >= active_total;
    w.door_seq = door;
    w.name = collective;
    w.dma_lanes = dmaLanePolicy(collective.c_str(), active_total * es * (size_t)std::max(send_segs, recv_segs), n_, kMaxDmaLanes, Config::get().dma_lanes);
    done += act;
    if (!works.empty()) {
      w.prev_nslices = works.back().geo.nslices;
      // one pitch for all rounds of a message: the round guards order reuse chunk by chunk, so chunk c must cover the
      // same bytes of the staging pools in every round (the last round's chunks are shorter, not denser)
      w.geo.pitch_bytes = works.front().geo.pitch_bytes;
    }
    works.push_back(std::move(w));
  }
  const double total_scale = (double)(scale == 0.0f ? 1.0f : scale) * (op == hlAvg ? 1.0 / n_ : 1.0);
  const bool reduces = collective == "allreduce" || collective == "reducescatter";
  if (!cuda_ && reduces && total_scale != 1.0) {
    Work& lw = works.back();
    lw.host_scale = total_scale;
    lw.scale_off = stride;
    lw.scale_count = active_total;
    lw.scale_segs = recv_segs;
    lw.scale_seg_stride = seg_count;
  }
  {
    std::unique_lock<std::mutex> lk(mu_);
    const size_t depth = (size_t)std::max(1, Config::get().executor_queue_depth);
    if (!cv_done_.wait_for(lk, std::chrono::milliseconds(Config::get().executor_timeout_ms), [&] { return queue_.size() < depth || stop_; }))
      return fail(hlTimeout, "PCIe executor queue stayed full");
  }
  // Nothing below may fail between parking the stream and queueing the work.
  if (cuda_) {
    HL_CUDA(cudaSetDevice(device_));
    const CudaDriver* drv = CudaDriver::get();
    if (stream_mem_ops_) {
      HL_CU(drv, cuStreamWriteValue64((CUstream)us, (CUdeviceptr)(door_dev_ + 0), door, 0));
      HL_CU(drv, cuStreamWaitValue64((CUstream)us, (CUdeviceptr)(door_dev_ + 1), door, CU_STREAM_WAIT_VALUE_GEQ));
    } else {
      HL_CHECK(nvl::launchDoorbell(door_dev_ + 0, door, door_dev_ + 1, door, (uint64_t)Config::get().executor_timeout_ms * 1000000ull,
                                   door_dev_ + 2, collective.c_str(), us));
      kernel_launches_++;
    }
  }
  {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& w : works) {
      w.seq = next_seq_++;
      queue_.push_back(std::move(w));
    }
  }
  cv_.notify_all();
  if (cuda_ && reduces && total_scale != 1.0) {
    // the stream is parked behind the doorbell here, so this runs after completion
    for (int sgi = 0; sgi < recv_segs; ++sgi) {
      nvl::ReduceLandingArgs a;
      memset(&a, 0, sizeof(a));
      a.dst = r + ((size_t)sgi * seg_count + stride) * es;
      a.src[0] = a.dst;
      a.nsrc = 1;
      a.count = active_total;
      a.dtype = t;
      a.op = hlSum;
      a.scale = (float)total_scale;
      HL_CHECK(nvl::launchReduceLanding(a, 0, us));
      kernel_launches_++;
    }
  }
  return hlSuccess;
}


// ---------------------------------------------------------------------- small messages
// Below HYLINK_SMALL_MSG_THRESHOLD_BYTES (1 MiB per rank) the graph executor's fixed costs dominate: a doorbell round
// trip to the CPU thread, one event per slice, a cross-rank barrier. Small calls therefore never reach that thread.
// Everything is enqueued on the caller's stream and ordered by stream memory operations on flag words that live in
// the shared pinned pool, so that GPUs signal one another through host memory without any CPU in the path:
//   wait  done[p][q] >= s - 2 for every q   (the slots of this parity are free: call s - 2 has been read everywhere)
//   copy  the input into slot [p][rank] of the pool (copy engine, device to host)
//   write ready[p][rank] = s ; wait ready[p][q] >= s for every q
//   ONE launch of the landing-reduce kernel that reads all n slots over PCIe and writes the result (all-reduce,
//   reduce-scatter), or n copy-engine transfers out of the slots (all-gather, all-to-all, broadcast)
//   write done[p][rank] = s
// (p = s & 1). The flag waits have no time-out of their own, so the executor thread keeps a list of the calls in
// flight and, when one is overdue, releases every flag from the CPU (they are host memory) and latches an error:
// a stream is never left parked.
// Parity: the reference's small-message executor (pcie-ccl-cuda/src/fastpath/small_message_executor.cpp:239-284,
// 555-588, 766-856) has a thread per communicator, three streams and per-slot scratch, negotiates "all direct" against
// "host staged" per call through shared memory and ends with a shm barrier; its direct mode copies between peers,
// which on this machine is the dedicated-link path's job.
hlResult_t PcieImpl::submitSmall(const std::string& collective, const void* send, void* recv, size_t seg_count, int send_segs, int recv_segs,
                                 hlDataType_t t, hlRedOp_t op, float scale, int root, cudaStream_t us, bool* handled) {
  *handled = false;
  const size_t es = hlTypeSize(t);
  const size_t in_bytes = seg_count * es * (size_t)send_segs;
  if (!cuda_ || !small_dev_ || !stream_mem_ops_ || n_ < 2 || n_ > 8 || in_bytes == 0 || in_bytes > small_slot_bytes_) return hlSuccess;
  if (in_bytes > Config::get().small_msg_threshold_bytes) return hlSuccess;
  const bool reduces = collective == "allreduce" || collective == "reducescatter";
  const bool is_int = !(t == hlFloat16 || t == hlBfloat16 || t == hlFloat32 || t == hlFloat64);
  if (reduces && op == hlAvg && is_int) return hlSuccess;   // integer averages divide: the ordinary path does that
  if (!reduces && collective != "allgather" && collective != "alltoall" && collective != "broadcast") return hlSuccess;
  const CudaDriver* drv = CudaDriver::get();
  if (!drv) return hlSuccess;
  *handled = true;
  TraceScope range("pcie", "small-message", rank_);
  range.setBytes((long long)in_bytes);
  HL_CUDA(cudaSetDevice(device_));
  const uint64_t s = ++small_seq_;
  const int p = (int)(s & 1);
  auto dptr = [&](bool done, int q) { return (CUdeviceptr)(uintptr_t)smallFlag(done, p, q, true); };
  auto slot = [&](int q, bool device) { return (device ? small_dev_ : small_host_) + 4096 + ((size_t)p * n_ + (size_t)q) * small_slot_bytes_; };
  {
    std::lock_guard<std::mutex> lk(mu_);
    small_pending_.push_back({s, nowNs()});
    small_used_ = true;
  }
  cv_.notify_all();   // the watchdog starts counting
  if (s > 2)
    for (int q = 0; q < n_; ++q) HL_CU(drv, cuStreamWaitValue64((CUstream)us, dptr(true, q), s - 2, CU_STREAM_WAIT_VALUE_GEQ));
  const bool contributes = collective != "broadcast" || rank_ == root;
  if (contributes) {
    HL_CUDA(cudaMemcpyAsync(slot(rank_, false), send, in_bytes, cudaMemcpyDeviceToHost, us));
    copy_ops_++;
  }
  HL_CU(drv, cuStreamWriteValue64((CUstream)us, dptr(false, rank_), s, 0));
  for (int q = 0; q < n_; ++q)
    if (q != rank_) HL_CU(drv, cuStreamWaitValue64((CUstream)us, dptr(false, q), s, CU_STREAM_WAIT_VALUE_GEQ));
  const size_t seg_bytes = seg_count * es;
  if (reduces) {
    nvl::ReduceLandingArgs a;
    memset(&a, 0, sizeof(a));
    a.dst = recv;
    a.nsrc = n_;
    for (int q = 0; q < n_; ++q) a.src[q] = slot(q, true) + (collective == "reducescatter" ? (size_t)rank_ * seg_bytes : 0);
    a.count = seg_count;
    a.dtype = t;
    a.op = op == hlAvg ? hlSum : op;
    a.scale = (scale == 0.0f ? 1.0f : scale) * (op == hlAvg ? 1.0f / (float)n_ : 1.0f);
    HL_CHECK(nvl::launchReduceLanding(a, 0, us));
    kernel_launches_++;
  } else if (collective == "broadcast") {
    if (rank_ != root || recv != send) {
      HL_CUDA(cudaMemcpyAsync(recv, slot(root, false), in_bytes, cudaMemcpyHostToDevice, us));
      copy_ops_++;
    }
  } else {
    for (int k = 0; k < n_; ++k) {
      const int q = (rank_ + k) % n_;
      const char* from = slot(q, false) + (collective == "alltoall" ? (size_t)rank_ * seg_bytes : 0);
      HL_CUDA(cudaMemcpyAsync((char*)recv + (size_t)q * seg_bytes, from, seg_bytes, cudaMemcpyHostToDevice, us));
      copy_ops_++;
    }
  }
  HL_CU(drv, cuStreamWriteValue64((CUstream)us, dptr(true, rank_), s, 0));
  HL_CUDA(cudaEventRecord(small_ev_, us));
  small_calls_++;
  (void)recv_segs;
  return hlSuccess;
}

// Executor thread, between work items: forget the small calls that are through, release everything when one is overdue.
void PcieImpl::watchSmallCalls() {
  if (!small_host_) return;
  const int limit_ms = Config::get().small_msg_timeout_ms > 0 ? Config::get().small_msg_timeout_ms : Config::get().executor_timeout_ms;
  const uint64_t limit = (uint64_t)limit_ms * 1000000ull;
  bool overdue = false;
  {
    std::lock_guard<std::mutex> lk(mu_);
    while (!small_pending_.empty()) {
      const SmallPending& f = small_pending_.front();
      const uint64_t seen = __atomic_load_n((uint64_t*)smallFlag(true, (int)(f.seq & 1), rank_, false), __ATOMIC_ACQUIRE);
      if (seen >= f.seq) {
        small_pending_.pop_front();
        continue;
      }
      overdue = nowNs() - f.t_ns > limit || shared_->failed.load(std::memory_order_relaxed);
      break;
    }
  }
  if (overdue && last_result_.load() == hlSuccess) {
    HL_ERR("rank %d: a small-message collective did not complete within %d ms: releasing every flag", rank_, limit_ms);
    for (int k = 0; k < 4 * kMaxRanks; ++k) __atomic_store_n((uint64_t*)small_host_ + k, kReleaseAll, __ATOMIC_RELEASE);
    fail(hlTimeout, "small-message collective timed out (a peer never arrived)");
    failAll(hlTimeout);
    std::lock_guard<std::mutex> lk(mu_);
    small_pending_.clear();
  }
}

hlResult_t PcieImpl::drain() {
  if (small_used_ && small_ev_) {
    // small calls live on the caller's streams only; the watchdog releases their waits if a peer is lost
    cudaError_t e = cudaEventSynchronize(small_ev_);
    if (e != cudaSuccess) return fail(hlDeviceError, "drain: %s", cudaGetErrorString(e));
  }
  std::unique_lock<std::mutex> lk(mu_);
  const uint64_t target = next_door_ - 1;
  const int tmo = Config::get().executor_timeout_ms;
  if (!cv_done_.wait_for(lk, std::chrono::milliseconds(tmo), [&] { return completed_door_.load() >= target || last_result_.load() != hlSuccess; }))
    return fail(hlTimeout, "drain: PCIe executor did not finish within %d ms", tmo);
  return (hlResult_t)last_result_.load();
}

// ---------------------------------------------------------------------- executor thread
void PcieImpl::releaseDoorbell(uint64_t value) {
  __atomic_store_n((uint64_t*)(door_host_ + 1), value, __ATOMIC_RELEASE);  // plain CPU store releases the parked stream
}

void PcieImpl::failAll(hlResult_t r) {
  last_result_.store(r);
  shared_->failed.store(1);
  bs_->latchFailure();
  releaseDoorbell(kReleaseAll);  // never leave a user stream parked
  std::lock_guard<std::mutex> lk(mu_);
  queue_.clear();
  completed_door_.store(next_door_);
  cv_done_.notify_all();
}

void PcieImpl::threadMain() {
  if (cuda_) cudaSetDevice(device_);
  pinThreadToNumaNode(phys_of_logical_[(size_t)numa_[(size_t)rank_]]);
  for (;;) {
    Work w;
    {
      std::unique_lock<std::mutex> lk(mu_);
      // with small calls in flight the thread also wakes up by itself to look after their deadlines
      if (small_pending_.empty()) cv_.wait(lk, [&] { return stop_ || !queue_.empty() || !small_pending_.empty(); });
      else cv_.wait_for(lk, std::chrono::milliseconds(50), [&] { return stop_ || !queue_.empty(); });
      if (queue_.empty()) {
        if (stop_) return;
        lk.unlock();
        watchSmallCalls();
        continue;
      }
      w = std::move(queue_.front());
      queue_.pop_front();
    }
    cv_done_.notify_all();
    hlResult_t r = hlSuccess;
    if (w.first_round) r = waitReady(w);
    if (r == hlSuccess) r = runWork(w);
    if (r != hlSuccess) {
      HL_ERR("rank %d: PCIe collective '%s' failed: %s (%s)", rank_, w.name.c_str(), hlGetErrorString(r), lastError());
      failAll(r);
      continue;
    }
    if (w.last_round) {
      if (w.host_scale != 1.0) {
        const size_t es = hlTypeSize(w.dtype);
        for (int sgi = 0; sgi < w.scale_segs; ++sgi)
          hostScale(w.recv + ((size_t)sgi * w.scale_seg_stride + w.scale_off) * es, w.scale_count, w.dtype, w.host_scale);
      }
      releaseDoorbell(w.door_seq);
      completed_door_.store(w.door_seq);
      {
        std::lock_guard<std::mutex> lk(mu_);
      }
      cv_done_.notify_all();
    }
  }
}

hlResult_t PcieImpl::waitReady(const Work& w) {
  if (!cuda_) return hlSuccess;
  // The GPU writes ready = door_seq when everything queued before the
  // collective on the caller's stream has finished: inputs are valid.
  const uint64_t t0 = nowNs();
  const uint64_t limit = (uint64_t)Config::get().executor_timeout_ms * 1000000ull;
  uint32_t spins = 0;
  while (__atomic_load_n((uint64_t*)(door_host_ + 0), __ATOMIC_ACQUIRE) < w.door_seq) {
    if ((++spins & 63) == 0) {
      if (shared_->failed.load(std::memory_order_relaxed)) return fail(hlRemoteError, "a peer's executor failed");
      if (nowNs() - t0 > limit) return fail(hlTimeout, "doorbell: the caller's stream never reached the collective");
      if (spins > 4096) std::this_thread::yield();
    } else {
      cpuRelax();
    }
  }
  return hlSuccess;
}

cudaEvent_t PcieImpl::getEvent(Lane& l) {
  if (!l.free_events.empty()) {
    cudaEvent_t e = l.free_events.back();
    l.free_events.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
  return e;
}

Lane& PcieImpl::laneFor(ir::Op op, int salt, int active) {
  if (!cuda_) return lanes_[kLaneHost][0];
  const size_t use = (size_t)std::max(1, std::min(active, (int)lanes_[kLaneD2H].size()));
  switch (op) {
    case ir::Op::D2H: return lanes_[kLaneD2H][(size_t)salt % use];
    case ir::Op::H2D: return lanes_[kLaneH2D][(size_t)salt % use];
    case ir::Op::D2D: return lanes_[kLaneD2D][0];
    case ir::Op::D2DReduce: return lanes_[kLaneReduce][0];
    default: return lanes_[kLaneHost][0];
  }
}

char* PcieImpl::resolve(const Work& w, const ir::Loc& l, size_t* len_bytes, bool* remote_pending) {
  const ir::Geometry& geo = w.geo;
  const ir::CompiledGraph& g = w.plan->graph;
  const size_t full = geo.chunk_elems * geo.elem;
  *len_bytes = full;
  if (l.space == ir::Buf::Host) return host_base_[(size_t)l.owner] + (size_t)l.chunk * geo.pitch_bytes;
  char* base = nullptr;
  int slot = 0;
  switch (l.space) {
    case ir::Buf::Input: slot = 0; base = (char*)w.send; break;
    case ir::Buf::Output: slot = 1; base = w.recv; break;
    case ir::Buf::Scratch: slot = 2; base = internal_ + (size_t)g.internal_chunks * geo.pitch_bytes; break;
    default: slot = 3; base = internal_; break;
  }
  if (l.owner != rank_) {
    // a peer's device buffer (threads-as-ranks mode): its executor publishes the bases when its inputs are ready
    if (shared_->ready_seq[l.owner].load(std::memory_order_acquire) < w.seq) {
      *remote_pending = true;
      return nullptr;
    }
    base = (char*)(uintptr_t)shared_->ptrs[l.owner][slot].load(std::memory_order_acquire);
  }
  if (l.space == ir::Buf::Input || l.space == ir::Buf::Output) {
    size_t off = 0, bytes = 0;
    ir::deviceChunkSpan(geo, l.space == ir::Buf::Input ? geo.cps_in : geo.cps_out, l.chunk, &off, &bytes);
    *len_bytes = bytes;
    return base + off;
  }
  return base + (size_t)l.chunk * geo.pitch_bytes;
}

hlResult_t PcieImpl::runWork(const Work& w) {
  const ir::CompiledGraph& g = w.plan->graph;
  const ir::Geometry& geo = w.geo;
  const std::vector<int>& mine = g.by_rank[(size_t)rank_];
  const int ns = geo.nslices;
  const uint64_t tag = w.seq << kSeqShift;
  TraceScope whole("pcie", w.name.c_str(), rank_);
  whole.setBytes((long long)(w.geo.chunk_elems * w.geo.elem) * std::max(1, std::max(g.input_chunks, g.output_chunks)));
  struct Local {
    int issued = 0, done = 0;
  };
  std::vector<Local> st(mine.size());
  auto publish = [&](int slot) { shared_->progress[g.nodes[(size_t)mine[(size_t)slot]].id].store(tag | (uint64_t)st[(size_t)slot].done, std::memory_order_release); };
  auto progressOf = [&](int node_id) -> int {
    const uint64_t v = shared_->progress[node_id].load(std::memory_order_acquire);
    const uint64_t t = v >> kSeqShift;
    if (t == w.seq) return (int)(v & kSliceMask);
    return t > w.seq ? ns : 0;
  };
  // publish this rank's bases for peers that read them directly (threads-as-ranks mode)
  shared_->ptrs[rank_][0].store((uint64_t)(uintptr_t)w.send, std::memory_order_relaxed);
  shared_->ptrs[rank_][1].store((uint64_t)(uintptr_t)w.recv, std::memory_order_relaxed);
  shared_->ptrs[rank_][2].store((uint64_t)(uintptr_t)(internal_ + (size_t)g.internal_chunks * geo.pitch_bytes), std::memory_order_relaxed);
  shared_->ptrs[rank_][3].store((uint64_t)(uintptr_t)internal_, std::memory_order_relaxed);
  shared_->ready_seq[rank_].store(w.seq, std::memory_order_release);

  // Landing fusion: an H2D whose only reader is a D2DReduce of this rank is not copied at all; the reduce kernel
  // reads the pinned host chunk over PCIe itself, and several such reduces into one destination are folded in ONE
  // launch (up to eight sources) when their data is there together. The H2D node still exists for everybody who
  // waits for it: it is reported done, slice by slice, when the reduce that consumed the host chunk is done.
  const bool fuse = fuse_landing_ && !Config::get().skip_dma;
  std::vector<int> local_of(g.nodes.size(), -1);
  for (size_t i = 0; i < mine.size(); ++i) local_of[(size_t)mine[i]] = (int)i;
  size_t remaining = 0;
  for (size_t i = 0; i < mine.size(); ++i) {
    const ir::Node& n = g.nodes[(size_t)mine[i]];
    if (n.op == ir::Op::NOP || n.skip || Config::get().skip_dma) {
      st[i].issued = st[i].done = ns;
      publish((int)i);
    } else {
      st[i].done = 0;
      if (fuse && n.fused_into >= 0) st[i].issued = ns;   // never issued on its own
      publish((int)i);
      ++remaining;
    }
  }
  // Rounds of one message reuse the staging chunks without a barrier in between: a node that overwrites a chunk waits
  // (before its first slice) until everybody who used that chunk in the previous round is through with it there.
  static const bool round_barrier = envBool({"HYLINK_PCIE_ROUND_BARRIER"}, false);
  auto doneInPreviousRound = [&](int node_id) -> bool {
    const uint64_t v = shared_->progress[node_id].load(std::memory_order_acquire);
    const uint64_t t = v >> kSeqShift;
    if (t >= w.seq) return true;                       // its rank is already in this round: it finished the last one
    return t + 1 == w.seq && (int)(v & kSliceMask) >= w.prev_nslices;
  };
  auto guardsClear = [&](const ir::Node& n) -> bool {
    if (w.first_round || round_barrier) return true;
    for (int gnode : n.round_guards)
      if (!doneInPreviousRound(gnode)) return false;
    return true;
  };
  // inputs of slice k of a fused reduce: its own wait list with the H2D node replaced by what the H2D waited for,
  // and (when folded behind `after`) without the reduce that precedes it in the same launch
  auto fusedReady = [&](const ir::Node& r, int k, int after) -> bool {
    for (int d : r.wait_for) {
      if (d == after) continue;
      if (d == r.fused_h2d) {
        for (int dd : g.nodes[(size_t)d].wait_for)
          if (progressOf(dd) < k + 1) return false;
        continue;
      }
      if (progressOf(d) < k + 1) return false;
    }
    return true;
  };
  const uint64_t t0 = nowNs();
  const uint64_t limit = (uint64_t)Config::get().executor_timeout_ms * 1000000ull;
  uint32_t idle = 0;
  auto complete = [&](InFlight& f) {
    for (int extra : f.also) {
      Local& x = st[(size_t)extra];
      ++x.done;
      publish(extra);
      if (x.done == ns) --remaining;
    }
    Local& l = st[(size_t)f.node_slot];
    ++l.done;
    publish(f.node_slot);
    if (l.done == ns) --remaining;
    if (traceEnabled()) traceComplete("dma", ir::opName(g.nodes[(size_t)mine[(size_t)f.node_slot]].op), rank_, f.t0_ns, nowNs(), (long long)f.bytes);
  };
  struct RangeRun {
    int node_slot = -1;
    std::shared_ptr<HostTicket> ticket;
    uint64_t t0_ns = 0;
    size_t bytes = 0;
  };
  std::vector<RangeRun> ranges;   // H2H nodes that a worker team owns (worker_pool.h: RangeJob)
  static const bool range_jobs = envBool({"HYLINK_H2H_RANGE_JOBS"}, true);
  static const int range_team = (int)envInt({"HYLINK_H2H_RANGE_THREADS"}, 4);
  while (remaining) {
    bool progressed = false;
    // 1a. nodes owned by worker teams: their progress word is written by the workers
    for (size_t ri = 0; ri < ranges.size();) {
      RangeRun& rr = ranges[ri];
      if (rr.ticket->failed.load()) return fail(hlInternalError, "host range job failed (a wait ran out, a peer failed, or unsupported type/op)");
      Local& l = st[(size_t)rr.node_slot];
      const int now_done = progressOf(g.nodes[(size_t)mine[(size_t)rr.node_slot]].id);
      if (now_done > l.done) {
        l.done = now_done;
        progressed = true;
      }
      if (l.done >= ns && rr.ticket->done()) {
        --remaining;
        if (traceEnabled()) traceComplete("h2h", ir::opName(g.nodes[(size_t)mine[(size_t)rr.node_slot]].op), rank_, rr.t0_ns, nowNs(), (long long)rr.bytes);
        ranges[ri] = std::move(ranges.back());
        ranges.pop_back();
        continue;
      }
      ++ri;
    }
    // 1. retire finished transfers, lane by lane, in issue order
    for (int k = 0; k < kNumLaneKinds; ++k)
      for (auto& lane : lanes_[k]) {
        while (!lane.inflight.empty()) {
          InFlight& f = lane.inflight.front();
          bool fin = false;
          if (f.ticket) {
            fin = f.ticket->done();
            if (fin && f.ticket->failed.load()) return fail(hlInternalError, "host reduce failed (unsupported type/op)");
          } else {
            cudaError_t e = cudaEventQuery(f.ev);
            if (e == cudaSuccess) fin = true;
            else if (e != cudaErrorNotReady) return fail(hlDeviceError, "cudaEventQuery: %s", cudaGetErrorString(e));
          }
          if (!fin) break;
          if (f.ev) lane.free_events.push_back(f.ev);
          complete(f);
          lane.inflight.pop_front();
          progressed = true;
        }
      }
    // 2. issue every slice whose inputs are there
    for (size_t i = 0; i < mine.size(); ++i) {
      Local& l = st[i];
      if (l.issued >= ns) continue;
      const ir::Node& n = g.nodes[(size_t)mine[i]];
      Lane& lane = laneFor(n.op, (int)i, w.dma_lanes);
      while (l.issued < ns && (int)lane.inflight.size() < kLaneDepth) {
        const int k = l.issued;
        if (k == 0 && !guardsClear(n)) break;
        if (fuse && n.op == ir::Op::D2DReduce && n.fused_h2d >= 0) {
          if (!fusedReady(n, k, -1)) break;
          size_t dlen = 0, hlen = 0;
          bool pending = false;
          char* dst = resolve(w, n.dst, &dlen, &pending);
          const size_t off = (size_t)k * geo.slice_bytes;
          const size_t len = off >= dlen ? 0 : std::min(geo.slice_bytes, dlen - off);
          InFlight f;
          f.node_slot = (int)i;
          f.bytes = len;
          f.t0_ns = nowNs();
          nvl::ReduceLandingArgs a;
          memset(&a, 0, sizeof(a));
          a.dst = dst + off;
          a.accumulate = 1;
          a.count = len / geo.elem;
          a.dtype = w.dtype;
          a.op = w.op;
          a.scale = 1.0f;
          auto hostSrc = [&](const ir::Node& h2d) {
            (void)resolve(w, h2d.src, &hlen, &pending);
            return host_dev_base_[(size_t)h2d.src.owner] + (size_t)h2d.src.chunk * geo.pitch_bytes + off;
          };
          a.src[a.nsrc++] = hostSrc(g.nodes[(size_t)n.fused_h2d]);
          f.also.push_back(local_of[(size_t)n.fused_h2d]);
          // fold the reduces that follow into the same destination and whose landed data is there already
          int prev = n.id;
          for (size_t j = i + 1; j < mine.size() && a.nsrc < 8; ++j) {
            const ir::Node& m = g.nodes[(size_t)mine[j]];
            if (m.op != ir::Op::D2DReduce || m.fused_h2d < 0 || !(m.dst == n.dst)) continue;
            if (st[j].issued != k || !fusedReady(m, k, prev)) break;   // the chain is ordered: stop at the first that is not ready
            a.src[a.nsrc++] = hostSrc(g.nodes[(size_t)m.fused_h2d]);
            f.also.push_back((int)j);
            f.also.push_back(local_of[(size_t)m.fused_h2d]);
            ++st[j].issued;
            prev = m.id;
            folded_sources_++;
          }
          if (len == 0) {
            f.ticket = std::make_shared<HostTicket>();
          } else {
            HL_CHECK(nvl::launchReduceLanding(a, 0, lane.stream));
            kernel_launches_++;
            fused_slices_++;
            f.ev = getEvent(lane);
            cudaError_t e = cudaEventRecord(f.ev, lane.stream);
            if (e != cudaSuccess) return fail(hlDeviceError, "cudaEventRecord: %s", cudaGetErrorString(e));
          }
          lane.inflight.push_back(std::move(f));
          ++l.issued;
          progressed = true;
          continue;
        }
        bool ready = true;
        for (int d : n.wait_for)
          if (progressOf(d) < k + 1) {
            ready = false;
            break;
          }
        if (!ready) break;
        size_t slen = 0, dlen = 0, s2len = 0;
        bool pending = false;
        char* src = resolve(w, n.src, &slen, &pending);
        char* dst = resolve(w, n.dst, &dlen, &pending);
        char* src2 = n.op == ir::Op::H2HReduce ? resolve(w, n.src2, &s2len, &pending) : nullptr;
        if (pending) break;
        const size_t node_len = std::min(slen, dlen);
        if (k == 0 && range_jobs && ns > 1 && (n.op == ir::Op::H2H || n.op == ir::Op::H2HReduce)) {
          // The whole node goes to a team of workers that follows the inputs slice by slice and publishes the node's
          // progress word itself; this thread only reads the word back (step 1).
          RangeJob job;
          job.kind = n.op == ir::Op::H2HReduce ? HostJob::Reduce : HostJob::Copy;
          job.dst = dst;
          job.a = src;
          job.b = src2;
          job.bytes = n.op == ir::Op::H2HReduce ? std::min(node_len, s2len) : node_len;
          job.slice_bytes = geo.slice_bytes;
          job.nslices = ns;
          job.dtype = w.dtype;
          job.op = w.op;
          job.non_temporal = true;
          job.numa = n.dst.space == ir::Buf::Host ? n.dst.owner : numa_[(size_t)rank_];
          job.team = range_team;
          job.out = &shared_->progress[n.id];
          for (int d : n.wait_for) job.deps.push_back(&shared_->progress[d]);
          job.seq = w.seq;
          job.seq_shift = kSeqShift;
          job.abort = &shared_->failed;
          job.deadline_ns = t0 + limit;
          RangeRun rr;
          rr.node_slot = (int)i;
          rr.ticket = std::make_shared<HostTicket>();
          rr.t0_ns = nowNs();
          rr.bytes = job.bytes;
          pool_->submitRange(job, rr.ticket);
          ranges.push_back(std::move(rr));
          range_jobs_++;
          l.issued = ns;
          progressed = true;
          break;
        }
        const size_t off = (size_t)k * geo.slice_bytes;
        const size_t len = off >= node_len ? 0 : std::min(geo.slice_bytes, node_len - off);
        {
          // host-side fault injection: the failure is made here, where the transfer would have been issued
          const Config& cfg = Config::get();
          if ((cfg.fault_copy_error_at || cfg.fault_stall_at) && (cfg.fault_rank < 0 || cfg.fault_rank == rank_)) {
            const long op_index = ++issued_ops_;
            if (op_index == cfg.fault_stall_at) std::this_thread::sleep_for(std::chrono::milliseconds(cfg.fault_stall_ms));
            if (op_index == cfg.fault_copy_error_at)
              return fail(hlDeviceError, "%s slice: injected failure of transfer %ld (HYLINK_FAULT_INJECT)", ir::opName(n.op), op_index);
          }
        }
        InFlight f;
        f.node_slot = (int)i;
        f.bytes = len;
        f.t0_ns = nowNs();
        const bool host_op = !cuda_ || n.op == ir::Op::H2H || n.op == ir::Op::H2HReduce;
        if (len == 0) {
          f.ticket = std::make_shared<HostTicket>();  // empty trailing slice of a short chunk: done at once
        } else if (host_op) {
          HostJob job;
          job.dst = dst + off;
          job.bytes = len;
          job.dtype = w.dtype;
          job.op = w.op;
          job.numa = n.dst.space == ir::Buf::Host ? n.dst.owner : numa_[(size_t)rank_];
          if (n.op == ir::Op::H2HReduce) {
            job.kind = HostJob::Reduce;
            job.a = src + off;
            job.b = src2 + off;
          } else if (n.op == ir::Op::D2DReduce) {
            job.kind = HostJob::Reduce;
            job.a = dst + off;
            job.b = src + off;
          } else {
            job.kind = HostJob::Copy;
            job.a = src + off;
            job.non_temporal = n.dst.space == ir::Buf::Host;
          }
          f.ticket = std::make_shared<HostTicket>();
          pool_->submit(job, f.ticket);
        } else {
          cudaError_t e = cudaSuccess;
          if (n.op == ir::Op::D2DReduce) {
            nvl::ReduceLandingArgs a;
            memset(&a, 0, sizeof(a));
            a.dst = dst + off;
            a.src[0] = src + off;
            a.nsrc = 1;
            a.accumulate = 1;
            a.count = len / geo.elem;
            a.dtype = w.dtype;
            a.op = w.op;
            a.scale = 1.0f;
            HL_CHECK(nvl::launchReduceLanding(a, 0, lane.stream));
            kernel_launches_++;
          } else {
            const cudaMemcpyKind kind = n.op == ir::Op::D2H ? cudaMemcpyDeviceToHost : (n.op == ir::Op::H2D ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice);
            e = cudaMemcpyAsync(dst + off, src + off, len, kind, lane.stream);
            copy_ops_++;
          }
          if (e != cudaSuccess) return fail(hlDeviceError, "%s slice: %s", ir::opName(n.op), cudaGetErrorString(e));
          f.ev = getEvent(lane);
          e = cudaEventRecord(f.ev, lane.stream);
          if (e != cudaSuccess) return fail(hlDeviceError, "cudaEventRecord: %s", cudaGetErrorString(e));
        }
        lane.inflight.push_back(std::move(f));
        ++l.issued;
        progressed = true;
      }
    }
    if (progressed) {
      idle = 0;
      continue;
    }
    if ((++idle & 255u) == 0) {
      if (shared_->failed.load(std::memory_order_relaxed)) return fail(hlRemoteError, "a peer's executor failed");
      if (nowNs() - t0 > limit) {
        std::string stuck;
        for (size_t i = 0; i < mine.size() && stuck.size() < 400; ++i)
          if (st[i].done < ns) {
            const ir::Node& n = g.nodes[(size_t)mine[i]];
            stuck += std::string(" ") + ir::opName(n.op) + "@line" + std::to_string(n.line) + ":" + std::to_string(st[i].done) + "/" + std::to_string(ns);
          }
        return fail(hlTimeout, "schedule stalled after %d ms; unfinished nodes:%s", Config::get().executor_timeout_ms, stuck.c_str());
      }
      if (idle > 2048) std::this_thread::yield();
    } else {
      cpuRelax();
    }
  }
  bs_->heartbeat();
  // Peers may still be reading this rank's staging chunks (and, for direct schedules, its device buffers): after the
  // last round of a message nobody moves on before everyone is done. Between the rounds of one message the round
  // guards order the reuse of every chunk, so no barrier is needed there.
  if (!w.last_round && !round_barrier && !g.uses_remote_device) return hlSuccess;
  return bs_->barrier(kBarExec, Config::get().executor_timeout_ms);
}

int dmaLanePolicy(const char* collective, size_t message_bytes, int world, int max_lanes, int forced) {
  const int limit = std::max(1, max_lanes);
  auto clamp = [limit](int v) { return std::max(1, std::min(v, limit)); };
  if (message_bytes == 0) return 1;
  if (forced > 0) return clamp(forced);
  const std::string c = collective ? collective : "";
  const size_t mib = (size_t)1 << 20;
  if (c == "allgather") return clamp(message_bytes <= 16 * mib ? 4 : 2);
  if (c == "reducescatter") return clamp(message_bytes <= 32 * mib ? 4 : (message_bytes <= 128 * mib ? 3 : 2));
  if (c == "allreduce") return clamp(message_bytes <= 16 * mib ? 4 : (message_bytes <= 64 * mib ? 3 : 2));
  if (c == "alltoall") return clamp(world >= 8 ? (message_bytes <= 4 * mib ? 8 : 4) : (message_bytes <= 16 * mib ? 4 : 2));   // n - 1 peers per direction
  return 1;
}

// ====================================================================== facade
namespace {
std::mutex g_reg_mu;
std::vector<PcieImpl*> g_registry;
}  // namespace

PciePath::~PciePath() {
  {
    std::lock_guard<std::mutex> lk(g_reg_mu);
    g_registry.erase(std::remove(g_registry.begin(), g_registry.end(), impl_), g_registry.end());
  }
  delete impl_;
}

size_t PciePath::ctrlBytes(int) { return (sizeof(SharedArea) + 4095) & ~(size_t)4095; }

hlResult_t PciePath::create(Bootstrap* bs, int device, void* ctrl_area, PciePath** out) {
  std::unique_ptr<PciePath> p(new PciePath());
  p->impl_ = new PcieImpl(bs, device, ctrl_area);
  HL_CHECK(p->impl_->init());
  {
    std::lock_guard<std::mutex> lk(g_reg_mu);
    g_registry.push_back(p->impl_);
  }
  *out = p.release();
  return hlSuccess;
}

hlResult_t PciePath::allReduce(const void* send, void* recv, size_t count, hlDataType_t t, hlRedOp_t op, float scale, hlStream_t stream) {
  // Optional composition (HYLINK_PCIE_AR_COMPOSE=1): an out-of-place all-reduce whose count divides by the rank count
  // runs as reduce-scatter into this rank's slot of the output followed by an in-place all-gather, the way
  // pcie-ccl-ascend/src/api/pccl_api.cpp:572-607 does. Off by default: the all-reduce schedules here already are a
  // reduce-scatter phase and a gather phase in ONE graph, without the barrier between two messages.
  static const bool compose = envBool({"HYLINK_PCIE_AR_COMPOSE", "PCCL_ALLREDUCE_RS_AG"}, false);
  const size_t es = hlTypeSize(t);
  const int n = impl_->n_;
  if (compose && es && n > 1 && count % (size_t)n == 0 && count >= (size_t)n) {
    const size_t seg = count / (size_t)n, bytes = count * es;
    const char* s = (const char*)send;
    char* r = (char*)recv;
    const bool disjoint = s + bytes <= r || r + bytes <= s;
    if (disjoint) {
      char* slot = r + (size_t)impl_->rank_ * seg * es;
      HL_CHECK(impl_->submit("reducescatter", "", send, slot, seg, 0, n, 1, t, op, scale, 0, stream));
      composed_.fetch_add(1, std::memory_order_relaxed);
      return impl_->submit("allgather", "", slot, recv, seg, 0, 1, n, t, hlSum, 1.0f, 0, stream);
    }
  }
  return impl_->submit("allreduce", "", send, recv, count, 0, 1, 1, t, op, scale, 0, stream);
}
uint64_t PciePath::composedAllReduces() const { return composed_.load(); }
hlResult_t PciePath::reduceScatter(const void* send, void* recv, size_t seg_count, size_t stride, hlDataType_t t, hlRedOp_t op,
                                   float scale, hlStream_t stream) {
  return impl_->submit("reducescatter", "", send, recv, seg_count, stride, impl_->n_, 1, t, op, scale, 0, stream);
}
hlResult_t PciePath::allGather(const void* send, void* recv, size_t seg_count, size_t stride, hlDataType_t t, hlStream_t stream) {
  return impl_->submit("allgather", "", send, recv, seg_count, stride, 1, impl_->n_, t, hlSum, 1.0f, 0, stream);
}
hlResult_t PciePath::allToAll(const void* send, void* recv, size_t seg_count, size_t stride, hlDataType_t t, hlStream_t stream) {
  return impl_->submit("alltoall", "", send, recv, seg_count, stride, impl_->n_, impl_->n_, t, hlSum, 1.0f, 0, stream);
}
hlResult_t PciePath::broadcast(const void* send, void* recv, size_t count, hlDataType_t t, int root, hlStream_t stream) {
  return impl_->submit("broadcast", "", send ? send : recv, recv, count, 0, 1, 1, t, hlSum, 1.0f, root, stream);
}
hlResult_t PciePath::submitIr(const char* xml, const void* send, void* recv, size_t seg_count, size_t stride, int send_segs,
                              int recv_segs, hlDataType_t t, hlRedOp_t op, hlStream_t stream) {
  if (!xml) return fail(hlInvalidArgument, "null schedule text");
  return impl_->submit("custom", xml, send, recv, seg_count, stride, send_segs, recv_segs, t, op, 1.0f, 0, stream);
}
hlResult_t PciePath::drain() { return impl_->drain(); }
hlResult_t PciePath::lastResult() const { return impl_->lastResult(); }
uint64_t PciePath::kernelLaunches() const { return impl_->kernelLaunches(); }
uint64_t PciePath::copyOps() const { return impl_->copyOps(); }
uint64_t PciePath::fusedSlices() const { return impl_->fusedSlices(); }
uint64_t PciePath::rangeJobs() const { return impl_->rangeJobs(); }
uint64_t PciePath::smallCalls() const { return impl_->smallCalls(); }
uint64_t PciePath::foldedSources() const { return impl_->foldedSources(); }
const std::vector<int>& PciePath::rankNuma() const { return impl_->rankNuma(); }

}  // namespace hl

// Blocks until every executor of the process is idle (used by the interposers
// of host-blocking CUDA calls).
extern "C" void hlDrainAllExecutors(void) {
  std::vector<hl::PcieImpl*> snapshot;
  {
    std::lock_guard<std::mutex> lk(hl::g_reg_mu);
    snapshot = hl::g_registry;
  }
  for (auto* e : snapshot) e->drainHostSide();
}
