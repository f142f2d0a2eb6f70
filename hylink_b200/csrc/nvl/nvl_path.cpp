#include "nvl/nvl_path.h"

#include <algorithm>
#include <cstring>
#include <memory>

namespace hl {

static constexpr size_t kFlagBytes = (size_t)HL_FLAG_KINDS * HL_MAX_BLOCKS * HL_MAX_RANKS * sizeof(uint64_t);

static constexpr size_t kZcArgBytes = (size_t)HL_MAX_RANKS * 2 * sizeof(uint64_t);   // behind the flag words (HL_ZC_ARGS_WORD_OFF)

static size_t flagAreaBytes() { return (kFlagBytes + kZcArgBytes + 4095) & ~(size_t)4095; }

// Low-latency region behind the flag area: [2 parities][2 phases][HL_MAX_RANKS sources] slots (nvl_ll_kernels.cu).
static constexpr size_t kLlSlots = 2 * 2 * HL_MAX_RANKS;
static size_t llSlotBytesFromEnv(bool emu) {
  static const long long v = envInt({"HYLINK_LL_SLOT_BYTES"}, 4LL << 20);   // 0: no low-latency kernels
  size_t s = v <= 0 ? 0 : ((size_t)v + 4095) & ~(size_t)4095;
  if (emu && s > ((size_t)1 << 20)) s = (size_t)1 << 20;   // emulated groups (tests) hold nranks regions on one GPU
  return s;
}

NvlPath::~NvlPath() {
  if (device_ >= 0) cudaSetDevice(device_);
  cudaDeviceSynchronize();
  if (order_ev_) cudaEventDestroy(order_ev_);
  if (dcomm_) cudaFree(dcomm_);
  if (abort_dev_) cudaFree(abort_dev_);
  if (seq_dev_) cudaFree(seq_dev_);
  if (timeline_dev_) cudaFree(timeline_dev_);
  if (status_host_) cudaFreeHost(status_host_);
  if (emu_) {
    for (int q = 0; q < nranks_; ++q) {
      if (emu_mem_[q]) cudaFree(emu_mem_[q]);
      if (emu_heap_[q]) cudaFree(emu_heap_[q]);
    }
  } else {
    const bool gone = bs_ ? bs_->anyFailed() : true;
    if (heap_region_.mode != kSymmNone) symmFree(bs_, &heap_region_, gone);
    symmFree(bs_, &region_, gone);
  }
  cudaGetLastError();
}

hlResult_t NvlPath::finishInit(int timeout_ms) {
  const int nl = localRanks();
  HL_CUDA(cudaHostAlloc((void**)&status_host_, sizeof(uint64_t) * 8 * nl, cudaHostAllocMapped | cudaHostAllocPortable));
  memset(status_host_, 0, sizeof(uint64_t) * 8 * nl);
  uint64_t* status_dev = nullptr;
  HL_CUDA(cudaHostGetDevicePointer((void**)&status_dev, status_host_, 0));
  HL_CUDA(cudaMalloc((void**)&abort_dev_, sizeof(uint32_t) * 16 * nl));
  HL_CUDA(cudaMemset(abort_dev_, 0, sizeof(uint32_t) * 16 * nl));
  HL_CUDA(cudaMalloc((void**)&seq_dev_, sizeof(uint64_t) * 8 * nl));
  HL_CUDA(cudaMemset(seq_dev_, 0, sizeof(uint64_t) * 8 * nl));
  if (envBool({"HYLINK_KERNEL_TIMELINE"}, false)) {
    HL_CUDA(cudaMalloc((void**)&timeline_dev_, sizeof(uint64_t) * HL_TL_WORDS * nl));
    HL_CUDA(cudaMemset(timeline_dev_, 0, sizeof(uint64_t) * HL_TL_WORDS * nl));
  }
  HlCommDev h[HL_MAX_RANKS];
  memset(h, 0, sizeof(h));
  for (int i = 0; i < nl; ++i) {
    HlCommDev& c = h[i];
    c.rank = emu_ ? i : rank_;
    c.nranks = nranks_;
    c.max_blocks = HL_MAX_BLOCKS;
    for (int q = 0; q < nranks_; ++q) {
      uint8_t* base = (uint8_t*)(emu_ ? emu_mem_[q] : region_.ptr[q]);
      c.stage[q] = base;
      c.flags[q] = (uint64_t*)(base + stage_bytes_);
    }
    for (int q = 0; q < nranks_ && ll_slot_bytes_; ++q) {
      uint8_t* base = (uint8_t*)(emu_ ? emu_mem_[q] : region_.ptr[q]);
      c.ll[q] = base + stage_bytes_ + flagAreaBytes();
    }
    c.ll_slot_bytes = ll_slot_bytes_;
    c.mc_stage = emu_ ? nullptr : (uint8_t*)region_.mc;
    c.status = status_dev + 8 * i;
    c.abort_word = abort_dev_ + 16 * i;
    c.seq_words = seq_dev_ + 8 * i;
    c.timeline = timeline_dev_ ? timeline_dev_ + (size_t)HL_TL_WORDS * i : nullptr;
    c.stage_bytes = stage_bytes_;
    c.timeout_ns = (uint64_t)timeout_ms * 1000000ull;
  }
  memcpy(host_comm_, h, sizeof(h));
  HL_CUDA(cudaMalloc((void**)&dcomm_, sizeof(HlCommDev) * nl));
  HL_CUDA(cudaMemcpy(dcomm_, h, sizeof(HlCommDev) * nl, cudaMemcpyHostToDevice));
  HL_CUDA(cudaEventCreateWithFlags(&order_ev_, cudaEventDisableTiming));
  HL_CHECK(nvl::prepareKernels());
  HL_CUDA(cudaDeviceSynchronize());
  return hlSuccess;
}

hlResult_t NvlPath::createReal(Bootstrap* bs, int device, NvlPath** out) {
  const Config& cfg = Config::get();
  std::unique_ptr<NvlPath> p(new NvlPath());
  p->bs_ = bs;
  p->rank_ = bs->rank();
  p->nranks_ = bs->nranks();
  p->device_ = device;
  p->stage_bytes_ = (cfg.symm_stage_bytes + 4095) & ~(size_t)4095;
  HL_CUDA(cudaSetDevice(device));
  p->ll_slot_bytes_ = p->nranks_ > 1 ? llSlotBytesFromEnv(false) : 0;
  HL_CHECK(symmAlloc(bs, device, p->stage_bytes_ + flagAreaBytes() + kLlSlots * p->ll_slot_bytes_, cfg.nvls, cfg.symm_mode, &p->region_));
  p->has_mc_ = p->region_.mc != nullptr;
  // flags (and the tags of the low-latency region) start at zero on every rank before anybody launches
  HL_CUDA(cudaMemset((uint8_t*)p->region_.ptr[p->rank_] + p->stage_bytes_, 0, flagAreaBytes() + kLlSlots * p->ll_slot_bytes_));
  HL_CUDA(cudaDeviceSynchronize());
  HL_CHECK(p->finishInit(cfg.nvl_timeout_ms));
  HL_CHECK(bs->barrier(kBarSymm));
  HL_INFO("NVLink path ready: rank %d/%d dev %d symm=%d nvls=%d stage=%zu MiB", p->rank_, p->nranks_, device,
          p->region_.mode, (int)p->has_mc_, p->stage_bytes_ >> 20);
  *out = p.release();
  return hlSuccess;
}

hlResult_t NvlPath::createEmu(int nranks, int device, size_t stage_bytes, int timeout_ms, NvlPath** out) {
  if (nranks < 1 || nranks > HL_MAX_RANKS) return fail(hlInvalidArgument, "emulated nranks %d out of range", nranks);
  std::unique_ptr<NvlPath> p(new NvlPath());
  p->emu_ = true;
  p->nranks_ = nranks;
  p->emu_active_ = nranks;
  p->device_ = device;
  p->stage_bytes_ = (stage_bytes + 4095) & ~(size_t)4095;
  HL_CUDA(cudaSetDevice(device));
  p->ll_slot_bytes_ = nranks > 1 ? llSlotBytesFromEnv(true) : 0;
  for (int q = 0; q < nranks; ++q) {
    HL_CUDA(cudaMalloc(&p->emu_mem_[q], p->stage_bytes_ + flagAreaBytes() + kLlSlots * p->ll_slot_bytes_));
    HL_CUDA(cudaMemset((uint8_t*)p->emu_mem_[q] + p->stage_bytes_, 0, flagAreaBytes() + kLlSlots * p->ll_slot_bytes_));
  }
  HL_CHECK(p->finishInit(timeout_ms));
  *out = p.release();
  return hlSuccess;
}

uint64_t NvlPath::deviceStatus(int i, uint64_t* detail, uint64_t* block) const {
  volatile uint64_t* s = status_host_ + 8 * i;
  if (detail) *detail = s[1];
  if (block) *block = s[2];
  return s[0];
}

hlResult_t NvlPath::resetAfterError() {
  HL_CUDA(cudaSetDevice(device_));
  HL_CUDA(cudaDeviceSynchronize());
  const int nl = localRanks();
  if (!emu_ && bs_) HL_CHECK(bs_->barrier(kBarSymm));
  if (emu_) {
    for (int q = 0; q < nranks_; ++q) HL_CUDA(cudaMemset((uint8_t*)emu_mem_[q] + stage_bytes_, 0, flagAreaBytes() + kLlSlots * ll_slot_bytes_));
  } else {
    HL_CUDA(cudaMemset((uint8_t*)region_.ptr[rank_] + stage_bytes_, 0, flagAreaBytes() + kLlSlots * ll_slot_bytes_));
  }
  HL_CUDA(cudaMemset(abort_dev_, 0, sizeof(uint32_t) * 16 * nl));
  HL_CUDA(cudaMemset(seq_dev_, 0, sizeof(uint64_t) * 8 * nl));
  memset(status_host_, 0, sizeof(uint64_t) * 8 * nl);
  HL_CUDA(cudaDeviceSynchronize());
  if (!emu_ && bs_) HL_CHECK(bs_->barrier(kBarSymm));
  return hlSuccess;
}

hlResult_t NvlPath::orderAfterPrevious(cudaStream_t s) {
  // Rule B of the kernels' protocol: consecutive launches of one communicator
  // must not overlap on this rank, whatever streams the caller uses.
  if (have_last_ && last_stream_ != s) {
    HL_CUDA(cudaEventRecord(order_ev_, last_stream_));
    HL_CUDA(cudaStreamWaitEvent(s, order_ev_, 0));
  }
  last_stream_ = s;
  have_last_ = true;
  return hlSuccess;
}

bool NvlPath::nvlsPays() const {
  // Through the switch every GPU sends its whole buffer once (S bytes out)
  // whatever the rank count, while peer pulls move (n-1)/n * S in each
  // direction: NVLS halves the inbound side only, which starts to pay at four
  // ranks and loses at two.
  return has_mc_ && nranks_ >= Config::get().nvls_min_ranks;
}

size_t NvlPath::pipeMinBytes() const {
  const size_t forced = Config::get().pipe_min_bytes;
  if (forced) return forced;
  return nranks_ >= 8 ? ((size_t)256 << 20) : ((size_t)512 << 20);
}

bool NvlPath::nvlsUsable(int wire_dt, int op, bool deterministic) const {
  return has_mc_ && (wire_dt == hlFloat32 || wire_dt == hlFloat16 || wire_dt == hlBfloat16) && (op == hlSum || op == hlAvg) &&
         !deterministic;
}

int NvlPath::pickAllReduceAlgo(size_t wire_bytes, int wire_dt, int op, bool deterministic, int requested) const {
  const bool nvls_ok = nvlsUsable(wire_dt, op, deterministic);
  if (requested == hlAlgoNvls && !nvls_ok) requested = hlAlgoAuto;
  if (requested != hlAlgoAuto) return requested;
  if (wire_bytes <= Config::get().oneshot_max_bytes) return hlAlgoOneShot;
  if (nvls_ok && nvlsPays()) {
    // Measured on B200 (bf16, busbw GB/s): the switch kernels win below 32 MiB (one launch, two barriers); from
    // there the stores-only kernel is ahead (8 GPUs, 128 MiB: 568 push / 557 NVLS / 529 pipelined; 4 GPUs,
    // 256 MiB: 586 push / 540 pipelined) until the message is long enough for the pipelined NVLS kernel's large
    // tiles (8 GPUs, 1 GiB: 728 pipelined / 601 push; 4 GPUs, 1 GiB: 625 / 599).
    const size_t pipe_min = pipeMinBytes();
    if (wire_bytes >= pipe_min) return hlAlgoPipelined;
    if (wire_bytes >= Config::get().push_min_bytes) return hlAlgoPush;
    return hlAlgoNvls;
  }
  return hlAlgoPush;  // peer pointers: stores only (falls back to the staged two-shot when the call converts types)
}

hlResult_t NvlPath::stageAccess(bool write, size_t offset, void* host, size_t bytes) {
  // a one-rank communicator is built on the single-device flavour of the path: its only staging region serves
  if (emu_ && nranks_ > 1) return fail(hlUnsupported, "stage access needs a real communicator");
  if (!host || offset + bytes > stage_bytes_) return fail(hlInvalidArgument, "stage access out of range");
  HL_CUDA(cudaSetDevice(device_));
  HL_CUDA(cudaDeviceSynchronize());
  char* p = (char*)(emu_ ? emu_mem_[0] : region_.ptr[rank_]) + offset;
  HL_CUDA(write ? cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice) : cudaMemcpy(host, p, bytes, cudaMemcpyDeviceToHost));
  return hlSuccess;
}

hlResult_t NvlPath::readTimeline(int local_rank, uint64_t* out, size_t* words) {
  if (!words) return fail(hlInvalidArgument, "timeline: null length");
  if (!timeline_dev_) return fail(hlUnsupported, "the kernel timeline is off (HYLINK_KERNEL_TIMELINE=1 before the communicator is created)");
  if (local_rank < 0 || local_rank >= localRanks()) return fail(hlInvalidArgument, "timeline: bad local rank %d", local_rank);
  if (!out || *words < (size_t)HL_TL_WORDS) {
    *words = HL_TL_WORDS;
    return out ? fail(hlInvalidArgument, "timeline: buffer too small") : hlSuccess;
  }
  HL_CUDA(cudaSetDevice(device_));
  HL_CUDA(cudaDeviceSynchronize());
  HL_CUDA(cudaMemcpy(out, timeline_dev_ + (size_t)HL_TL_WORDS * local_rank, sizeof(uint64_t) * HL_TL_WORDS, cudaMemcpyDeviceToHost));
  *words = HL_TL_WORDS;
  return hlSuccess;
}

hlResult_t NvlPath::linkProbe(int mode, int blocks, int threads, int unroll, int layout, size_t bytes, cudaStream_t s) {
  if (emu_ && nranks_ > 1) return fail(hlUnsupported, "link probe needs a real communicator");
  if (nranks_ < 2 && mode != 2 && mode != 6) return fail(hlInvalidArgument, "link probe needs a peer");
  const size_t half = stage_bytes_ / 2 / 16 * 16;
  if (bytes < 16 || bytes > half) return fail(hlInvalidArgument, "link probe: %zu bytes exceed half of the staging region (%zu)", bytes, half);
  HL_CHECK(orderAfterPrevious(s));
  if (mode == 5 || mode == 6) {  // bulk-copy engine: 5 to the peer, 6 local; `threads` carries the tile size in bytes
    HL_CHECK(nvl::launchLinkProbeBulk(dcomm_, mode == 5, blocks, (uint32_t)threads, bytes / 16 * 16, half, (rank_ + 1) % nranks_, s));
    ++launches_;
    return hlSuccess;
  }
  HL_CHECK(nvl::launchLinkProbe(dcomm_, mode, blocks, threads, unroll, layout, bytes / 16, half / 16, (rank_ + 1) % nranks_, s));
  ++launches_;
  return hlSuccess;
}


// ---------------------------------------------------------------------- registered memory
static constexpr uint64_t kHeapAlign = 512;

hlResult_t NvlPath::ensureHeap() {
  if (heap_bytes_ || heap_failed_) return heap_bytes_ ? hlSuccess : hlUnsupported;
  const Config& cfg = Config::get();
  size_t want = cfg.symm_heap_bytes;
  HL_CUDA(cudaSetDevice(device_));
  HL_CUDA(cudaDeviceSynchronize());   // the per-communicator constants are rewritten below: no launch may be in flight
  const int nl = localRanks();
  if (emu_) {
    want = std::min<size_t>(want, (size_t)256 << 20);   // n heaps on one device
    for (int q = 0; q < nranks_; ++q) {
      if (cudaMalloc(&emu_heap_[q], want) != cudaSuccess) {
        cudaGetLastError();
        heap_failed_ = true;
        return hlUnsupported;
      }
    }
  } else {
    hlResult_t r = symmAlloc(bs_, device_, want, cfg.nvls, cfg.symm_mode, &heap_region_);
    if (r != hlSuccess) {
      HL_WARN("registered-memory heap of %zu MiB could not be created; buffers will be staged", want >> 20);
      heap_failed_ = true;
      heap_region_ = SymmRegion();
      return hlUnsupported;
    }
    heap_mc_ = heap_region_.mc != nullptr;
  }
  for (int i = 0; i < nl; ++i) {
    HlCommDev& c = host_comm_[i];
    for (int q = 0; q < nranks_; ++q) c.heap[q] = (uint8_t*)(emu_ ? emu_heap_[q] : heap_region_.ptr[q]);
    c.mc_heap = emu_ ? nullptr : (uint8_t*)heap_region_.mc;
    c.heap_bytes = want;
  }
  HL_CUDA(cudaMemcpy(dcomm_, host_comm_, sizeof(HlCommDev) * nl, cudaMemcpyHostToDevice));
  HL_CUDA(cudaDeviceSynchronize());
  heap_bytes_ = want;
  heap_free_.clear();
  heap_used_.clear();
  heap_free_[0] = want;
  if (!emu_ && bs_) HL_CHECK(bs_->barrier(kBarSymm));
  HL_INFO("registered-memory heap ready: %zu MiB per rank, multicast=%d", want >> 20, (int)heap_mc_);
  return hlSuccess;
}

hlResult_t NvlPath::heapAlloc(size_t bytes, void** ptrs) {
  if (!ptrs || bytes == 0) return fail(hlInvalidArgument, "heap allocation of %zu bytes", bytes);
  if (ensureHeap() != hlSuccess) return hlUnsupported;
  const uint64_t need = ((uint64_t)bytes + kHeapAlign - 1) & ~(kHeapAlign - 1);
  for (auto it = heap_free_.begin(); it != heap_free_.end(); ++it) {   // first fit: the same choice on every rank
    if (it->second < need) continue;
    const uint64_t off = it->first, len = it->second;
    heap_free_.erase(it);
    if (len > need) heap_free_[off + need] = len - need;
    heap_used_[off] = need;
    for (int i = 0; i < localRanks(); ++i) ptrs[i] = host_comm_[i].heap[host_comm_[i].rank] + off;
    return hlSuccess;
  }
  return hlUnsupported;   // exhausted (identically on every rank)
}

hlResult_t NvlPath::heapFree(void* p) {
  if (!heap_bytes_ || !p) return hlInvalidArgument;
  const uint8_t* base = host_comm_[0].heap[host_comm_[0].rank];
  if ((const uint8_t*)p < base || (const uint8_t*)p >= base + heap_bytes_) return hlInvalidArgument;
  uint64_t off = (uint64_t)((const uint8_t*)p - base);
  auto it = heap_used_.find(off);
  if (it == heap_used_.end()) return fail(hlInvalidArgument, "not the start of a registered allocation");
  uint64_t len = it->second;
  heap_used_.erase(it);
  auto next = heap_free_.lower_bound(off);
  if (next != heap_free_.end() && next->first == off + len) {   // merge with the following hole
    len += next->second;
    next = heap_free_.erase(next);
  }
  if (next != heap_free_.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == off) {   // and with the one before
      prev->second += len;
      return hlSuccess;
    }
  }
  heap_free_[off] = len;
  return hlSuccess;
}

size_t NvlPath::heapInUse() const {
  size_t t = 0;
  for (auto& kv : heap_used_) t += kv.second;
  return t;
}

bool NvlPath::heapOffset(int i, const void* p, size_t bytes, uint64_t* off) const {
  if (!heap_bytes_ || !p) return false;
  const uint8_t* base = host_comm_[i].heap[host_comm_[i].rank];
  const uint8_t* q = (const uint8_t*)p;
  if (q < base || q + bytes > base + heap_bytes_) return false;
  *off = (uint64_t)(q - base);
  return true;
}

// Which flavour of zero-copy kernel a call gets (0 none, 1 NVLS, 2 peer pointers). Measured on 4 B200 (bf16, busbw):
//  * all-gather / broadcast: posted peer stores (688 GB/s at 1 GiB) beat multimem.st (529) at every size;
//  * reduce-scatter: peer loads (638 GB/s at 1 GiB) beat multimem.ld_reduce (522): through the switch every GPU
//    sends its WHOLE input out (its own contribution travels to the switch too), so the call is bound by outbound
//    traffic at busbw = (n-1)/n of the link, while peer pulls send (n-1)/n of the input and reach the link rate;
//  * all-reduce: the switch wins where latency counts (48 vs 17 GB/s at 1 MiB) and on long messages (683 vs 663 at
//    1 GiB), peer loads + stores win in between (573 vs 520 at 64 MiB), where they run the link at a higher rate.
//    From eight ranks on the switch moves 1.125x the message per GPU where peer pointers move 1.75x.
int NvlPath::zeroCopyFlavour(const NvlCall& c, int coll, size_t wire_bytes) const {
  if (!Config::get().zero_copy && c.algo == hlAlgoAuto) return 0;
  if (c.algo != hlAlgoAuto && c.algo != hlAlgoZeroCopy && c.algo != hlAlgoZeroCopyNvls && c.algo != hlAlgoZeroCopyP2p) return 0;
  if (c.algo == hlAlgoZeroCopyP2p) return 2;
  const bool reduce = coll <= 1;
  const bool mc_ok = heap_mc_ && (!reduce || ((c.wire_dt == hlFloat32 || c.wire_dt == hlFloat16 || c.wire_dt == hlBfloat16) &&
                                               (c.op == hlSum || c.op == hlAvg) && !c.deterministic));
  if (c.algo == hlAlgoZeroCopyNvls) return mc_ok ? 1 : 0;
  static const int reduce_pref = (int)envInt({"HYLINK_ZC_REDUCE_NVLS"}, -1), gather_pref = (int)envInt({"HYLINK_ZC_GATHER_NVLS"}, 0);
  const int pref = reduce ? reduce_pref : gather_pref;
  if (!mc_ok || pref == 0) return 2;
  if (pref == 1) return 1;
  if (nranks_ < Config::get().nvls_min_ranks) return 2;
  if (coll == 1) {
    // Reduce-scatter: one multimem.ld_reduce per packet instead of a load from every peer is the shorter chain while
    // latency decides (4 GPUs, whole input 2 / 4 / 16 MiB: 59 / 109 / 267 GB/s through the switch, 54 / 100 / 265
    // with peer loads); from 32 MiB on the switch flavour is bound by outbound traffic (every GPU sends its whole
    // input, its own segment included) and peer loads win (1 GiB: 522 against 638 GB/s).
    static const long long rs_nvls_max = envInt({"HYLINK_ZC_RS_NVLS_MAX"}, 32LL << 20);
    return wire_bytes < (size_t)rs_nvls_max ? 1 : 2;
  }
  if (coll != 0) return 2;
  // A call with a CTA budget shares the GPU with compute kernels (gradient buckets under a backward pass): the
  // switch does the adding and every byte crosses this GPU's memory system once, which needs the fewest SMs
  // (GPT-2-medium DDP on 4 GPUs, 25 MB buckets, 32 CTAs: 54.45 ms per step through the switch, 54.62 with peer
  // loads and stores, 54.55 on NCCL).
  if (c.max_blocks > 0 && c.max_blocks <= 64) return 1;
  static const long long p2p_lo = envInt({"HYLINK_ZC_AR_P2P_MIN"}, -1), p2p_hi = envInt({"HYLINK_ZC_AR_P2P_MAX"}, -1);
  const size_t lo = p2p_lo >= 0 ? (size_t)p2p_lo : (nranks_ <= 4 ? (size_t)16 << 20 : 0);
  const size_t hi = p2p_hi >= 0 ? (size_t)p2p_hi : (nranks_ <= 4 ? (size_t)256 << 20 : 0);
  return (wire_bytes >= lo && wire_bytes < hi) ? 2 : 1;
}

bool NvlPath::zeroCopyEligible(const NvlBufs& b, const NvlCall& c, bool in_remote, bool out_remote, uint64_t in_extent, uint64_t out_extent,
                               uint64_t* in_off, uint64_t* out_off) const {
  if (!heap_bytes_ || c.in_dt != c.wire_dt || c.out_dt != c.wire_dt) return false;
  const uint64_t ws = hlTypeSize((hlDataType_t)c.wire_dt);
  const uint64_t epp = 16 / ws;
  if (c.count % epp) return false;                            // whole 16-byte packets only
  if ((c.in_seg_stride % epp) || (c.out_seg_stride % epp)) return false;
  *in_off = *out_off = 0;
  for (int i = 0; i < localRanks(); ++i) {
    if (((uintptr_t)b.in[i] | (uintptr_t)b.out[i]) & 15) return false;
    uint64_t io = 0, oo = 0;
    if (in_remote && !heapOffset(i, b.in[i], in_extent * ws, &io)) return false;
    if (out_remote && !heapOffset(i, b.out[i], out_extent * ws, &oo)) return false;
    if (i == 0) {
      *in_off = io;
      *out_off = oo;
    } else if (io != *in_off || oo != *out_off) {
      return false;
    }
  }
  return true;
}

hlResult_t NvlPath::launchZeroCopy(int kind, const NvlBufs& b, const NvlCall& c, uint64_t in_off, uint64_t out_off, size_t bytes_per_rank,
                                   cudaStream_t s) {
  HL_CUDA(cudaSetDevice(device_));
  HL_CHECK(orderAfterPrevious(s));
  const int nl = localRanks();
  HlEmuCalls calls;
  memset(&calls, 0, sizeof(calls));
  for (int i = 0; i < nl; ++i) {
    HlCallArgs& a = calls.c[i];
    a.in = b.in[i];
    a.out = b.out[i];
    a.count = c.count;
    a.in_seg_stride = c.in_seg_stride ? c.in_seg_stride : c.count;
    a.out_seg_stride = c.out_seg_stride ? c.out_seg_stride : c.count;
    a.scale = (c.scale == 0.0f ? 1.0f : c.scale) * (c.op == hlAvg ? 1.0f / (float)nranks_ : 1.0f);
    a.op = c.op;
    a.in_dt = c.in_dt;
    a.out_dt = c.out_dt;
    a.root = c.root;
    a.int_div = (c.op == hlAvg) ? nranks_ : 0;
    a.kind = kind;
    a.zc_in_off = in_off;
    a.zc_out_off = out_off;
  }
  // one CTA per 16 KiB of this rank's share (every thread owns a packet or two, so that all remote accesses of a
  // small call are in flight at once), up to one per SM
  int cap = c.max_blocks > 0 ? c.max_blocks : (Config::get().nvl_max_blocks > 0 ? Config::get().nvl_max_blocks : 148);
  if (emu_) cap = std::min(cap, std::max(1, 148 / nranks_));
  static const size_t per_cta = (size_t)envInt({"HYLINK_ZC_BYTES_PER_CTA"}, 16LL << 10);
  const size_t want = std::max<size_t>(1, (bytes_per_rank + per_cta - 1) / per_cta);
  const int blocks = (int)std::min<size_t>(want, (size_t)std::min(cap, HL_MAX_BLOCKS));
  HL_CHECK(nvl::launch(kind, c.wire_dt, dcomm_, calls, emu_ ? emu_active_ : 1, blocks, s, nranks_));
  ++launches_;
  return hlSuccess;
}

int NvlPath::blocksFor(int kind, size_t wire_bytes_per_rank, int max_blocks) const {
  int cap = max_blocks > 0 ? max_blocks : (Config::get().nvl_max_blocks > 0 ? Config::get().nvl_max_blocks : 148);
  if (emu_) cap = std::min(cap, std::max(1, 148 / nranks_));
  cap = std::min(cap, HL_MAX_BLOCKS);
  // Latency-bound sizes want every thread to own one or two packets so that
  // all remote accesses of a phase are in flight at once: one CTA (512
  // threads x 16 B) per 8 KiB for the one-shot kernel, per 16 KiB otherwise.
  // The push all-reduce pays two grid-wide flag rounds whose cost grows with the CTA count: below 16 MiB a
  // smaller grid is faster (8 MiB on 2 GPUs: 207 GB/s with 96 CTAs, 164 GB/s with 148).
  if (kind == kNvlAllReducePush && wire_bytes_per_rank < (16u << 20)) cap = std::min(cap, 96);
  const size_t per_cta = kind == kNvlAllReduceOneShot ? (8u << 10) : (16u << 10);
  size_t want = (wire_bytes_per_rank + per_cta - 1) / per_cta;
  if (want < 1) want = 1;
  return (int)std::min<size_t>(want, (size_t)cap);
}

hlResult_t NvlPath::launchSliced(int kind, const NvlBufs& b, const NvlCall& c, bool segmented, cudaStream_t s) {
  const size_t ws = hlTypeSize((hlDataType_t)c.wire_dt);
  const size_t is = hlTypeSize((hlDataType_t)c.in_dt), os = hlTypeSize((hlDataType_t)c.out_dt);
  if (!ws || !is || !os) return fail(hlInvalidArgument, "unknown data type");
  const bool trio = [&](int d) { return d == hlFloat32 || d == hlFloat16 || d == hlBfloat16; }(c.wire_dt);
  if (!trio && (c.in_dt != c.wire_dt || c.out_dt != c.wire_dt))
    return fail(hlUnsupported, "type conversion is only available between fp32, fp16 and bf16");
  if (trio) {
    auto is_trio = [](int d) { return d == hlFloat32 || d == hlFloat16 || d == hlBfloat16; };
    if (!is_trio(c.in_dt) || !is_trio(c.out_dt)) return fail(hlUnsupported, "cannot convert integer/fp64 buffers to a float wire type");
  }
  HL_CUDA(cudaSetDevice(device_));
  HL_CHECK(orderAfterPrevious(s));
  const int nl = localRanks();
  const uint64_t epp = 16 / ws;                         // elements per wire packet
  const uint64_t cap_packets = stage_bytes_ / 16;
  uint64_t per_launch;                                  // elements handled per launch (per segment when segmented)
  const bool pipe = kind == kNvlAllReducePipeP2p || kind == kNvlAllReducePipeNvls || kind == kNvlReduceScatterPipeP2p ||
                    kind == kNvlReduceScatterPipeNvls || kind == kNvlAllGatherLanes;
  const bool pipe_ar = kind == kNvlAllReducePipeP2p || kind == kNvlAllReducePipeNvls;
  if (segmented || kind == kNvlAllReduceTwoShot || kind == kNvlAllReduceNvls || pipe_ar || kind == kNvlAllReducePush) {
    // the P2P pipelined all-reduce keeps inputs and results in separate halves of the staging region
    const uint64_t regions = (kind == kNvlAllReducePipeP2p || kind == kNvlAllReducePush) ? 2 : 1;
    uint64_t sp = (cap_packets / ((uint64_t)nranks_ * regions)) & ~(uint64_t)63;
    if (sp == 0) return fail(hlInvalidArgument, "staging region too small");
    per_launch = (segmented ? sp : sp * (uint64_t)nranks_) * epp;
  } else {
    per_launch = (cap_packets & ~(uint64_t)63) * epp;
  }
  uint64_t done = 0;
  do {
    const uint64_t len = std::min<uint64_t>(per_launch, c.count - done);
    HlEmuCalls calls;
    memset(&calls, 0, sizeof(calls));
    for (int i = 0; i < nl; ++i) {
      HlCallArgs& a = calls.c[i];
      a.in = b.in[i] ? (const char*)b.in[i] + done * is : nullptr;
      a.out = b.out[i] ? (char*)b.out[i] + done * os : nullptr;
      a.count = len;
      a.in_seg_stride = c.in_seg_stride ? c.in_seg_stride : c.count;
      a.out_seg_stride = c.out_seg_stride ? c.out_seg_stride : c.count;
      a.scale = (c.scale == 0.0f ? 1.0f : c.scale) * (c.op == hlAvg ? 1.0f / (float)nranks_ : 1.0f);
      a.op = c.op;
      a.in_dt = c.in_dt;
      a.out_dt = c.out_dt;
      a.root = c.root;
      a.int_div = (c.op == hlAvg) ? nranks_ : 0;
      a.kind = kind;
    }
    const size_t wire_bytes = (size_t)len * ws * (segmented && kind != kNvlAllGather && kind != kNvlAllGatherNvls && kind != kNvlAllGatherPush && kind != kNvlAllGatherLanes ? nranks_ : 1);
    int blocks = blocksFor(kind, wire_bytes, c.max_blocks);
    if (pipe) {
      // Tiles: as large as possible (every tile costs two flag round trips) while each CTA still gets
      // about eight of them, evenly, so that its three stages overlap: measured on 8 GPUs, 1 GiB moves at
      // 728 GB/s with 8192-packet tiles against 669 GB/s with 2048, while 256 MiB drops to 548 GB/s when
      // 8192-packet tiles leave fewer than two tiles per CTA.
      const uint64_t np = (len + epp - 1) / epp;
      const uint64_t sp = pipe_ar ? (np + (uint64_t)nranks_ - 1) / (uint64_t)nranks_ : np;
      // Peer-pointer variants give every stage of a tile CTAs of its own (three for all-reduce: push, fold,
      // copy-out; four for reduce-scatter: push and three folders); a "lane" is one such group and walks tiles lane, lane + lanes, ...
      const bool cta_roles = kind == kNvlAllReducePipeP2p || kind == kNvlReduceScatterPipeP2p || kind == kNvlAllGatherLanes;
      // reduce-scatter, all-gather: one pusher and `parts` HBM-side CTAs per lane (three unless HYLINK_LANE_PARTS says otherwise)
      static const int parts = std::min(7, std::max(1, (int)envInt({"HYLINK_LANE_PARTS"}, 3)));
      const int roles = !cta_roles ? 1 : (pipe_ar ? 3 : 1 + parts);
      for (int i = 0; i < nl; ++i) calls.c[i].lane_parts = parts;
      uint64_t lanes = std::max(1, blocks / roles);
      uint64_t tps = (sp + lanes * 8 - 1) / (lanes * 8);
      tps = std::min<uint64_t>(8192, std::max<uint64_t>(256, (tps + 63) & ~(uint64_t)63));
      static const long long forced = envInt({"HYLINK_PIPE_TILE_PACKETS"}, 0);   // read once: this sits on the launch path
      if (forced > 0) tps = std::max<uint64_t>(64, (uint64_t)forced & ~(uint64_t)63);
      const uint64_t tiles = (sp + tps - 1) / tps;
      lanes = std::min<uint64_t>(lanes, tiles);
      blocks = (int)lanes * roles;
      for (int i = 0; i < nl; ++i) calls.c[i].tile_packets = tps;
    }
    const int rows = emu_ ? emu_active_ : 1;
    HL_CHECK(nvl::launch(kind, c.wire_dt, dcomm_, calls, rows, blocks, s, nranks_));
    ++launches_;
    done += len;
  } while (done < c.count);
  return hlSuccess;
}

// ---- barrier-free small-message kernels ------------------------------------------------------------------------
static bool disjoint(const void* a, size_t na, const void* b, size_t nb) {
  const char* x = (const char*)a;
  const char* y = (const char*)b;
  return x + na <= y || y + nb <= x;
}

int NvlPath::lowLatencyChoice(const NvlBufs& b, const NvlCall& c, int coll, size_t wire_bytes) const {
  const bool asked = c.algo == hlAlgoLowLatency;
  if (!asked && c.algo != hlAlgoAuto) return 0;
  const int no = asked ? -1 : 0;
  if (!ll_slot_bytes_ || nranks_ < 2) return no;
  // A call with a small CTA budget overlaps with compute kernels and may wait long for a late peer: thousands of
  // polling threads are the wrong neighbour for a GEMM; the barrier-based kernels wait with n threads per CTA.
  if (!asked && c.max_blocks > 0 && c.max_blocks <= 64) return 0;
  if (!asked) {
    // Measured on 4 GPUs (kernel time from the timeline, bf16; barrier-based zero-copy kernel -> this one): 64 KiB
    // reduce-scatter 12.1 -> 4.2 us, all-gather 10.1 -> 6.8; 1 MiB all-reduce 18.0 -> 12.4, reduce-scatter 19.8 -> 8.2,
    // all-gather 17.1 -> 6.8; 2 MiB 20.1 -> 15.3, 17.4 -> 12.0, 16.9 -> 7.9; 4 MiB 23.2 -> 25.2, 21.5 -> 16.6,
    // 20.4 -> 13.8; 8 MiB reduce-scatter 28.2 -> 23.7, all-gather 23.2 -> 24.3. The two flag rounds of the other
    // kernels cost 10-15 us whatever the size; flagged packets cost half the link rate instead.
    static const long long ar_max = envInt({"HYLINK_LL_AR_MAX"}, 2LL << 20), rs_max = envInt({"HYLINK_LL_RS_MAX"}, 8LL << 20),
                           ag_max = envInt({"HYLINK_LL_AG_MAX"}, 4LL << 20), a2a_max = envInt({"HYLINK_LL_A2A_MAX"}, 4LL << 20);
    const long long lim = coll == 0 ? ar_max : (coll == 1 ? rs_max : (coll == 2 ? ag_max : a2a_max));
    if ((long long)wire_bytes > lim) return 0;
  }
  if (c.in_dt != c.wire_dt || c.out_dt != c.wire_dt) return no;
  const uint64_t ws = hlTypeSize((hlDataType_t)c.wire_dt);
  if (!ws) return no;
  const uint64_t epp = 16 / ws;
  const uint64_t istride = c.in_seg_stride ? c.in_seg_stride : c.count, ostride = c.out_seg_stride ? c.out_seg_stride : c.count;
  // Nothing below depends on a pointer's alignment or on the count being whole packets: ranks must agree on the
  // kernel, and only sizes and types are the same on all of them by the definition of a collective.
  const uint64_t np = (c.count + epp - 1) / epp;
  const uint64_t per_src = coll == 0 ? (np + (uint64_t)nranks_ - 1) / (uint64_t)nranks_ : np;   // packets one rank sends to one peer
  if (((per_src + 31) / 32) * 1024 > ll_slot_bytes_) return no;   // packets are stored in groups of 32 (1 KiB)
  const size_t n = (size_t)nranks_;
  for (int i = 0; i < localRanks(); ++i) {
    const char* in = (const char*)b.in[i];
    const char* out = (const char*)b.out[i];
    if (!in || !out) return no;
    // in place only where every location is read by the thread that later overwrites it
    if (coll == 0) {
      if (in != out && !disjoint(in, c.count * ws, out, c.count * ws)) return no;
    } else if (coll == 1) {
      const size_t in_bytes = ((n - 1) * istride + c.count) * ws;
      bool slot = false;
      for (size_t q = 0; q < n; ++q) slot = slot || out == in + q * istride * ws;
      if (!slot && !disjoint(in, in_bytes, out, c.count * ws)) return no;
    } else if (coll == 2) {
      const size_t out_bytes = ((n - 1) * ostride + c.count) * ws;
      bool slot = false;
      for (size_t q = 0; q < n; ++q) slot = slot || in == out + q * ostride * ws;
      if (!slot && !disjoint(in, c.count * ws, out, out_bytes)) return no;
    } else {
      const size_t in_bytes = ((n - 1) * istride + c.count) * ws, out_bytes = ((n - 1) * ostride + c.count) * ws;
      if (!(in == out && istride == ostride) && !disjoint(in, in_bytes, out, out_bytes)) return no;
    }
  }
  return 1;
}

hlResult_t NvlPath::launchLowLatency(int kind, const NvlBufs& b, const NvlCall& c, uint64_t packets, cudaStream_t s) {
  HL_CUDA(cudaSetDevice(device_));
  HL_CHECK(orderAfterPrevious(s));
  const int nl = localRanks();
  HlEmuCalls calls;
  memset(&calls, 0, sizeof(calls));
  for (int i = 0; i < nl; ++i) {
    HlCallArgs& a = calls.c[i];
    a.in = b.in[i];
    a.out = b.out[i];
    a.count = c.count;
    a.in_seg_stride = c.in_seg_stride ? c.in_seg_stride : c.count;
    a.out_seg_stride = c.out_seg_stride ? c.out_seg_stride : c.count;
    a.scale = (c.scale == 0.0f ? 1.0f : c.scale) * (c.op == hlAvg ? 1.0f / (float)nranks_ : 1.0f);
    a.op = c.op;
    a.in_dt = c.in_dt;
    a.out_dt = c.out_dt;
    a.int_div = (c.op == hlAvg) ? nranks_ : 0;
    a.kind = kind;
  }
  // one thread per packet it sends to (and receives from) every peer; at most one CTA per SM, so that the CTAs
  // with the same index are resident on every rank at the same time (they wait for one another's packets)
  int cap = c.max_blocks > 0 ? std::min(c.max_blocks, 148) : 148;
  if (Config::get().nvl_max_blocks > 0) cap = std::min(cap, Config::get().nvl_max_blocks);
  if (emu_) cap = std::min(cap, std::max(1, 148 / nranks_));
  const uint64_t want = std::max<uint64_t>(1, (packets + HL_NVL_THREADS - 1) / HL_NVL_THREADS);
  const int blocks = (int)std::min<uint64_t>(want, (uint64_t)cap);
  HL_CHECK(nvl::launch(kind, c.wire_dt, dcomm_, calls, emu_ ? emu_active_ : 1, blocks, s, nranks_));
  ++launches_;
  return hlSuccess;
}

static bool wantsZeroCopy(int algo) { return algo == hlAlgoZeroCopy || algo == hlAlgoZeroCopyNvls || algo == hlAlgoZeroCopyP2p; }

hlResult_t NvlPath::allReduce(const NvlBufs& b, const NvlCall& c, cudaStream_t s) {
  if (c.count == 0) return hlSuccess;
  const size_t wire_bytes = c.count * hlTypeSize((hlDataType_t)c.wire_dt);
  {
    const int ll = lowLatencyChoice(b, c, 0, wire_bytes);
    if (ll < 0) return fail(hlUnsupported, "all-reduce: the low-latency kernel converts no types and needs a message that fits its slots");
    if (ll > 0) {
      const uint64_t np = (wire_bytes + 15) / 16;
      return launchLowLatency(kNvlLlAllReduce, b, c, (np + (uint64_t)nranks_ - 1) / (uint64_t)nranks_, s);
    }
  }
  {
    uint64_t io, oo;
    const int zc = nranks_ > 1 ? zeroCopyFlavour(c, 0, wire_bytes) : 0;
    if (zc && zeroCopyEligible(b, c, true, true, c.count, c.count, &io, &oo))
      return launchZeroCopy(zc == 1 ? kNvlZcAllReduceNvls : kNvlZcAllReduceP2p, b, c, io, oo, wire_bytes / (size_t)nranks_, s);
    if (wantsZeroCopy(c.algo)) return fail(hlUnsupported, "all-reduce: zero-copy needs registered, 16-byte aligned buffers of whole 16-byte packets");
  }
  int algo = pickAllReduceAlgo(wire_bytes, c.wire_dt, c.op, c.deterministic, c.algo);
  if (algo == hlAlgoOneShot && wire_bytes > stage_bytes_) algo = hlAlgoTwoShotP2p;
  const bool same = c.in_dt == c.wire_dt && c.out_dt == c.wire_dt;  // the push kernels do not convert
  int kind;
  if (algo == hlAlgoOneShot) kind = kNvlAllReduceOneShot;
  else if (algo == hlAlgoNvls) kind = kNvlAllReduceNvls;
  else if (algo == hlAlgoPush) kind = same ? kNvlAllReducePush : kNvlAllReduceTwoShot;
  else if (algo == hlAlgoPipelined) {
    if (nvlsUsable(c.wire_dt, c.op, c.deterministic) && nvlsPays()) kind = kNvlAllReducePipeNvls;
    else kind = same ? kNvlAllReducePipeP2p : kNvlAllReduceTwoShot;
  } else kind = kNvlAllReduceTwoShot;
  return launchSliced(kind, b, c, false, s);
}

// Gathered bytes from which the peer-pointer all-gather uses the lane kernel (2 GPUs, bf16: 550 against 462 GB/s at
// 256 MiB, 622 against 486 GB/s at 1 GiB, 375 against 390 GB/s at 64 MiB).
size_t NvlPath::agLanesMinBytes() const {
  static const size_t v = (size_t)envInt({"HYLINK_AG_LANES_MIN_BYTES"}, 128LL << 20);  // read once: this sits on the launch path
  return v;
}
size_t NvlPath::lanesMinBytes() const {
  static const size_t v = (size_t)envInt({"HYLINK_RS_LANES_MIN_BYTES"}, 128LL << 20);
  return v;
}

hlResult_t NvlPath::reduceScatter(const NvlBufs& b, const NvlCall& c, cudaStream_t s) {
  if (c.count == 0) return hlSuccess;
  const size_t wire_bytes = c.count * hlTypeSize((hlDataType_t)c.wire_dt) * (size_t)nranks_;
  {
    const int ll = lowLatencyChoice(b, c, 1, wire_bytes);
    if (ll < 0) return fail(hlUnsupported, "reduce-scatter: the low-latency kernel converts no types and needs a message that fits its slots");
    if (ll > 0) return launchLowLatency(kNvlLlReduceScatter, b, c, (wire_bytes / (size_t)nranks_ + 15) / 16, s);
  }
  {
    uint64_t io, oo;
    const int zc = nranks_ > 1 ? zeroCopyFlavour(c, 1, wire_bytes) : 0;
    const uint64_t stride = c.in_seg_stride ? c.in_seg_stride : c.count;
    if (zc && zeroCopyEligible(b, c, true, false, stride * (uint64_t)(nranks_ - 1) + c.count, c.count, &io, &oo))
      return launchZeroCopy(zc == 1 ? kNvlZcReduceScatterNvls : kNvlZcReduceScatterP2p, b, c, io, 0, wire_bytes / (size_t)nranks_, s);
    if (wantsZeroCopy(c.algo)) return fail(hlUnsupported, "reduce-scatter: zero-copy needs a registered, 16-byte aligned input of whole 16-byte packets");
  }
  const bool nvls = nvlsUsable(c.wire_dt, c.op, c.deterministic) && c.algo != hlAlgoTwoShotP2p && c.algo != hlAlgoOneShot &&
                    (c.algo == hlAlgoNvls || c.algo == hlAlgoPipelined || nvlsPays());
  const bool same = c.in_dt == c.wire_dt && c.out_dt == c.wire_dt;
  int kind = nvls ? kNvlReduceScatterNvls : kNvlReduceScatter;
  if (nvls) {
    if (c.algo == hlAlgoPipelined || (c.algo == hlAlgoAuto && wire_bytes >= pipeMinBytes())) kind = kNvlReduceScatterPipeNvls;
    else if (same && (c.algo == hlAlgoPush || (c.algo == hlAlgoAuto && wire_bytes >= Config::get().push_min_bytes))) kind = kNvlReduceScatterPush;
  } else if (same && c.algo != hlAlgoTwoShotP2p && c.algo != hlAlgoOneShot) {
    // Peer pointers: the phased stores-only kernel, and from 128 MiB the lane kernel that folds while it pushes
    // (2 GPUs, bf16: 513 against 449 GB/s at 256 MiB, 580 against 485 GB/s at 1 GiB; 347 against 359 at 64 MiB).
    const bool lanes = c.algo == hlAlgoPipelined || (c.algo == hlAlgoAuto && wire_bytes >= lanesMinBytes());
    kind = lanes ? kNvlReduceScatterPipeP2p : kNvlReduceScatterPush;
  }
  return launchSliced(kind, b, c, true, s);
}

hlResult_t NvlPath::allGather(const NvlBufs& b, const NvlCall& c, cudaStream_t s) {
  if (c.count == 0) return hlSuccess;
  {
    const size_t seg_wire = c.count * hlTypeSize((hlDataType_t)c.wire_dt);
    const int ll = lowLatencyChoice(b, c, 2, seg_wire * (size_t)nranks_);
    if (ll < 0) return fail(hlUnsupported, "all-gather: the low-latency kernel converts no types and needs a message that fits its slots");
    if (ll > 0) return launchLowLatency(kNvlLlAllGather, b, c, (seg_wire + 15) / 16, s);
  }
  {
    uint64_t io, oo;
    const int zc = nranks_ > 1 ? zeroCopyFlavour(c, 2, 0) : 0;
    const uint64_t stride = c.out_seg_stride ? c.out_seg_stride : c.count;
    if (zc && zeroCopyEligible(b, c, false, true, c.count, stride * (uint64_t)(nranks_ - 1) + c.count, &io, &oo))
      return launchZeroCopy(zc == 1 ? kNvlZcAllGatherNvls : kNvlZcAllGatherP2p, b, c, 0, oo, c.count * hlTypeSize((hlDataType_t)c.wire_dt), s);
    if (wantsZeroCopy(c.algo)) return fail(hlUnsupported, "all-gather: zero-copy needs a registered, 16-byte aligned output of whole 16-byte packets");
  }
  const bool nvls = has_mc_ && c.algo == hlAlgoNvls;
  if (nvls) return launchSliced(kNvlAllGatherNvls, b, c, true, s);
  // peer pointers: the stores-only kernel unless the call converts types or asks for the pull kernel by name
  const bool same = c.in_dt == c.wire_dt && c.out_dt == c.wire_dt;
  static const bool ag_push = envBool({"HYLINK_AG_PUSH"}, true);
  const bool push = same && c.algo != hlAlgoTwoShotP2p && ag_push;
  const size_t seg_bytes = c.count * hlTypeSize((hlDataType_t)c.wire_dt);
  const bool lanes = push && (c.algo == hlAlgoPipelined || (c.algo == hlAlgoAuto && seg_bytes * (size_t)nranks_ >= agLanesMinBytes()));
  return launchSliced(lanes ? kNvlAllGatherLanes : (push ? kNvlAllGatherPush : kNvlAllGather), b, c, true, s);
}

hlResult_t NvlPath::broadcast(const NvlBufs& b, const NvlCall& c, cudaStream_t s) {
  if (c.count == 0) return hlSuccess;
  if (c.root < 0 || c.root >= nranks_) return fail(hlInvalidArgument, "broadcast root %d out of range", c.root);
  {
    uint64_t io, oo;
    const int zc = nranks_ > 1 ? zeroCopyFlavour(c, 2, 0) : 0;
    if (zc && zeroCopyEligible(b, c, false, true, c.count, c.count, &io, &oo))
      return launchZeroCopy(zc == 1 ? kNvlZcBroadcastNvls : kNvlZcBroadcastP2p, b, c, 0, oo, c.count * hlTypeSize((hlDataType_t)c.wire_dt), s);
    if (wantsZeroCopy(c.algo)) return fail(hlUnsupported, "broadcast: zero-copy needs a registered, 16-byte aligned buffer of whole 16-byte packets");
  }
  const bool nvls = has_mc_ && c.algo != hlAlgoTwoShotP2p && c.algo != hlAlgoOneShot;
  return launchSliced(nvls ? kNvlBroadcastNvls : kNvlBroadcast, b, c, false, s);
}

hlResult_t NvlPath::allToAll(const NvlBufs& b, const NvlCall& c, cudaStream_t s) {
  if (c.count == 0) return hlSuccess;
  {
    const size_t seg_wire = c.count * hlTypeSize((hlDataType_t)c.wire_dt);
    const int ll = lowLatencyChoice(b, c, 3, seg_wire * (size_t)nranks_);
    if (ll < 0) return fail(hlUnsupported, "all-to-all: the low-latency kernel converts no types and needs a message that fits its slots");
    if (ll > 0) return launchLowLatency(kNvlLlAllToAll, b, c, (seg_wire + 15) / 16, s);
  }
  return launchSliced(kNvlAllToAll, b, c, true, s);
}

hlResult_t NvlPath::barrier(cudaStream_t s) {
  HL_CUDA(cudaSetDevice(device_));
  HL_CHECK(orderAfterPrevious(s));
  HlEmuCalls calls;
  memset(&calls, 0, sizeof(calls));
  ++launches_;
  return nvl::launch(kNvlBarrier, hlFloat32, dcomm_, calls, emu_ ? emu_active_ : 1, 1, s);
}

}  // namespace hl
