// Host side of the dedicated-link path: owns the symmetric staging region and
// the flag area, chooses algorithm and CTA count per call, slices messages
// that exceed the staging capacity, and launches the sm_100a kernels.
//
// Two flavours share all of the code: a real path (one rank per process or
// thread, peers reached over NVLink) and an emulated group (N ranks on ONE
// device, launched as one cooperative grid) that lets a single-GPU machine
// check the cross-rank protocol of every kernel.
//
// Parity: stands where the reference's fast backend calls the vendor library
// (multipath-orchestrator/libampccl/backend/fast_backend.cc:7-103,
// original_collective_api.cc:60-148).
#pragma once
#include <cuda_runtime.h>

#include <map>

#include "ctrl/bootstrap.h"
#include "nvl/nvl_launch.h"
#include "nvl/symm_mem.h"

namespace hl {

struct NvlBufs {
  const void* in[HL_MAX_RANKS];
  void* out[HL_MAX_RANKS];
};

struct NvlCall {
  uint64_t count = 0;           // AR/bcast: elements; AG/RS/A2A: handled prefix of a segment
  uint64_t in_seg_stride = 0;   // elements between input segments (RS, A2A); 0 = count
  uint64_t out_seg_stride = 0;  // elements between output segments (AG, A2A); 0 = count
  int in_dt = hlFloat32, out_dt = hlFloat32, wire_dt = hlFloat32;
  int op = hlSum;
  float scale = 1.0f;
  int root = 0;
  int algo = hlAlgoAuto;
  int max_blocks = 0;
  bool deterministic = false;
};

class NvlPath {
 public:
  ~NvlPath();
  static hlResult_t createReal(Bootstrap* bs, int device, NvlPath** out);
  static hlResult_t createEmu(int nranks, int device, size_t stage_bytes, int timeout_ms, NvlPath** out);

  int nranks() const { return nranks_; }
  int localRanks() const { return emu_ ? nranks_ : 1; }
  bool hasNvls() const { return has_mc_; }
  int symmMode() const { return region_.mode; }
  size_t stageBytes() const { return stage_bytes_; }
  uint64_t launches() const { return launches_; }
  // Emulation only: launch just the first k ranks' rows (the others never
  // signal), to exercise the bounded-wait error path without hanging anything.
  void setEmuActiveRanks(int k) { emu_active_ = k; }

  hlResult_t allReduce(const NvlBufs& b, const NvlCall& c, cudaStream_t s);
  hlResult_t reduceScatter(const NvlBufs& b, const NvlCall& c, cudaStream_t s);
  hlResult_t allGather(const NvlBufs& b, const NvlCall& c, cudaStream_t s);
  hlResult_t broadcast(const NvlBufs& b, const NvlCall& c, cudaStream_t s);
  hlResult_t allToAll(const NvlBufs& b, const NvlCall& c, cudaStream_t s);
  hlResult_t barrier(cudaStream_t s);
  // Measurement aid: copies `bytes` between the first half of the staging region of this rank and the second half
  // of the next rank's (direction and launch shape by argument). Real paths only.
  hlResult_t linkProbe(int mode, int blocks, int threads, int unroll, int layout, size_t bytes, cudaStream_t s);

  // Test aid of the link probe: host copy into / out of this rank's staging region (synchronises the device).
  hlResult_t stageAccess(bool write, size_t offset, void* host, size_t bytes);
  // Copies the kernel timeline ring of local rank i (HL_TL_WORDS words; layout in nvl_types.h) after a device
  // synchronize. With out == nullptr only the needed length is returned.
  hlResult_t readTimeline(int local_rank, uint64_t* out, size_t* words);
  // Device status of local rank i: HL_DEV_OK or the code a kernel recorded.
  uint64_t deviceStatus(int i = 0, uint64_t* detail = nullptr, uint64_t* block = nullptr) const;
  // Clears the poison after a recorded timeout (all ranks, collectively, with
  // no launch in flight); flags and sequence restart from a common value.
  hlResult_t resetAfterError();
  // Registered memory: a symmetric heap (same size on every rank, every peer's heap mapped here, one multicast alias
  // with NVLS), created at the first allocation. Allocation and release are collective in effect: every rank must
  // issue the same sequence of sizes, so that a buffer sits at the same offset everywhere. `ptrs` receives one
  // pointer per local rank (one, except in the emulated group). Returns hlUnsupported when the heap is exhausted
  // or cannot be created; the caller then falls back to ordinary device memory.
  hlResult_t heapAlloc(size_t bytes, void** ptrs);
  hlResult_t heapFree(void* ptr_of_local_rank0);
  bool heapOffset(int local_rank, const void* p, size_t bytes, uint64_t* off) const;
  size_t heapBytes() const { return heap_bytes_; }
  size_t heapInUse() const;
  int pickAllReduceAlgo(size_t wire_bytes, int wire_dt, int op, bool deterministic, int requested) const;
  bool nvlsPays() const;
  size_t pipeMinBytes() const;
  size_t agLanesMinBytes() const;
  size_t lanesMinBytes() const;   // peer-pointer reduce-scatter: from this size on the lane kernel
  bool nvlsUsable(int wire_dt, int op, bool deterministic) const;
  int blocksFor(int kind, size_t wire_bytes_per_rank, int max_blocks) const;

 private:
  NvlPath() = default;
  hlResult_t finishInit(int timeout_ms);
  hlResult_t launchSliced(int kind, const NvlBufs& b, const NvlCall& c, bool segmented, cudaStream_t s);
  hlResult_t orderAfterPrevious(cudaStream_t s);
  hlResult_t ensureHeap();
  // Zero-copy kernels: which buffers peers reach in place (and therefore have to be registered, aligned and whole packets).
  bool zeroCopyEligible(const NvlBufs& b, const NvlCall& c, bool in_remote, bool out_remote, uint64_t in_extent, uint64_t out_extent,
                        uint64_t* in_off, uint64_t* out_off) const;
  hlResult_t launchZeroCopy(int kind, const NvlBufs& b, const NvlCall& c, uint64_t in_off, uint64_t out_off, size_t bytes_per_rank,
                            cudaStream_t s);
  int zeroCopyFlavour(const NvlCall& c, int coll, size_t wire_bytes) const;
  // Barrier-free small-message kernels: 1 when the call should and can take them, 0 when not, -1 when the caller
  // asked for them by name and the call does not qualify. coll: 0 all-reduce, 1 reduce-scatter, 2 all-gather, 3 all-to-all.
  int lowLatencyChoice(const NvlBufs& b, const NvlCall& c, int coll, size_t wire_bytes) const;
  hlResult_t launchLowLatency(int kind, const NvlBufs& b, const NvlCall& c, uint64_t packets_per_thread_range, cudaStream_t s);   // coll: 0 all-reduce, 1 reduce-scatter, 2 gather / broadcast
  Bootstrap* bs_ = nullptr;
  bool emu_ = false;
  int emu_active_ = 0;
  int rank_ = 0, nranks_ = 1, device_ = 0;
  size_t stage_bytes_ = 0;
  size_t ll_slot_bytes_ = 0;   // one slot of the low-latency region (0: the region does not exist)
  bool has_mc_ = false;
  SymmRegion region_;
  void* emu_mem_[HL_MAX_RANKS] = {nullptr};
  HlCommDev* dcomm_ = nullptr;     // device array: 1 entry (real) or nranks (emu)
  uint64_t* status_host_ = nullptr; // pinned, mapped; 8 words per local rank
  uint32_t* abort_dev_ = nullptr;   // one word per local rank
  uint64_t* timeline_dev_ = nullptr;  // kernel timeline ring per local rank, null when off
  uint64_t* seq_dev_ = nullptr;    // per local rank: flag base, tile base, finished-CTA counter (advanced by the kernels)
  uint64_t launches_ = 0;
  SymmRegion heap_region_;
  void* emu_heap_[HL_MAX_RANKS] = {nullptr};
  size_t heap_bytes_ = 0;
  bool heap_failed_ = false;
  bool heap_mc_ = false;
  std::map<uint64_t, uint64_t> heap_free_;   // offset -> length
  std::map<uint64_t, uint64_t> heap_used_;
  HlCommDev host_comm_[HL_MAX_RANKS];
  cudaEvent_t order_ev_ = nullptr;
  cudaStream_t last_stream_ = nullptr;
  bool have_last_ = false;
};

}  // namespace hl
