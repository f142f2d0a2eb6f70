// PCIe path facade: host-staged collectives driven by the schedule IR.
// See pcie/pcie_path.cpp for the design notes.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <vector>

#include "core/core.h"
#include "ctrl/bootstrap.h"

namespace hl {

// Copy-engine lanes (streams per direction) a collective of `message_bytes` uses: small messages are a burst of
// short transfers and want many lanes so that several are in flight per direction, long ones saturate the link
// with two and only pay for more in submission time. `forced` > 0 overrides the table (HYLINK_DMA_LANES);
// the result lies in [1, max_lanes]. Broadcast and unknown collectives use one lane per direction.
// Parity: pcie-ccl-ascend/src/executor/dma_lane_policy.hpp:12-67 (its table is tuned for 1-12 HCCS DMA lanes;
// this one for the copy engines of a CUDA device).
int dmaLanePolicy(const char* collective, size_t message_bytes, int world, int max_lanes, int forced);


class PcieImpl;

class PciePath {
 public:
  ~PciePath();
  // Bytes this layer needs inside the communicator's shared control block.
  static size_t ctrlBytes(int nranks);
  // device >= 0: CUDA device; device == -2: host-memory stand-in device.
  static hlResult_t create(Bootstrap* bs, int device, void* ctrl_area, PciePath** out);

  // `stride`: leading elements of every segment that belong to the other
  // path; this path handles [stride, seg_count) of each segment.
  hlResult_t allReduce(const void* send, void* recv, size_t count, hlDataType_t t, hlRedOp_t op, float scale,
                       hlStream_t stream);
  hlResult_t reduceScatter(const void* send, void* recv, size_t seg_count, size_t stride, hlDataType_t t,
                           hlRedOp_t op, float scale, hlStream_t stream);
  hlResult_t allGather(const void* send, void* recv, size_t seg_count, size_t stride, hlDataType_t t,
                       hlStream_t stream);
  hlResult_t allToAll(const void* send, void* recv, size_t seg_count, size_t stride, hlDataType_t t,
                      hlStream_t stream);
  hlResult_t broadcast(const void* send, void* recv, size_t count, hlDataType_t t, int root, hlStream_t stream);
  // Runs a schedule given as XML text (the reference's pcclSubmitIR).
  hlResult_t submitIr(const char* xml, const void* send, void* recv, size_t seg_count, size_t stride, int send_segs,
                      int recv_segs, hlDataType_t t, hlRedOp_t op, hlStream_t stream);
  // Blocks the host until everything submitted so far has completed.
  hlResult_t drain();
  hlResult_t lastResult() const;
  uint64_t kernelLaunches() const;
  uint64_t copyOps() const;
  uint64_t fusedSlices() const;
  uint64_t rangeJobs() const;   // H2H nodes handed to worker teams as a whole
  uint64_t smallCalls() const;
  uint64_t foldedSources() const;
  uint64_t composedAllReduces() const;   // all-reduces run as reduce-scatter + in-place all-gather (HYLINK_PCIE_AR_COMPOSE)
  // Logical NUMA node of every rank.
  const std::vector<int>& rankNuma() const;
  PcieImpl* impl() { return impl_; }

 private:
  PciePath() = default;
  PcieImpl* impl_ = nullptr;
  std::atomic<uint64_t> composed_{0};
};

}  // namespace hl
