// PCIe path facade: host-staged collectives driven by the schedule IR.
// See pcie/pcie_path.cpp for the design notes.
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

#include "core/core.h"
#include "ctrl/bootstrap.h"

namespace hl {

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
  // Logical NUMA node of every rank.
  const std::vector<int>& rankNuma() const;
  PcieImpl* impl() { return impl_; }

 private:
  PciePath() = default;
  PcieImpl* impl_ = nullptr;
};

}  // namespace hl
