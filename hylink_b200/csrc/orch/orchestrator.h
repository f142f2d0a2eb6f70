// Multipath orchestrator facade: forks a collective over the NVLink path and
// the PCIe path, joins them on the device, and retunes the split online.
// See orch/orchestrator.cpp for the design notes.
#pragma once
#include <string>

#include "core/core.h"

struct hlComm;

namespace hl {

class OrchImpl;

class Orchestrator {
 public:
  ~Orchestrator();
  static size_t ctrlBytes(int nranks);
  static hlResult_t create(hlComm* comm, void* ctrl_area, Orchestrator** out);
  // Intercept policy: is this message large enough to be worth forking?
  bool shouldSplit(size_t bytes) const;
  hlResult_t allReduce(const void* send, void* recv, size_t count, hlDataType_t t, hlRedOp_t op, float scale, int algo,
                       hlStream_t stream);
  hlResult_t reduceScatter(const void* send, void* recv, size_t recvcount, hlDataType_t t, hlRedOp_t op, float scale,
                           hlStream_t stream);
  hlResult_t allGather(const void* send, void* recv, size_t sendcount, hlDataType_t t, hlStream_t stream);
  hlResult_t allToAll(const void* send, void* recv, size_t count, hlDataType_t t, hlStream_t stream);
  void fillStats(hlCommStats* out) const;
  std::string dumpTuning() const;
  hlResult_t loadTuning(const char* json);

 private:
  Orchestrator() = default;
  OrchImpl* impl_ = nullptr;
};

}  // namespace hl
