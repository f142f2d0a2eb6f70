// The communicator object behind hlComm_t / pcclComm_t / ncclComm_t.
#pragma once
#include <atomic>
#include <memory>
#include <mutex>

#include "ctrl/bootstrap.h"
#include "nvl/nvl_path.h"

namespace hl {
class PciePath;
class Orchestrator;
}

struct hlComm {
  int rank = 0;
  int nranks = 1;
  int device = -1;           // CUDA ordinal, or -2 for the host-memory device
  bool host_device = false;
  hl::Bootstrap* bs = nullptr;
  hl::NvlPath* nvl = nullptr;
  hl::PciePath* pcie = nullptr;
  hl::Orchestrator* orch = nullptr;
  std::atomic<int> async_error{hlSuccess};
  std::mutex mu;
  hlCommStats stats{};
  uint64_t id_hash = 0;
};

namespace hl {
// Maps a device status recorded by a kernel to the communicator's latched error.
hlResult_t pollDeviceStatus(hlComm* c);
}
