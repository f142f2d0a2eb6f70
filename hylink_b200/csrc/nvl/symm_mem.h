// Symmetric peer-mapped device memory for the NVLink path.
//
// Every rank contributes one allocation of the same size; afterwards each
// rank holds a pointer to every peer's allocation (loads and stores through
// it travel over NVLink) and, when the fabric supports it, one multicast
// pointer whose stores land in all ranks' memory and whose load-reduce sums
// them inside NVSwitch (NVLS).
//
// Modes: (1) cuMemCreate with POSIX file-descriptor handles, descriptors
// passed between processes as SCM_RIGHTS messages, peers imported and mapped,
// plus cuMulticastCreate/BindMem; (2) cudaMalloc + cudaIpc handles (no
// multicast); (3) one process, threads as ranks: plain pointers with peer
// access enabled.
//
// Parity: the reference publishes device buffers between processes with
// cudaIpcGetMemHandle / cudaIpcOpenMemHandle only
// (pcie-ccl-cuda/src/core/process_state.cpp:329-510) and uses the cuMem +
// SCM_RIGHTS mechanism for pinned HOST memory
// (pcie-ccl-cuda/src/memory/host_pool.cpp:95-385); it never maps device memory
// through multicast objects because its NVLink path is the vendor library.
#pragma once
#include "ctrl/bootstrap.h"
#include "hal/cuda_driver.h"

namespace hl {

enum SymmMode { kSymmNone = 0, kSymmVmm = 1, kSymmIpc = 2, kSymmInProcess = 3 };

struct SymmRegion {
  size_t bytes = 0;
  size_t map_bytes = 0;
  int mode = kSymmNone;
  int device = -1;
  int nranks = 0;
  int rank = 0;
  void* ptr[kMaxRanks] = {nullptr};
  void* mc = nullptr;
  unsigned long long handle[kMaxRanks] = {0};
  unsigned long long mc_handle = 0;
  bool mc_bound = false;
};

// Collective over the communicator's bootstrap. `want_mc`: -1 try, 0 never,
// 1 fail if impossible. `mode_pref`: "auto" | "vmm" | "ipc".
hlResult_t symmAlloc(Bootstrap* bs, int device, size_t bytes, int want_mc, const std::string& mode_pref,
                     SymmRegion* out);
// Collective unless `peers_gone` (then no barrier is attempted).
void symmFree(Bootstrap* bs, SymmRegion* r, bool peers_gone);

}  // namespace hl
