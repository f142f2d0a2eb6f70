// GPU -> NUMA discovery, thread pinning and page placement without libnuma.
//
// Parity: pcie-ccl-cuda/src/topology/topology.cpp:22-240 (sysfs numa_node of
// the GPU's PCI function, logical compaction, PCCL_GPU_NUMA_MAP override) and
// src/topology/numa.cpp:40-127 (libnuma pinning). Here affinity and placement
// use sched_setaffinity and the mbind system call directly, so the library has
// no build- or run-time dependency on libnuma.
#pragma once
#include <string>
#include <vector>

#include "ctrl/bootstrap.h"

namespace hl {

// Physical NUMA node of a CUDA device (-1 when unknown).
int numaOfCudaDevice(int device);
std::vector<int> cpusOfNumaNode(int node);
int numaNodeCount();
bool pinThreadToNumaNode(int node);
// Best effort; false when the kernel refuses (containers often do).
bool bindMemoryToNumaNode(void* p, size_t bytes, int node);

// Accepts "00001111" or "0,0,0,0,1,1,1,1".
std::vector<int> parseGpuNumaMap(const std::string& text);
// Renumbers physical ids to 0..k-1 in order of first appearance.
std::vector<int> compactNuma(const std::vector<int>& physical, std::vector<int>* physical_of_logical);

// ---- pairwise PCIe / link topology ----------------------------------------------------------------------------------
// What decides whether a schedule may copy between two GPUs directly (the `_direct` schedule files): the two sit
// under one PCIe switch (NVML reports their common ancestor as a single switch), peer access works both ways, and no
// NVLink joins them (with NVLink the dedicated-link path carries that traffic). NVML is opened with dlopen at the
// first query (HYLINK_NVML_LIB names another library, which is how the tests supply a fake one); without it no
// pair counts as switch-local unless HYLINK_FORCE_PCIE_SWITCH / PCCL_FORCE_PCIE_SWITCH says so.
// Parity: pcie-ccl-cuda/src/topology/topology.cpp:22-78,121-167 and src/ir/ir_loader.cpp:254-304.
struct PairTopology {
  int n = 0;
  std::vector<unsigned char> pix, nvlink, peer;   // n x n, row-major: [i * n + j]
  bool at(const std::vector<unsigned char>& m, int i, int j) const { return i == j || (i < n && j < n && m[(size_t)i * n + j] != 0); }
};
// One pair, by PCI bus id ("0000:3b:00.0"). False when NVML is unavailable.
bool nvmlPairQuery(const std::string& bus_a, const std::string& bus_b, bool* same_switch, bool* nvlink);
// Collective: bus ids are exchanged, every rank then fills the whole matrix locally.
hlResult_t discoverPairTopology(Bootstrap* bs, int device, PairTopology* out);
// The selection rule for `<collective>_<pattern>_direct.xml`.
bool directVariantAllowed(const std::string& collective, const std::string& pattern, const PairTopology& t);

// Collective: every rank learns the logical NUMA node of every rank, and the
// physical node behind each logical id.
hlResult_t discoverRankNuma(Bootstrap* bs, int device, std::vector<int>* logical, std::vector<int>* physical_of_logical);

}  // namespace hl
