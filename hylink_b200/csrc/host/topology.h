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

// Collective: every rank learns the logical NUMA node of every rank, and the
// physical node behind each logical id.
hlResult_t discoverRankNuma(Bootstrap* bs, int device, std::vector<int>* logical, std::vector<int>* physical_of_logical);

}  // namespace hl
