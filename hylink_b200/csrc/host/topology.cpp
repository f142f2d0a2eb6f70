#include "host/topology.h"

#include <cuda_runtime.h>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <fstream>
#include <sstream>

#include "hal/cuda_driver.h"

namespace hl {

int numaOfCudaDevice(int device) {
  if (device < 0 || !cudaAvailable()) return -1;
  char bus[64] = {0};
  if (cudaDeviceGetPCIBusId(bus, sizeof(bus), device) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  std::string id(bus);
  for (auto& c : id) c = (char)tolower(c);
  std::ifstream f("/sys/bus/pci/devices/" + id + "/numa_node");
  int node = -1;
  if (f) f >> node;
  return node;
}

std::vector<int> cpusOfNumaNode(int node) {
  std::vector<int> cpus;
  std::ifstream f("/sys/devices/system/node/node" + std::to_string(node) + "/cpulist");
  std::string s;
  if (!f || !std::getline(f, s)) return cpus;
  std::stringstream ss(s);
  std::string part;
  while (std::getline(ss, part, ',')) {
    int a = 0, b = 0;
    if (sscanf(part.c_str(), "%d-%d", &a, &b) == 2) {
      for (int c = a; c <= b; ++c) cpus.push_back(c);
    } else if (sscanf(part.c_str(), "%d", &a) == 1) {
      cpus.push_back(a);
    }
  }
  return cpus;
}

int numaNodeCount() {
  int n = 0;
  while (n < 64) {
    std::ifstream f("/sys/devices/system/node/node" + std::to_string(n) + "/cpulist");
    if (!f) break;
    ++n;
  }
  return n < 1 ? 1 : n;
}

bool pinThreadToNumaNode(int node) {
  if (node < 0) return false;
  std::vector<int> cpus = cpusOfNumaNode(node);
  if (cpus.empty()) return false;
  cpu_set_t allowed, want;
  CPU_ZERO(&allowed);
  if (sched_getaffinity(0, sizeof(allowed), &allowed) != 0) return false;
  CPU_ZERO(&want);
  int k = 0;
  for (int c : cpus)
    if (c < CPU_SETSIZE && CPU_ISSET(c, &allowed)) {
      CPU_SET(c, &want);
      ++k;
    }
  if (!k) return false;  // the container's cpuset excludes that node: keep the current mask
  return sched_setaffinity(0, sizeof(want), &want) == 0;
}

bool bindMemoryToNumaNode(void* p, size_t bytes, int node) {
#ifdef SYS_mbind
  if (node < 0 || node >= 64) return false;
  unsigned long mask = 1ul << node;
  const int MPOL_PREFERRED_ = 1;
  long r = syscall(SYS_mbind, p, bytes, MPOL_PREFERRED_, &mask, sizeof(mask) * 8, 0);
  return r == 0;
#else
  (void)p; (void)bytes; (void)node;
  return false;
#endif
}

std::vector<int> parseGpuNumaMap(const std::string& text) {
  std::vector<int> v;
  if (text.find(',') != std::string::npos) {
    std::stringstream ss(text);
    std::string part;
    while (std::getline(ss, part, ',')) v.push_back(atoi(part.c_str()));
  } else {
    for (char c : text)
      if (isdigit((unsigned char)c)) v.push_back(c - '0');
  }
  return v;
}

std::vector<int> compactNuma(const std::vector<int>& physical, std::vector<int>* phys_of_logical) {
  std::vector<int> order, logical(physical.size(), 0);
  for (size_t i = 0; i < physical.size(); ++i) {
    const int p = physical[i] < 0 ? 0 : physical[i];
    auto it = std::find(order.begin(), order.end(), p);
    if (it == order.end()) {
      order.push_back(p);
      logical[i] = (int)order.size() - 1;
    } else {
      logical[i] = (int)(it - order.begin());
    }
  }
  if (phys_of_logical) *phys_of_logical = order;
  return logical;
}

hlResult_t discoverRankNuma(Bootstrap* bs, int device, std::vector<int>* logical, std::vector<int>* phys_of_logical) {
  const int n = bs->nranks();
  std::vector<int> physical((size_t)n, 0);
  const std::vector<int> forced = parseGpuNumaMap(Config::get().gpu_numa_map);
  int mine = 0;
  if ((int)forced.size() >= n) {
    mine = forced[(size_t)bs->rank()];
  } else if (device >= 0) {
    mine = numaOfCudaDevice(device);
    if (mine < 0) mine = 0;
  }
  int32_t v = mine, all[kMaxRanks];
  HL_CHECK(bs->allGather(&v, sizeof(v), all));
  for (int q = 0; q < n; ++q) physical[(size_t)q] = all[q];
  *logical = compactNuma(physical, phys_of_logical);
  if ((int)forced.size() >= n && phys_of_logical) {
    // a forced map names logical nodes; spread them over the machine's nodes round-robin
    const int nodes = numaNodeCount();
    for (auto& p : *phys_of_logical) p = p % nodes;
  }
  return hlSuccess;
}

}  // namespace hl
