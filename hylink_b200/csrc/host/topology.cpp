#include "host/topology.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <sched.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
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

// ---------------------------------------------------------------------- NVML by dlopen
namespace {
struct Nvml {
  void* handle = nullptr;
  int (*init)() = nullptr;
  int (*byBus)(const char*, void**) = nullptr;
  int (*ancestor)(void*, void*, int*) = nullptr;
  int (*p2p)(void*, void*, int, int*) = nullptr;   // optional
  bool ready = false;
  Nvml() {
    const std::string lib = envStr({"HYLINK_NVML_LIB"}, "libnvidia-ml.so.1");
    handle = dlopen(lib.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!handle) return;
    init = reinterpret_cast<int (*)()>(dlsym(handle, "nvmlInit_v2"));
    byBus = reinterpret_cast<int (*)(const char*, void**)>(dlsym(handle, "nvmlDeviceGetHandleByPciBusId_v2"));
    ancestor = reinterpret_cast<int (*)(void*, void*, int*)>(dlsym(handle, "nvmlDeviceGetTopologyCommonAncestor"));
    p2p = reinterpret_cast<int (*)(void*, void*, int, int*)>(dlsym(handle, "nvmlDeviceGetP2PStatus"));
    ready = init && byBus && ancestor && init() == 0;
  }
};
Nvml& nvml() {
  static Nvml* api = new Nvml();   // never unloaded: NVML stays initialised for the life of the process
  return *api;
}
constexpr int kNvmlTopologySingle = 10;     // NVML_TOPOLOGY_SINGLE: the path crosses one PCIe switch
constexpr int kNvmlP2pCapsNvlink = 2;       // NVML_P2P_CAPS_INDEX_NVLINK
}  // namespace

bool nvmlPairQuery(const std::string& bus_a, const std::string& bus_b, bool* same_switch, bool* nvlink) {
  if (same_switch) *same_switch = false;
  if (nvlink) *nvlink = false;
  Nvml& api = nvml();
  if (!api.ready) return false;
  void *a = nullptr, *b = nullptr;
  if (api.byBus(bus_a.c_str(), &a) != 0 || api.byBus(bus_b.c_str(), &b) != 0) return false;
  int level = -1;
  if (api.ancestor(a, b, &level) != 0) return false;
  if (same_switch) *same_switch = level == kNvmlTopologySingle;
  int status = -1;
  if (nvlink && api.p2p && api.p2p(a, b, kNvmlP2pCapsNvlink, &status) == 0) *nvlink = status == 0;   // NVML_P2P_STATUS_OK
  return true;
}

hlResult_t discoverPairTopology(Bootstrap* bs, int device, PairTopology* out) {
  const int n = bs->nranks();
  struct Pub {
    char bus[32];
    int dev;
  } mine, all[kMaxRanks];
  memset(&mine, 0, sizeof(mine));
  mine.dev = device;
  if (device >= 0 && cudaAvailable() && cudaDeviceGetPCIBusId(mine.bus, sizeof(mine.bus), device) != cudaSuccess) {
    cudaGetLastError();
    mine.bus[0] = 0;
  }
  HL_CHECK(bs->allGather(&mine, sizeof(mine), all));
  out->n = n;
  out->pix.assign((size_t)n * n, 0);
  out->nvlink.assign((size_t)n * n, 0);
  out->peer.assign((size_t)n * n, 0);
  const bool force_switch = Config::get().force_pcie_switch, force_nvlink = Config::get().force_nvlink;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      if (i == j) continue;
      bool pix = false, nvl = false;
      if (all[i].bus[0] && all[j].bus[0]) nvmlPairQuery(all[i].bus, all[j].bus, &pix, &nvl);
      out->pix[(size_t)i * n + j] = pix || force_switch;
      out->nvlink[(size_t)i * n + j] = nvl || force_nvlink;
      int can = 0;
      if (all[i].dev >= 0 && all[j].dev >= 0 && cudaAvailable() && cudaDeviceCanAccessPeer(&can, all[i].dev, all[j].dev) != cudaSuccess) {
        cudaGetLastError();
        can = 0;
      }
      out->peer[(size_t)i * n + j] = (pix || force_switch) && can;
    }
  return hlSuccess;
}

bool directVariantAllowed(const std::string& collective, const std::string& pattern, const PairTopology& t) {
  const int n = (int)pattern.size();
  if (t.n != n || n < 2) return false;
  auto both = [&](int i, int j) { return t.at(t.peer, i, j) && t.at(t.peer, j, i); };
  if (collective.compare(0, 14, "broadcast_root") == 0 || collective == "broadcast") {
    // every rank copies from the root (or from its pair partner): peer access inside the pairs, or everywhere
    if (n == 2) return both(0, 1);
    if (n == 4) return both(0, 1) && both(2, 3);
    for (int i = 0; i < n; ++i)
      for (int j = i + 1; j < n; ++j)
        if (!both(i, j)) return false;
    return true;
  }
  const bool pair_patterns = pattern == "00" || pattern == "0000" || pattern == "0011";
  const bool coll_ok = collective == "allgather" || collective == "reducescatter" || (collective == "allreduce" && (pattern == "00" || pattern == "0000"));
  if (!pair_patterns || !coll_ok) return false;
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j)
      if (i != j && t.at(t.nvlink, i, j)) return false;   // NVLink carries device-to-device traffic on the other path
  for (int p = 0; p + 1 < n; p += 2)
    if (!(t.at(t.pix, p, p + 1) && both(p, p + 1))) return false;
  return true;
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
