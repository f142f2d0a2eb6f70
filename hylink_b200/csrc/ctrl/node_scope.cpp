#include "ctrl/node_scope.h"

#include <fcntl.h>
#include <signal.h>
#include <sys/file.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <thread>

#include "core/core.h"

namespace hl {

namespace {
constexpr uint32_t kMagic = 0x484c4e53;   // "HLNS"
constexpr int kMaxScopeRanks = 64;
constexpr uint64_t kMaxAgeNs = 600ull * 1000000000ull;   // entries of crashed jobs are ignored after ten minutes

struct Slot {
  int32_t valid, rank, pid, device;
  uint64_t stamp_ns;   // wall clock
};
struct Table {
  uint32_t magic;
  int32_t nranks;
  uint64_t comm_hash, node_hash;
  int32_t left;       // ranks that have dropped their entry
  int32_t pad;
  Slot slot[kMaxScopeRanks];
};

uint64_t fnv(const std::string& s, uint64_t h = 0xcbf29ce484222325ull) {
  for (unsigned char c : s) {
    h ^= c;
    h *= 0x100000001b3ull;
  }
  return h;
}

uint64_t wallNs() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

bool pidAlive(int pid) { return pid > 0 && (kill(pid, 0) == 0 || errno == EPERM); }

std::string tableName(uint64_t comm_hash, uint64_t node_hash) {
  char name[96];
  snprintf(name, sizeof(name), "/hylink_node_%016llx_%016llx", (unsigned long long)comm_hash, (unsigned long long)node_hash);
  return name;
}

Table* openTable(uint64_t comm_hash, int nranks, int* fd_out) {
  const uint64_t node = localNodeHash();
  const std::string name = tableName(comm_hash, node);
  int fd = shm_open(name.c_str(), O_CREAT | O_RDWR, 0600);
  if (fd < 0) return nullptr;
  if (ftruncate(fd, (off_t)sizeof(Table)) != 0) {
    close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, sizeof(Table), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) {
    close(fd);
    return nullptr;
  }
  Table* t = (Table*)p;
  flock(fd, LOCK_EX);
  if (t->magic != kMagic || t->comm_hash != comm_hash || t->node_hash != node || t->nranks != nranks) {
    memset(t, 0, sizeof(*t));   // first user, or a left-over of another layout
    t->magic = kMagic;
    t->comm_hash = comm_hash;
    t->node_hash = node;
    t->nranks = nranks;
  }
  flock(fd, LOCK_UN);
  *fd_out = fd;
  return t;
}

void closeTable(Table* t, int fd) {
  if (t) munmap(t, sizeof(Table));
  if (fd >= 0) close(fd);
}
}  // namespace

uint64_t localNodeHash() {
  static const uint64_t h = [] {
    char host[256] = {0};
    gethostname(host, sizeof(host) - 1);
    std::string boot;
    std::ifstream f("/proc/sys/kernel/random/boot_id");
    if (f) std::getline(f, boot);
    return fnv(std::string(host) + "|" + std::to_string((long)getuid()) + "|" + boot);
  }();
  return h;
}

NodeScope detectNodeScope(uint64_t comm_hash, int nranks, int rank, int device, int wait_ms) {
  NodeScope out;
  out.node_hash = localNodeHash();
  if (nranks < 1 || nranks > kMaxScopeRanks || rank < 0 || rank >= nranks) return out;
  int fd = -1;
  Table* t = openTable(comm_hash, nranks, &fd);
  if (!t) return out;
  flock(fd, LOCK_EX);
  Slot& mine = t->slot[rank];
  __atomic_store_n(&mine.valid, 0, __ATOMIC_SEQ_CST);
  mine.rank = rank;
  mine.pid = (int32_t)getpid();
  mine.device = device;
  mine.stamp_ns = wallNs();
  __atomic_store_n(&mine.valid, 1, __ATOMIC_SEQ_CST);
  flock(fd, LOCK_UN);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(wait_ms < 0 ? 0 : wait_ms);
  for (;;) {
    const uint64_t now = wallNs();
    int seen = 0;
    bool distinct = true, contiguous = true;
    for (int r = 0; r < nranks; ++r) {
      const Slot& s = t->slot[r];
      if (!__atomic_load_n(&s.valid, __ATOMIC_SEQ_CST)) continue;
      if (s.rank != r || !pidAlive(s.pid) || s.stamp_ns > now + 1000000000ull || now - std::min(now, s.stamp_ns) > kMaxAgeNs) continue;
      ++seen;
      if (s.device >= 0) {
        for (int q = 0; q < r; ++q)
          if (t->slot[q].valid && t->slot[q].device == s.device) distinct = false;
        if (t->slot[0].valid && t->slot[0].device >= 0 && s.device != t->slot[0].device + r) contiguous = false;
      }
    }
    out.seen = seen;
    out.all_local = seen == nranks;
    out.distinct = out.all_local && distinct;
    out.contiguous = out.all_local && contiguous;
    if (out.all_local || std::chrono::steady_clock::now() >= deadline) break;
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
  HL_INFO("node scope: comm %016llx nranks=%d seen=%d distinct=%d contiguous=%d", (unsigned long long)comm_hash, nranks, out.seen,
          (int)out.distinct, (int)out.contiguous);
  closeTable(t, fd);
  return out;
}

void leaveNodeScope(uint64_t comm_hash, int nranks, int rank) {
  if (nranks < 1 || nranks > kMaxScopeRanks || rank < 0 || rank >= nranks) return;
  int fd = -1;
  Table* t = openTable(comm_hash, nranks, &fd);
  if (!t) return;
  flock(fd, LOCK_EX);
  bool last = false;
  if (t->slot[rank].valid && t->slot[rank].pid == (int32_t)getpid()) {
    t->slot[rank].valid = 0;
    last = ++t->left >= nranks;
  }
  flock(fd, LOCK_UN);
  if (last) shm_unlink(tableName(comm_hash, localNodeHash()).c_str());
  closeTable(t, fd);
}

}  // namespace hl

extern "C" {
// C view for tools and tests: returns the number of ranks seen; *flags = all_local | distinct << 1 | contiguous << 2.
int hlNodeScopeDetect(uint64_t comm_hash, int nranks, int rank, int device, int wait_ms, int* flags) {
  const hl::NodeScope s = hl::detectNodeScope(comm_hash, nranks, rank, device, wait_ms);
  if (flags) *flags = (s.all_local ? 1 : 0) | (s.distinct ? 2 : 0) | (s.contiguous ? 4 : 0);
  return s.seen;
}
void hlNodeScopeLeave(uint64_t comm_hash, int nranks, int rank) { hl::leaveNodeScope(comm_hash, nranks, rank); }
}
