// Single-node rendezvous and control plane shared by all ranks of a
// communicator.
//
// One control block per communicator holds: a header, one slot per rank
// (pid, device, NUMA node, heartbeat, failure latch), sense-reversing barrier
// slots, and a mailbox per rank for small all-gathers (IPC handles, pointers).
// In multi-process mode the block is a POSIX shared-memory object named after
// the unique id; in single-process mode (zeroed id, ranks are threads) it is
// heap memory found through a process-wide table. File descriptors travel as
// SCM_RIGHTS datagrams over abstract-namespace unix sockets (multi-process) or
// as dup()ed numbers through the mailbox (single-process).
//
// Parity: covers pcie-ccl-cuda/src/memory/shm_allocator.cpp:98-363 (bootstrap
// shm, UDS fd server), the barrier of src/memory/shared_state.cpp:140-177 and
// the liveness probes of src/api/nccl_compat/compat_common.cpp:108-116.
// Unlike the reference the shm name is unlinked as soon as every rank has
// attached, so a crashed job leaves nothing behind in /dev/shm.
#pragma once
#include <atomic>
#include <string>
#include <vector>

#include "core/core.h"

namespace hl {

constexpr int kMaxRanks = 8;
constexpr int kBarrierSlots = 8;
constexpr size_t kMailboxBytes = 8192;
constexpr uint64_t kCtrlMagic = 0x484c4b3230304231ull;  // "HLK200B1"

struct alignas(64) RankSlot {
  std::atomic<int32_t> pid;
  std::atomic<int32_t> device;
  std::atomic<int32_t> numa;
  std::atomic<int32_t> failed;       // latched by the rank itself or by a peer that saw it die
  std::atomic<uint64_t> heartbeat_ns;
  std::atomic<uint64_t> user_word;   // free for upper layers (doorbell sequence mirrors)
};

struct alignas(64) BarrierSlot {
  std::atomic<uint32_t> count;
  std::atomic<uint32_t> sense;
};

struct CtrlBlock {
  std::atomic<uint64_t> magic;
  uint32_t nranks;
  uint32_t layout_version;
  std::atomic<uint32_t> attached;
  std::atomic<uint32_t> abort_flag;
  uint64_t extra_bytes;              // size of the upper layers' area behind the mailboxes
  RankSlot ranks[kMaxRanks];
  BarrierSlot barriers[kBarrierSlots];
  alignas(64) unsigned char mailbox[kMaxRanks][kMailboxBytes];
  // followed by extra_bytes of zero-initialised memory (see Bootstrap::extra())
};

enum BarrierSite { kBarInit = 0, kBarExchange = 1, kBarSymm = 2, kBarExec = 3, kBarOrch = 4, kBarUser = 5 };

class Bootstrap {
 public:
  ~Bootstrap();
  // extra_bytes: area for upper layers, identical on all ranks.
  static hlResult_t create(const hlUniqueId& id, int nranks, int rank, size_t extra_bytes, int timeout_ms,
                           Bootstrap** out);
  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  bool singleProcess() const { return single_process_; }
  CtrlBlock* block() const { return block_; }
  void* extra() const { return extra_; }
  size_t extraBytes() const { return block_ ? (size_t)block_->extra_bytes : 0; }
  const std::string& tag() const { return tag_; }

  // Returns hlTimeout when peers do not arrive in time, hlRemoteError when a
  // peer's process is gone or has latched a failure.
  hlResult_t barrier(int site = kBarUser, int timeout_ms = -1);
  // Every rank contributes `bytes` (<= kMailboxBytes); `all` receives nranks*bytes.
  hlResult_t allGather(const void* mine, size_t bytes, void* all);
  // Every rank contributes one fd (or -1); fds[q] receives a descriptor that is
  // valid in THIS process for rank q's object (fds[rank] == my_fd).
  hlResult_t exchangeFds(int my_fd, int* fds);
  // Root sends one fd to everyone.
  hlResult_t broadcastFd(int root, int my_fd, int* out_fd);
  void publishSelf(int device, int numa);
  void heartbeat();
  void latchFailure();
  bool peerAlive(int q) const;
  bool anyFailed() const;

 private:
  Bootstrap() = default;
  hlResult_t openUds();
  hlResult_t sendFdTo(int q, int fd, uint32_t tag);
  hlResult_t recvFd(int* from, int* fd, uint32_t tag, int timeout_ms);
  int rank_ = 0, nranks_ = 1;
  bool single_process_ = false;
  CtrlBlock* block_ = nullptr;
  void* extra_ = nullptr;
  size_t map_bytes_ = 0;
  std::string tag_;      // 16 hex digits derived from the unique id
  std::string shm_name_;
  int uds_ = -1;
  int timeout_ms_ = 120000;
  uint32_t local_sense_[kBarrierSlots] = {0};
  uint32_t fd_seq_ = 0;
  std::vector<std::pair<int, std::pair<int, uint32_t>>> early_;  // (from, (fd, tag)) received ahead of time
};

void setAttachTimeoutMs(int ms);
uint64_t hashId(const hlUniqueId& id);
bool idIsZero(const hlUniqueId& id);

}  // namespace hl
