#include "ctrl/bootstrap.h"

#include <atomic>
#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <new>
#include <thread>

namespace hl {

uint64_t hashId(const hlUniqueId& id) {
  uint64_t h = 0xcbf29ce484222325ull;  // FNV-1a
  for (int i = 0; i < HL_UNIQUE_ID_BYTES; ++i) {
    h ^= (unsigned char)id.internal[i];
    h *= 0x100000001b3ull;
  }
  return h;
}
// Ranks that are threads of one process rendezvous in process memory. Their id starts with a zero byte (ids made by
// hlGetUniqueId never do); the bytes behind it tell groups apart, so that two groups of the same size can be set up
// at the same time. The all-zero id (the reference's convention for single-process mode) is the group with tag 0.
bool idIsZero(const hlUniqueId& id) { return id.internal[0] == 0; }
static uint64_t inProcessTag(const hlUniqueId& id) {
  uint64_t h = 0;
  for (int i = 1; i < HL_UNIQUE_ID_BYTES; ++i)
    if (id.internal[i]) return hashId(id);
  return h;
}

// Rendezvous limit of the NEXT Bootstrap::create on this thread (0 = the
// configured barrier timeout). Lets a caller probe "are all ranks on this
// node?" with a short wait without shortening the run-time barriers.
static thread_local int g_attach_timeout_ms = 0;
void setAttachTimeoutMs(int ms) { g_attach_timeout_ms = ms; }

static void backoff(uint32_t& spins) {
  ++spins;
  if (spins < 256) cpuRelax();
  else if (spins < 2048) sched_yield();
  else {
    struct timespec ts = {0, 50000};
    nanosleep(&ts, nullptr);
  }
}

// ---- single-process groups --------------------------------------------
struct SpGroup {
  void* mem = nullptr;
  size_t bytes = 0;
  uint32_t taken = 0;
  int released = 0;
  uint64_t serial = 0;
  ~SpGroup() { free(mem); }
};
static std::mutex g_sp_mu;
static std::map<std::pair<int, uint64_t>, std::shared_ptr<SpGroup>> g_sp_open;  // (nranks, group tag) -> group still missing ranks
static std::map<CtrlBlock*, std::shared_ptr<SpGroup>> g_sp_live;
static uint64_t g_sp_serial = 0;

static size_t blockBytes(size_t extra) { return ((sizeof(CtrlBlock) + 4095) & ~(size_t)4095) + extra; }

static void initBlock(CtrlBlock* b, int nranks, size_t extra) {
  // memory is zero-filled by ftruncate / calloc; set what is not zero
  b->nranks = (uint32_t)nranks;
  b->layout_version = 1;
  b->extra_bytes = extra;
  b->magic.store(kCtrlMagic, std::memory_order_release);
}

Bootstrap::~Bootstrap() {
  if (uds_ >= 0) close(uds_);
  if (!block_) return;
  if (single_process_) {
    std::lock_guard<std::mutex> lk(g_sp_mu);
    auto it = g_sp_live.find(block_);
    if (it != g_sp_live.end()) {
      if (++it->second->released >= nranks_) g_sp_live.erase(it);
    }
  } else {
    munmap(block_, map_bytes_);
  }
}

hlResult_t Bootstrap::create(const hlUniqueId& id, int nranks, int rank, size_t extra_bytes, int timeout_ms,
                             Bootstrap** out) {
  if (nranks < 1 || nranks > kMaxRanks) return fail(hlInvalidArgument, "nranks %d out of [1,%d]", nranks, kMaxRanks);
  if (rank < 0 || rank >= nranks) return fail(hlInvalidArgument, "rank %d out of [0,%d)", rank, nranks);
  extra_bytes = (extra_bytes + 4095) & ~(size_t)4095;
  std::unique_ptr<Bootstrap> b(new Bootstrap());
  b->rank_ = rank;
  b->nranks_ = nranks;
  const int run_timeout = timeout_ms > 0 ? timeout_ms : Config::get().barrier_timeout_ms;
  b->timeout_ms_ = g_attach_timeout_ms > 0 ? g_attach_timeout_ms : run_timeout;
  g_attach_timeout_ms = 0;
  b->map_bytes_ = blockBytes(extra_bytes);
  b->single_process_ = idIsZero(id);
  char tag[32];
  if (b->single_process_) {
    std::lock_guard<std::mutex> lk(g_sp_mu);
    std::shared_ptr<SpGroup> g;
    const std::pair<int, uint64_t> key(nranks, inProcessTag(id));
    auto it = g_sp_open.find(key);
    if (it != g_sp_open.end() && !(it->second->taken & (1u << rank)) && it->second->bytes == b->map_bytes_) g = it->second;
    if (!g) {
      g = std::make_shared<SpGroup>();
      g->bytes = b->map_bytes_;
      if (posix_memalign(&g->mem, 4096, g->bytes) != 0) return fail(hlSystemError, "out of memory for control block");
      memset(g->mem, 0, g->bytes);
      g->serial = ++g_sp_serial;
      initBlock(new (g->mem) CtrlBlock, nranks, extra_bytes);
      g_sp_open[key] = g;
      g_sp_live[(CtrlBlock*)g->mem] = g;
    }
    g->taken |= (1u << rank);
    if (g->taken == (nranks >= 32 ? 0xffffffffu : ((1u << nranks) - 1))) g_sp_open.erase(key);
    b->block_ = (CtrlBlock*)g->mem;
    snprintf(tag, sizeof(tag), "sp%d_%llx", (int)getpid(), (unsigned long long)g->serial);
  } else {
    snprintf(tag, sizeof(tag), "%016llx", (unsigned long long)hashId(id));
    b->shm_name_ = std::string("/hylink_") + tag;
    bool creator = false;
    int fd = shm_open(b->shm_name_.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd >= 0) {
      creator = true;
      if (ftruncate(fd, (off_t)b->map_bytes_) != 0) {
        int e = errno;
        close(fd);
        shm_unlink(b->shm_name_.c_str());
        return fail(hlSystemError, "ftruncate(%s, %zu): %s", b->shm_name_.c_str(), b->map_bytes_, strerror(e));
      }
    } else if (errno == EEXIST) {
      const uint64_t t0 = nowNs();
      uint32_t spins = 0;
      for (;;) {
        fd = shm_open(b->shm_name_.c_str(), O_RDWR, 0600);
        if (fd >= 0) {
          struct stat st;
          if (fstat(fd, &st) == 0 && (size_t)st.st_size >= b->map_bytes_) break;
          close(fd);
          fd = -1;
        }
        if ((nowNs() - t0) / 1000000ull > (uint64_t)b->timeout_ms_)
          return fail(hlTimeout, "control block %s did not appear", b->shm_name_.c_str());
        backoff(spins);
      }
    } else {
      return fail(hlSystemError, "shm_open(%s): %s", b->shm_name_.c_str(), strerror(errno));
    }
    void* p = mmap(nullptr, b->map_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) return fail(hlSystemError, "mmap control block: %s", strerror(errno));
    b->block_ = (CtrlBlock*)p;
    if (creator) initBlock(b->block_, nranks, extra_bytes);
    const uint64_t t0 = nowNs();
    uint32_t spins = 0;
    while (b->block_->magic.load(std::memory_order_acquire) != kCtrlMagic) {
      if ((nowNs() - t0) / 1000000ull > (uint64_t)b->timeout_ms_) return fail(hlTimeout, "control block never initialised");
      backoff(spins);
    }
    if (b->block_->nranks != (uint32_t)nranks || b->block_->extra_bytes != extra_bytes)
      return fail(hlInvalidArgument, "control block mismatch: nranks %u vs %d, extra %llu vs %zu", b->block_->nranks,
                  nranks, (unsigned long long)b->block_->extra_bytes, extra_bytes);
  }
  b->tag_ = tag;
  b->extra_ = (char*)b->block_ + ((sizeof(CtrlBlock) + 4095) & ~(size_t)4095);
  b->block_->ranks[rank].pid.store((int32_t)getpid());
  b->block_->ranks[rank].heartbeat_ns.store(nowNs());
  if (!b->single_process_) HL_CHECK(b->openUds());
  const uint32_t att = b->block_->attached.fetch_add(1) + 1;
  // Everybody is in: the name has served its purpose.
  hlResult_t r = b->barrier(kBarInit);
  b->timeout_ms_ = run_timeout;
  if (!b->single_process_ && att == (uint32_t)nranks) shm_unlink(b->shm_name_.c_str());
  if (r != hlSuccess) {
    if (!b->single_process_) shm_unlink(b->shm_name_.c_str());
    return r;
  }
  *out = b.release();
  return hlSuccess;
}

void Bootstrap::publishSelf(int device, int numa) {
  block_->ranks[rank_].device.store(device);
  block_->ranks[rank_].numa.store(numa);
}
void Bootstrap::heartbeat() { block_->ranks[rank_].heartbeat_ns.store(nowNs(), std::memory_order_relaxed); }
void Bootstrap::latchFailure() {
  block_->ranks[rank_].failed.store(1);
  block_->abort_flag.store(1);
}
bool Bootstrap::peerAlive(int q) const {
  if (block_->ranks[q].failed.load()) return false;
  if (single_process_) return true;
  const int pid = block_->ranks[q].pid.load();
  if (pid <= 0) return true;  // not yet published
  return kill(pid, 0) == 0 || errno == EPERM;
}
bool Bootstrap::anyFailed() const {
  if (block_->abort_flag.load(std::memory_order_relaxed)) return true;
  for (int q = 0; q < nranks_; ++q)
    if (block_->ranks[q].failed.load(std::memory_order_relaxed)) return true;
  return false;
}

hlResult_t Bootstrap::barrier(int site, int timeout_ms) {
  if (nranks_ == 1) return hlSuccess;
  if (timeout_ms < 0) timeout_ms = timeout_ms_;
  BarrierSlot& s = block_->barriers[site % kBarrierSlots];
  const uint32_t sense = (local_sense_[site % kBarrierSlots] ^= 1u);
  if (s.count.fetch_add(1, std::memory_order_acq_rel) + 1 == (uint32_t)nranks_) {
    s.count.store(0, std::memory_order_relaxed);
    s.sense.store(sense, std::memory_order_release);
    return hlSuccess;
  }
  const uint64_t t0 = nowNs();
  uint32_t spins = 0;
  while (s.sense.load(std::memory_order_acquire) != sense) {
    backoff(spins);
    if ((spins & 1023u) == 0) {
      if (block_->abort_flag.load()) return fail(hlRemoteError, "barrier(site %d): communicator aborted by a peer", site);
      for (int q = 0; q < nranks_; ++q)
        if (q != rank_ && !peerAlive(q)) {
          block_->abort_flag.store(1);
          return fail(hlRemoteError, "barrier(site %d): rank %d is gone", site, q);
        }
      if ((nowNs() - t0) / 1000000ull > (uint64_t)timeout_ms)
        return fail(hlTimeout, "barrier(site %d) timed out after %d ms (rank %d of %d)", site, timeout_ms, rank_, nranks_);
    }
  }
  return hlSuccess;
}

hlResult_t Bootstrap::allGather(const void* mine, size_t bytes, void* all) {
  if (bytes > kMailboxBytes) return fail(hlInvalidArgument, "allGather blob of %zu bytes exceeds %zu", bytes, kMailboxBytes);
  memcpy(block_->mailbox[rank_], mine, bytes);
  HL_CHECK(barrier(kBarExchange));
  for (int q = 0; q < nranks_; ++q) memcpy((char*)all + (size_t)q * bytes, block_->mailbox[q], bytes);
  return barrier(kBarExchange);
}

// ---- fd passing --------------------------------------------------------
static void udsAddr(const std::string& tag, int rank, sockaddr_un* sa, socklen_t* len) {
  memset(sa, 0, sizeof(*sa));
  sa->sun_family = AF_UNIX;
  char name[96];
  int n = snprintf(name, sizeof(name), "hylink_%s_%d", tag.c_str(), rank);
  sa->sun_path[0] = '\0';  // abstract namespace: vanishes with the socket
  memcpy(sa->sun_path + 1, name, (size_t)n);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

hlResult_t Bootstrap::openUds() {
  uds_ = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (uds_ < 0) return fail(hlSystemError, "socket(AF_UNIX): %s", strerror(errno));
  sockaddr_un sa;
  socklen_t len;
  udsAddr(tag_, rank_, &sa, &len);
  if (bind(uds_, (sockaddr*)&sa, len) != 0) return fail(hlSystemError, "bind unix socket: %s", strerror(errno));
  return hlSuccess;
}

hlResult_t Bootstrap::sendFdTo(int q, int fd, uint32_t tag) {
  sockaddr_un sa;
  socklen_t len;
  udsAddr(tag_, q, &sa, &len);
  uint32_t payload[2] = {(uint32_t)rank_, tag};
  struct iovec iov = {payload, sizeof(payload)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_name = &sa;
  msg.msg_namelen = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  if (fd >= 0) {
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  const uint64_t t0 = nowNs();
  uint32_t spins = 0;
  for (;;) {
    if (sendmsg(uds_, &msg, 0) >= 0) return hlSuccess;
    if (errno != ECONNREFUSED && errno != ENOENT && errno != EAGAIN && errno != ENOBUFS && errno != EINTR)
      return fail(hlSystemError, "sendmsg(fd) to rank %d: %s", q, strerror(errno));
    if ((nowNs() - t0) / 1000000ull > (uint64_t)timeout_ms_) return fail(hlTimeout, "sendmsg(fd) to rank %d timed out", q);
    backoff(spins);
  }
}

hlResult_t Bootstrap::recvFd(int* from, int* fd, uint32_t tag, int timeout_ms) {
  for (size_t i = 0; i < early_.size(); ++i)
    if (early_[i].second.second == tag) {
      *from = early_[i].first;
      *fd = early_[i].second.first;
      early_.erase(early_.begin() + (long)i);
      return hlSuccess;
    }
  const uint64_t t0 = nowNs();
  for (;;) {
    pollfd p = {uds_, POLLIN, 0};
    int pr = poll(&p, 1, 100);
    if (pr < 0 && errno != EINTR) return fail(hlSystemError, "poll: %s", strerror(errno));
    if (pr > 0) {
      uint32_t payload[2] = {0, 0};
      struct iovec iov = {payload, sizeof(payload)};
      alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
      msghdr msg;
      memset(&msg, 0, sizeof(msg));
      msg.msg_iov = &iov;
      msg.msg_iovlen = 1;
      msg.msg_control = ctrl;
      msg.msg_controllen = sizeof(ctrl);
      ssize_t n = recvmsg(uds_, &msg, MSG_CMSG_CLOEXEC);
      if (n < 0) {
        if (errno == EINTR || errno == EAGAIN) continue;
        return fail(hlSystemError, "recvmsg: %s", strerror(errno));
      }
      int got = -1;
      for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c))
        if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(&got, CMSG_DATA(c), sizeof(int));
      if (payload[1] == tag) {
        *from = (int)payload[0];
        *fd = got;
        return hlSuccess;
      }
      early_.push_back({(int)payload[0], {got, payload[1]}});
      continue;
    }
    if (anyFailed()) return fail(hlRemoteError, "fd exchange: a peer failed");
    if ((nowNs() - t0) / 1000000ull > (uint64_t)timeout_ms) return fail(hlTimeout, "fd exchange timed out");
  }
}

hlResult_t Bootstrap::exchangeFds(int my_fd, int* fds) {
  const uint32_t tag = ++fd_seq_;
  if (single_process_) {
    // Same descriptor table: publish the number, readers dup() it.
    int all[kMaxRanks];
    HL_CHECK(allGather(&my_fd, sizeof(int), all));
    for (int q = 0; q < nranks_; ++q) fds[q] = (q == rank_) ? my_fd : (all[q] >= 0 ? dup(all[q]) : -1);
    return barrier(kBarExchange);  // owners may close only after everyone dup()ed
  }
  for (int q = 0; q < nranks_; ++q) fds[q] = -1;
  fds[rank_] = my_fd;
  for (int k = 1; k < nranks_; ++k) HL_CHECK(sendFdTo((rank_ + k) % nranks_, my_fd, tag));
  for (int k = 1; k < nranks_; ++k) {
    int from = -1, fd = -1;
    HL_CHECK(recvFd(&from, &fd, tag, timeout_ms_));
    if (from < 0 || from >= nranks_) return fail(hlInternalError, "fd exchange: bad sender %d", from);
    fds[from] = fd;
  }
  return barrier(kBarExchange);
}

hlResult_t Bootstrap::broadcastFd(int root, int my_fd, int* out_fd) {
  const uint32_t tag = ++fd_seq_;
  if (single_process_) {
    int all[kMaxRanks];
    int v = (rank_ == root) ? my_fd : -1;
    HL_CHECK(allGather(&v, sizeof(int), all));
    *out_fd = (rank_ == root) ? my_fd : dup(all[root]);
    return barrier(kBarExchange);
  }
  if (rank_ == root) {
    for (int q = 0; q < nranks_; ++q)
      if (q != root) HL_CHECK(sendFdTo(q, my_fd, tag));
    *out_fd = my_fd;
  } else {
    int from = -1;
    HL_CHECK(recvFd(&from, out_fd, tag, timeout_ms_));
  }
  return barrier(kBarExchange);
}

}  // namespace hl

// An id for ranks that are threads of ONE process: a zero byte, then a tag that tells this group from others.
extern "C" hlResult_t hlGetInProcessId(hlUniqueId* id) {
  if (!id) return hlInvalidArgument;
  static std::atomic<uint64_t> serial{0};
  memset(id, 0, sizeof(*id));
  snprintf(id->internal + 1, sizeof(id->internal) - 1, "inproc-%d-%llu", (int)getpid(), (unsigned long long)serial.fetch_add(1) + 1);
  return hlSuccess;
}

extern "C" hlResult_t hlGetUniqueId(hlUniqueId* id) {
  if (!id) return hlInvalidArgument;
  memset(id, 0, sizeof(*id));
  unsigned char rnd[24];
  int fd = open("/dev/urandom", O_RDONLY | O_CLOEXEC);
  bool ok = false;
  if (fd >= 0) {
    ok = read(fd, rnd, sizeof(rnd)) == (ssize_t)sizeof(rnd);
    close(fd);
  }
  if (!ok) {
    uint64_t a = hl::nowNs() ^ ((uint64_t)getpid() << 32), b = hl::wallUs();
    memcpy(rnd, &a, 8);
    memcpy(rnd + 8, &b, 8);
    memcpy(rnd + 16, &a, 8);
  }
  // printable, so that it can travel through environment variables and stores
  static const char* hex = "0123456789abcdef";
  for (size_t i = 0; i < sizeof(rnd); ++i) {
    id->internal[2 * i] = hex[rnd[i] >> 4];
    id->internal[2 * i + 1] = hex[rnd[i] & 15];
  }
  return hlSuccess;
}

// Self-check of the control plane, callable from tests without a GPU: barrier,
// mailbox all-gather and descriptor passing between `nranks` processes/threads.
extern "C" hlResult_t hlCtrlSelfTest(hlUniqueId id, int nranks, int rank, int rounds) {
  using namespace hl;
  Bootstrap* raw = nullptr;
  HL_CHECK(Bootstrap::create(id, nranks, rank, 8192, 20000, &raw));
  std::unique_ptr<Bootstrap> bs(raw);
  if (bs->extraBytes() < 8192) return fail(hlInternalError, "extra area too small");
  for (int it = 0; it < rounds; ++it) {
    int64_t mine = 1000 * it + rank, all[kMaxRanks];
    HL_CHECK(bs->allGather(&mine, sizeof(mine), all));
    for (int q = 0; q < nranks; ++q)
      if (all[q] != 1000 * it + q) return fail(hlInternalError, "allGather mismatch at rank %d", q);
    int fd = memfd_create("hylink_selftest", MFD_CLOEXEC);
    if (fd < 0) return fail(hlSystemError, "memfd_create: %s", strerror(errno));
    int64_t stamp = 7777 + 31 * it + rank;
    if (write(fd, &stamp, sizeof(stamp)) != (ssize_t)sizeof(stamp)) return fail(hlSystemError, "write memfd");
    int fds[kMaxRanks];
    HL_CHECK(bs->exchangeFds(fd, fds));
    for (int q = 0; q < nranks; ++q) {
      int64_t got = 0;
      if (pread(fds[q], &got, sizeof(got), 0) != (ssize_t)sizeof(got) || got != 7777 + 31 * it + q)
        return fail(hlInternalError, "fd from rank %d carries the wrong object", q);
      if (q != rank) close(fds[q]);
    }
    int bfd = -1;
    HL_CHECK(bs->broadcastFd(nranks - 1, fd, &bfd));
    int64_t got = 0;
    if (pread(bfd, &got, sizeof(got), 0) != (ssize_t)sizeof(got) || got != 7777 + 31 * it + (nranks - 1))
      return fail(hlInternalError, "broadcast fd carries the wrong object");
    if (bfd != fd) close(bfd);
    HL_CHECK(bs->barrier(kBarUser));
    close(fd);
  }
  // the shared extra area is really shared
  auto* words = reinterpret_cast<std::atomic<int>*>(bs->extra());
  words[rank].store(rank + 1);
  HL_CHECK(bs->barrier(kBarUser));
  for (int q = 0; q < nranks; ++q)
    if (words[q].load() != q + 1) return fail(hlInternalError, "extra area not shared");
  HL_CHECK(bs->barrier(kBarUser));
  return hlSuccess;
}
