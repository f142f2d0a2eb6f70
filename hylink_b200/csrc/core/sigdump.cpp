// Hang triage without a debugger: with HYLINK_SIGDUMP=1 (alias PCCL_SIGDUMP),
// `kill -USR1 <pid>` makes every thread of the process print its call stack to
// stderr or to HYLINK_SIGDUMP_FILE. A watcher thread receives SIGUSR1 through
// sigwait, walks /proc/self/task and sends each thread a real-time signal
// whose handler writes backtrace() frames with async-signal-safe calls only.
//
// Parity: pcie-ccl-cuda/src/util/sigdump.cpp:57-193.
#include <dirent.h>
#include <execinfo.h>
#include <fcntl.h>
#include <signal.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <mutex>
#include <thread>

#include "core/core.h"

namespace hl {

namespace {
int g_fd = 2;
int g_rt_signal = 0;
std::atomic<int> g_pending{0};
std::once_flag g_once;

void writeStr(const char* s) {
  ssize_t ignored = write(g_fd, s, strlen(s));
  (void)ignored;
}
void writeNum(long v) {
  char buf[24];
  int i = 23;
  buf[i] = 0;
  if (v == 0) buf[--i] = '0';
  while (v > 0 && i > 0) {
    buf[--i] = (char)('0' + v % 10);
    v /= 10;
  }
  writeStr(buf + i);
}

void dumpHandler(int, siginfo_t*, void*) {
  void* frames[48];
  const int n = backtrace(frames, 48);
  writeStr("---- hylink sigdump: thread ");
  writeNum((long)syscall(SYS_gettid));
  writeStr(" ----\n");
  backtrace_symbols_fd(frames, n, g_fd);
  g_pending.fetch_sub(1);
}

void watcher(sigset_t set) {
  for (;;) {
    int sig = 0;
    if (sigwait(&set, &sig) != 0) return;
    if (sig != SIGUSR1) continue;
    writeStr("==== hylink sigdump: process ");
    writeNum((long)getpid());
    writeStr(" ====\n");
    DIR* d = opendir("/proc/self/task");
    if (!d) continue;
    const long self = (long)syscall(SYS_gettid);
    while (dirent* e = readdir(d)) {
      const long tid = atol(e->d_name);
      if (tid <= 0 || tid == self) continue;
      g_pending.fetch_add(1);
      if (syscall(SYS_tgkill, (long)getpid(), tid, g_rt_signal) != 0) g_pending.fetch_sub(1);
    }
    closedir(d);
    for (int i = 0; i < 200 && g_pending.load() > 0; ++i) usleep(5000);
    writeStr("==== hylink sigdump: done ====\n");
  }
}
}  // namespace

void installSigdump() {
  std::call_once(g_once, [] {
    const Config& cfg = Config::get();
    if (!cfg.sigdump) return;
    if (!cfg.sigdump_file.empty()) {
      int fd = open(cfg.sigdump_file.c_str(), O_WRONLY | O_CREAT | O_APPEND | O_CLOEXEC, 0644);
      if (fd >= 0) g_fd = fd;
    }
    // make backtrace() load its unwinder now, not inside a signal handler
    void* warm[2];
    backtrace(warm, 2);
    g_rt_signal = SIGRTMIN + 5;
    struct sigaction sa;
    memset(&sa, 0, sizeof(sa));
    sa.sa_sigaction = dumpHandler;
    sa.sa_flags = SA_SIGINFO | SA_RESTART;
    sigaction(g_rt_signal, &sa, nullptr);
    sigset_t set;
    sigemptyset(&set);
    sigaddset(&set, SIGUSR1);
    // threads created from here on inherit the block; the watcher takes the signal with sigwait
    pthread_sigmask(SIG_BLOCK, &set, nullptr);
    std::thread(watcher, set).detach();
    HL_INFO("sigdump armed: kill -USR1 %d prints every thread's stack", (int)getpid());
  });
}

}  // namespace hl

extern "C" void hlInstallSigdump(void) { hl::installSigdump(); }
