#include "core/trace.h"

#include <nvtx3/nvToolsExt.h>

#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <mutex>
#include <vector>

#include "core/core.h"

namespace hl {

namespace {
std::mutex g_mu;
FILE* g_file = nullptr;
std::atomic<int> g_state{-1};  // -1 unknown, 0 off, 1 on
int g_rank = 0;
bool g_first = true;
std::string g_buf;

std::string expand(const std::string& pat, int rank) {
  std::string out;
  for (size_t i = 0; i < pat.size(); ++i) {
    if (pat[i] == '%' && i + 1 < pat.size() && (pat[i + 1] == 'p' || pat[i + 1] == 'r')) {
      out += std::to_string(pat[i + 1] == 'p' ? (int)getpid() : rank);
      ++i;
    } else {
      out.push_back(pat[i]);
    }
  }
  return out;
}

void openLocked(const std::string& path, int rank) {
  if (g_file) {
    if (!g_buf.empty()) fwrite(g_buf.data(), 1, g_buf.size(), g_file);
    g_buf.clear();
    fputs("\n]\n", g_file);
    fclose(g_file);
    g_file = nullptr;
  }
  g_rank = rank;
  if (path.empty()) {
    g_state.store(0);
    return;
  }
  g_file = fopen(expand(path, rank).c_str(), "w");
  if (!g_file) {
    g_state.store(0);
    return;
  }
  g_first = true;
  fputs("[\n", g_file);
  char meta[256];
  snprintf(meta, sizeof(meta),
           "{\"name\":\"clock\",\"ph\":\"M\",\"pid\":%d,\"tid\":0,\"args\":{\"wall_epoch_us\":%llu,\"steady_ns\":%llu,\"rank\":%d}}",
           (int)getpid(), (unsigned long long)wallUs(), (unsigned long long)nowNs(), rank);
  g_buf += meta;
  g_first = false;
  g_state.store(1);
}

void emit(const char* text) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_file) return;
  if (!g_first) g_buf += ",\n";
  g_first = false;
  g_buf += text;
  if (g_buf.size() > (1u << 20)) {
    fwrite(g_buf.data(), 1, g_buf.size(), g_file);
    g_buf.clear();
  }
}

struct AtExit {
  ~AtExit() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_file) openLocked("", g_rank);
  }
} g_at_exit;
}  // namespace

bool traceEnabled() {
  int s = g_state.load(std::memory_order_relaxed);
  if (s < 0) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_state.load() < 0) {
      const std::string path = Config::get().trace_file;
      const char* r = getenv("RANK");
      openLocked(path, r ? atoi(r) : 0);
    }
    s = g_state.load();
  }
  return s == 1;
}

void traceOpen(const std::string& path, int rank) {
  std::lock_guard<std::mutex> lk(g_mu);
  openLocked(path, rank);
}

void traceFlush() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_file) {
    if (!g_buf.empty()) fwrite(g_buf.data(), 1, g_buf.size(), g_file);
    g_buf.clear();
    fflush(g_file);
  }
}

void traceComplete(const char* category, const char* name, int lane, uint64_t t0_ns, uint64_t t1_ns, long long bytes) {
  if (!traceEnabled()) return;
  char line[384];
  int k = snprintf(line, sizeof(line), "{\"name\":\"%s\",\"cat\":\"%s\",\"ph\":\"X\",\"pid\":%d,\"tid\":%d,\"ts\":%.3f,\"dur\":%.3f", name,
                   category, (int)getpid(), g_rank * 1000 + lane, (double)t0_ns / 1000.0, (double)(t1_ns - t0_ns) / 1000.0);
  if (bytes >= 0 && k > 0 && k < (int)sizeof(line) - 40) k += snprintf(line + k, sizeof(line) - (size_t)k, ",\"args\":{\"bytes\":%lld}", bytes);
  if (k > 0 && k < (int)sizeof(line) - 2) snprintf(line + k, sizeof(line) - (size_t)k, "}");
  emit(line);
}

void traceInstant(const char* category, const char* name, int lane) {
  if (!traceEnabled()) return;
  char line[320];
  snprintf(line, sizeof(line), "{\"name\":\"%s\",\"cat\":\"%s\",\"ph\":\"i\",\"s\":\"t\",\"pid\":%d,\"tid\":%d,\"ts\":%.3f}", name, category,
           (int)getpid(), g_rank * 1000 + lane, (double)nowNs() / 1000.0);
  emit(line);
}

void traceCounter(const char* name, int lane, double value) {
  if (!traceEnabled()) return;
  char line[320];
  snprintf(line, sizeof(line), "{\"name\":\"%s\",\"ph\":\"C\",\"pid\":%d,\"tid\":%d,\"ts\":%.3f,\"args\":{\"value\":%g}}", name,
           (int)getpid(), g_rank * 1000 + lane, (double)nowNs() / 1000.0, value);
  emit(line);
}

// NVTX: every traced scope is also a named range for Nsight Systems / Nsight Compute. The NVTX v3 header needs
// no library at link time (it finds an attached tool's injection library by itself) and a range costs a few tens
// of nanoseconds when no tool is attached. HYLINK_NVTX=0 switches the ranges off.
bool nvtxEnabled() {
  static const bool on = envBool({"HYLINK_NVTX"}, true);
  // NVTX initialises itself at its first call with a lock-free hand-shake of its own; doing that first call here,
  // under a once-flag every caller passes, gives all threads a proper happens-before edge to the initialised state.
  static std::once_flag once;
  if (on) std::call_once(once, [] { nvtxMarkA("hylink"); });
  return on;
}

TraceScope::TraceScope(const char* category, const char* name, int lane) : cat_(category), name_(name), lane_(lane), t0_(0) {
  if (traceEnabled()) t0_ = nowNs();
  nvtx_ = nvtxEnabled();
  if (nvtx_) nvtxRangePushA(name);
}
TraceScope::~TraceScope() {
  if (nvtx_) nvtxRangePop();
  if (t0_) traceComplete(cat_, name_, lane_, t0_, nowNs(), bytes_);
}
void nvtxMark(const char* name) {
  if (nvtxEnabled()) nvtxMarkA(name);
}

}  // namespace hl

extern "C" {
void hlTraceOpen(const char* path, int rank) { hl::traceOpen(path ? path : "", rank); }
void hlTraceFlush(void) { hl::traceFlush(); }
}
