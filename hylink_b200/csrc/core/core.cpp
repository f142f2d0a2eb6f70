#include "core/core.h"

#include <sys/syscall.h>
#include <unistd.h>

#include <cstring>
#include <mutex>

namespace hl {

static thread_local char g_last_error[1024] = {0};

void setLastError(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}
const char* lastError() { return g_last_error; }

hlResult_t fail(hlResult_t r, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  HL_ERR("%s: %s", hlGetErrorString(r), g_last_error);
  return r;
}

static std::atomic<int> g_log_level{-1};

static int parseLevel(const char* s) {
  if (!s || !*s) return kLogWarn;
  if (s[0] >= '0' && s[0] <= '9') return atoi(s);
  std::string v(s);
  for (auto& c : v) c = (char)toupper(c);
  if (v == "OFF" || v == "NONE") return kLogOff;
  if (v == "ERROR") return kLogError;
  if (v == "WARN" || v == "WARNING") return kLogWarn;
  if (v == "INFO") return kLogInfo;
  if (v == "DEBUG") return kLogDebug;
  if (v == "TRACE") return kLogTrace;
  return kLogWarn;
}

int logLevel() {
  int l = g_log_level.load(std::memory_order_relaxed);
  if (l < 0) {
    l = parseLevel(envFirst({"HYLINK_LOG_LEVEL", "AMPCCL_LOG_LEVEL", "PCCL_LOG_LEVEL"}));
    g_log_level.store(l, std::memory_order_relaxed);
  }
  return l;
}
void setLogLevel(int level) { g_log_level.store(level, std::memory_order_relaxed); }

static bool useColour() {
  static int c = -1;
  if (c < 0) {
    const char* force = envFirst({"HYLINK_LOG_COLOR", "AMPCCL_LOG_COLOR"});   // 0 / 1 overrides the terminal test
    if (force) c = (force[0] == '1' || force[0] == 'y' || force[0] == 'Y' || force[0] == 't' || force[0] == 'T') ? 1 : 0;
    else c = (getenv("NO_COLOR") == nullptr && isatty(2)) ? 1 : 0;
  }
  return c == 1;
}

void logLine(int level, const char* file, int line, const char* fmt, ...) {
  static const char* names[] = {"OFF", "ERROR", "WARN", "INFO", "DEBUG", "TRACE"};
  static const char* colours[] = {"", "\033[31m", "\033[33m", "\033[32m", "\033[36m", "\033[90m"};
  char body[1536];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(body, sizeof(body), fmt, ap);
  va_end(ap);
  const char* base = strrchr(file, '/');
  base = base ? base + 1 : file;
  uint64_t us = wallUs();
  int lv = level < 0 ? 0 : (level > 5 ? 5 : level);
  long tid = (long)syscall(SYS_gettid);
  if (useColour())
    fprintf(stderr, "%s[HYLINK][%s] %llu.%06llu %d/%ld %s:%d %s\033[0m\n", colours[lv], names[lv],
            (unsigned long long)(us / 1000000), (unsigned long long)(us % 1000000), (int)getpid(),
            tid, base, line, body);
  else
    fprintf(stderr, "[HYLINK][%s] %llu.%06llu %d/%ld %s:%d %s\n", names[lv],
            (unsigned long long)(us / 1000000), (unsigned long long)(us % 1000000), (int)getpid(),
            tid, base, line, body);
}

void logAlways(const char* fmt, ...) {
  char body[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(body, sizeof(body), fmt, ap);
  va_end(ap);
  // Prefix kept compatible with the log scrapers of the reference's sweep
  // scripts (multipath-orchestrator/tests/nccl_test/test_scripts).
  fprintf(stderr, "[AMPCCL][OFF] %s\n", body);
}

void cpuRelax() {
#if defined(__x86_64__)
  __builtin_ia32_pause();
#elif defined(__aarch64__)
  asm volatile("yield");
#endif
}

const char* envFirst(std::initializer_list<const char*> names) {
  for (const char* n : names) {
    const char* v = getenv(n);
    if (v && *v) return v;
  }
  return nullptr;
}
long long envInt(std::initializer_list<const char*> names, long long dflt) {
  const char* v = envFirst(names);
  if (!v) return dflt;
  return parseBytes(v, dflt);
}
double envDouble(std::initializer_list<const char*> names, double dflt) {
  const char* v = envFirst(names);
  if (!v) return dflt;
  char* end = nullptr;
  double d = strtod(v, &end);
  return end == v ? dflt : d;
}
bool envBool(std::initializer_list<const char*> names, bool dflt) {
  const char* v = envFirst(names);
  if (!v) return dflt;
  char c = v[0];
  if (c == '1' || c == 'y' || c == 'Y' || c == 't' || c == 'T') return true;
  if (c == 'o' || c == 'O') return (v[1] == 'n' || v[1] == 'N');
  return false;
}
std::string envStr(std::initializer_list<const char*> names, const std::string& dflt) {
  const char* v = envFirst(names);
  return v ? std::string(v) : dflt;
}
long long parseBytes(const char* s, long long dflt) {
  if (!s || !*s) return dflt;
  char* end = nullptr;
  double d = strtod(s, &end);
  if (end == s) return dflt;
  long long mul = 1;
  switch (*end) {
    case 'k': case 'K': mul = 1LL << 10; break;
    case 'm': case 'M': mul = 1LL << 20; break;
    case 'g': case 'G': mul = 1LL << 30; break;
    default: break;
  }
  return (long long)(d * (double)mul);
}

static std::mutex g_cfg_mu;
static Config* g_cfg = nullptr;

static Config* loadConfig() {
  Config* c = new Config();
  c->host_buffer_bytes = (size_t)envInt({"HYLINK_HOST_BUFFER_SIZE", "PCCL_HOST_BUFFER_SIZE"}, 512LL << 20);
  c->internal_buffer_bytes = (size_t)envInt({"HYLINK_INTERNAL_BUFFER_BYTES", "PCCL_INTERNAL_BUFFER_BYTES"}, 256LL << 20);
  c->subchunk_slice_bytes = (size_t)envInt({"HYLINK_SUBCHUNK_SLICE_SIZE", "PCCL_SUBCHUNK_SLICE_SIZE"}, 0);
  if (c->subchunk_slice_bytes && c->subchunk_slice_bytes < 4096) c->subchunk_slice_bytes = 0;
  c->host_ring_slots = (int)envInt({"HYLINK_HOST_RING_SLOTS", "PCCL_HOST_RING_SLOTS"}, 3);
  c->small_ir_max_bytes = (size_t)envInt({"HYLINK_SMALL_IR_MAX_BYTES", "PCCL_SMALL_IR_MAX_BYTES"}, 4LL << 20);
  c->small_msg_threshold_bytes = (size_t)envInt({"HYLINK_SMALL_MSG_THRESHOLD_BYTES", "PCCL_SMALL_MSG_THRESHOLD_BYTES"}, 1LL << 20);
  c->small_msg_fastpath = envBool({"HYLINK_SMALL_MSG_FASTPATH", "PCCL_SMALL_MSG_FASTPATH"}, true);
  c->small_msg_timeout_ms = (int)envInt({"HYLINK_SMALL_MSG_FASTPATH_TIMEOUT_MS", "PCCL_SMALL_MSG_FASTPATH_TIMEOUT_MS"}, 0);   // 0: the executor's
  c->executor_queue_depth = (int)envInt({"HYLINK_EXECUTOR_QUEUE_DEPTH", "PCCL_EXECUTOR_QUEUE_DEPTH"}, 64);
  c->executor_timeout_ms = (int)envInt({"HYLINK_EXECUTOR_TIMEOUT_MS", "PCCL_EXECUTOR_TIMEOUT_MS"}, 60000);
  c->barrier_timeout_ms = (int)envInt({"HYLINK_BARRIER_TIMEOUT_MS", "PCCL_BARRIER_TIMEOUT_MS"}, 120000);
  c->remote_buffer_timeout_ms = (int)envInt({"HYLINK_REMOTE_BUFFER_TIMEOUT_MS", "PCCL_REMOTE_BUFFER_TIMEOUT_MS"}, 30000);
  c->skip_dma = envBool({"HYLINK_SKIP_DMA", "PCCL_SKIP_DMA"}, false);
  c->warmup_kernel = envBool({"HYLINK_WARMUP_KERNEL", "PCCL_WARMUP_KERNEL"}, true);
  c->disable_stream_mem_ops = envBool({"HYLINK_DISABLE_STREAM_MEM_OPS", "PCCL_DISABLE_STREAM_MEM_OPS"}, false);
  c->d2h_lead_window = (int)envInt({"HYLINK_D2H_LEAD_WINDOW"}, 4);
  c->h2h_workers = (int)envInt({"HYLINK_H2H_WORKERS"}, 0);
  c->dma_lanes = (int)envInt({"HYLINK_DMA_LANES", "PCCL_FORCE_DMA_LANES"}, 0);
  c->ir_path = envStr({"HYLINK_IR_PATH", "PCCL_IR_PATH", "PCCL_IR_DIR"}, "");
  c->gpu_numa_map = envStr({"HYLINK_GPU_NUMA_MAP", "PCCL_GPU_NUMA_MAP"}, "");
  c->force_pcie_switch = envBool({"HYLINK_FORCE_PCIE_SWITCH", "PCCL_FORCE_PCIE_SWITCH"}, false);
  c->force_nvlink = envBool({"HYLINK_FORCE_NVLINK", "PCCL_FORCE_NVLINK"}, false);
  c->host_reduce_simd = envBool({"HYLINK_HOST_REDUCE_SIMD"}, true);

  c->symm_stage_bytes = (size_t)envInt({"HYLINK_SYMM_STAGE_BYTES"}, 1LL << 30);
  c->nvl_timeout_ms = (int)envInt({"HYLINK_NVL_TIMEOUT_MS"}, 20000);
  c->nvls = (int)envInt({"HYLINK_NVLS"}, -1);
  c->symm_mode = envStr({"HYLINK_SYMM_MODE"}, "auto");
  c->symm_heap_bytes = (size_t)envInt({"HYLINK_SYMM_HEAP_BYTES"}, 8LL << 30);
  c->zero_copy = envBool({"HYLINK_ZERO_COPY"}, true);
  // the reference's switches for peers reading user buffers in place (its CUDA-IPC buffer registry)
  if (envBool({"PCCL_DISABLE_DEVICE_IPC"}, false)) c->zero_copy = false;
  if (envBool({"PCCL_FORCE_DEVICE_IPC"}, false)) c->zero_copy = true;
  c->ipc_close_on_finalize = envBool({"HYLINK_CUDA_IPC_CLOSE_ON_FINALIZE", "PCCL_CUDA_IPC_CLOSE_ON_FINALIZE"}, true);
  // Settings of the reference that have nothing to switch here: say so once instead of ignoring them silently.
  static const struct { const char* name; const char* why; } kNoEffect[] = {
      {"PCCL_NRANKS", "the rank count comes from the communicator"},
      {"PCCL_BOOTSTRAP_ADDR", "single node only: the control plane is shared memory"},
      {"PCCL_D2D_PUSH", "peer copies between GPUs ride the NVLink kernels"},
      {"PCCL_D2D_INPUT_FIRST", "peer copies between GPUs ride the NVLink kernels"},
      {"PCCL_NCCL_COMPAT_MODE", "threads and processes use the same rendezvous; nothing to detect"},
      {"PCCL_HOST_POOL_SHM", "shared host pools are always memfd-backed and registered"},
      {"PCCL_COLD_START_DRAIN", "the context is warmed up by a kernel at communicator creation"},
      {"AMPCCL_PCCL_UNIQUE_ID", "both paths share one communicator and one id"},
      {"AMPCCL_PCCL_FORCE_ZERO_UNIQUE_ID", "both paths share one communicator and one id"},
  };
  for (const auto& e : kNoEffect)
    if (const char* v = getenv(e.name)) HL_INFO("%s=%s is accepted and has no effect here: %s", e.name, v, e.why);
  c->oneshot_max_bytes = (size_t)envInt({"HYLINK_ONESHOT_MAX_BYTES"}, 128LL << 10);
  c->pipe_min_bytes = (size_t)envInt({"HYLINK_PIPE_MIN_BYTES"}, 0);
  c->push_min_bytes = (size_t)envInt({"HYLINK_PUSH_MIN_BYTES"}, 32LL << 20);
  c->nvls_min_ranks = (int)envInt({"HYLINK_NVLS_MIN_RANKS"}, 4);
  c->nvl_max_blocks = (int)envInt({"HYLINK_NVL_MAX_BLOCKS"}, 0);

  c->orch_enable = envBool({"HYLINK_ORCH_ENABLE", "AMPCCL_ENABLE"}, false);
  c->algo = envStr({"HYLINK_ALGO", "AMPCCL_ALGO"}, "split_ratio");
  c->static_alpha = envDouble({"HYLINK_STATIC_ALPHA", "AMPCCL_STATIC_ALPHA"}, 0.05);
  c->min_msg_bytes = (size_t)envInt({"HYLINK_MIN_MSG_SIZE", "AMPCCL_MIN_MSG_SIZE"}, 256LL << 20);
  c->min_msg_bytes_8 = (size_t)envInt({"HYLINK_MIN_MSG_SIZE_8", "AMPCCL_MIN_MSG_SIZE_8RANKS"}, 1LL << 30);
  c->min_chunk_bytes = (size_t)envInt({"HYLINK_MIN_CHUNK_SIZE", "AMPCCL_MIN_CHUNK_SIZE"}, 4096);
  c->node_scope_wait_ms = (int)envInt({"HYLINK_NODE_SCOPE_WAIT_MS", "AMPCCL_NODE_SCOPE_WAIT_MS"}, 200);
  c->avg_bw_log = envBool({"HYLINK_AVG_BW_LOG", "AMPCCL_AVG_BW_LOG"}, false);
  c->avg_bw_warmup = (int)envInt({"HYLINK_AVG_BW_LOG_WARMUP", "AMPCCL_AVG_BW_LOG_WARMUP"}, 5);
  c->fast_only_bw_log = envBool({"HYLINK_FAST_ONLY_BW_LOG", "AMPCCL_FAST_ONLY_BW_LOG"}, false);
  c->pcie_child_comms = envBool({"HYLINK_PCIE_CHILD_COMMS", "AMPCCL_PCIE_CHILD_COMMS"}, false);

  c->fault_rank = -1;
  c->fault_copy_error_at = c->fault_stall_at = 0;
  c->fault_stall_ms = 0;
  {
    const std::string spec = envStr({"HYLINK_FAULT_INJECT"}, "");
    size_t pos = 0;
    while (pos < spec.size()) {
      size_t end = spec.find(',', pos);
      if (end == std::string::npos) end = spec.size();
      const std::string item = spec.substr(pos, end - pos);
      pos = end + 1;
      const size_t at = item.find('@');
      const long k = at == std::string::npos ? 1 : atol(item.c_str() + at + 1);
      if (item.compare(0, 10, "copy_error") == 0) c->fault_copy_error_at = k > 0 ? k : 1;
      else if (item.compare(0, 9, "stall_ms=") == 0) {
        c->fault_stall_ms = atoi(item.c_str() + 9);
        c->fault_stall_at = k > 0 ? k : 1;
      } else if (item.compare(0, 5, "rank=") == 0) c->fault_rank = atoi(item.c_str() + 5);
      else if (!item.empty()) fprintf(stderr, "[hylink] HYLINK_FAULT_INJECT: unknown item '%s' ignored\n", item.c_str());
    }
  }

  c->trace_file = envStr({"HYLINK_TRACE_FILE", "PCCL_TRACE_FILE"}, "");
  c->sigdump = envBool({"HYLINK_SIGDUMP", "PCCL_SIGDUMP"}, false);
  c->sigdump_file = envStr({"HYLINK_SIGDUMP_FILE", "PCCL_SIGDUMP_FILE"}, "");
  return c;
}

const Config& Config::get() {
  std::lock_guard<std::mutex> lk(g_cfg_mu);
  if (!g_cfg) g_cfg = loadConfig();
  return *g_cfg;
}
void Config::reload() {
  std::lock_guard<std::mutex> lk(g_cfg_mu);
  // The previous object is leaked on purpose: readers may still hold a reference.
  g_cfg = loadConfig();
  g_log_level.store(-1);
}

size_t subchunkSliceFor(size_t chunk_bytes) {
  size_t forced = Config::get().subchunk_slice_bytes;
  if (forced) return forced;
  const size_t lo = (size_t)512 << 10, hi = (size_t)4 << 20, big_hi = (size_t)16 << 20;
  size_t s = lo;
  while (s * 2 <= chunk_bytes / 8 && s * 2 <= hi) s *= 2;
  if (chunk_bytes >= ((size_t)512 << 20))
    while (s * 2 <= chunk_bytes / 64 && s * 2 <= big_hi) s *= 2;
  return s;
}

}  // namespace hl

extern "C" {

size_t hlTypeSize(hlDataType_t t) {
  switch (t) {
    case hlInt8: case hlUint8: return 1;
    case hlFloat16: case hlBfloat16: return 2;
    case hlInt32: case hlUint32: case hlFloat32: return 4;
    case hlInt64: case hlUint64: case hlFloat64: return 8;
    default: return 0;
  }
}

const char* hlGetErrorString(hlResult_t r) {
  switch (r) {
    case hlSuccess: return "success";
    case hlInvalidArgument: return "invalid argument";
    case hlSystemError: return "system error";
    case hlInternalError: return "internal error";
    case hlDeviceError: return "device error";
    case hlNetworkError: return "network error";
    case hlTimeout: return "timeout";
    case hlUnsupported: return "unsupported";
    case hlRemoteError: return "remote rank error";
    default: return "unknown result";
  }
}

const char* hlGetLastError(void) { return hl::lastError(); }
int hlVersion(void) { return 100; }

}  // extern "C"

// Re-reads every environment variable (tests flip settings between communicators).
extern "C" void hlConfigReload(void) { hl::Config::reload(); }

// A few settings by name, as the library resolved them from the environment (-1: unknown name). For tests and for
// "which value did my variable end up as" questions.
extern "C" long long hlConfigValue(const char* name) {
  const hl::Config& c = hl::Config::get();
  const std::string k = name ? name : "";
  if (k == "zero_copy") return c.zero_copy ? 1 : 0;
  if (k == "ipc_close_on_finalize") return c.ipc_close_on_finalize ? 1 : 0;
  if (k == "small_msg_timeout_ms") return c.small_msg_timeout_ms;
  if (k == "small_msg_threshold_bytes") return (long long)c.small_msg_threshold_bytes;
  if (k == "executor_timeout_ms") return c.executor_timeout_ms;
  if (k == "barrier_timeout_ms") return c.barrier_timeout_ms;
  if (k == "host_buffer_bytes") return (long long)c.host_buffer_bytes;
  if (k == "internal_buffer_bytes") return (long long)c.internal_buffer_bytes;
  if (k == "orch_enable") return c.orch_enable ? 1 : 0;
  if (k == "min_msg_bytes") return (long long)c.min_msg_bytes;
  return -1;
}
