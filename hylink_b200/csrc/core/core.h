// Core utilities shared by every layer: result plumbing, levelled logging,
// typed configuration parsed once from the environment, and clocks.
//
// Parity: the reference scatters these over pcie-ccl-cuda/src/util/log.hpp:69-142,
// util/checks.hpp, core/config.cpp:11-54 and
// multipath-orchestrator/libampccl/common/{config.h:19-394,log.h:22-60}; all of
// it is environment-variable driven. Here one Config object is parsed once and
// keeps the reference's variable names as aliases.
#pragma once
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "hylink/hylink.h"

namespace hl {

// ---------------------------------------------------------------- errors
void setLastError(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
const char* lastError();
hlResult_t fail(hlResult_t r, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define HL_CHECK(expr)                          \
  do {                                          \
    hlResult_t _r = (expr);                     \
    if (_r != hlSuccess) return _r;             \
  } while (0)

// ---------------------------------------------------------------- logging
enum LogLevel { kLogOff = 0, kLogError = 1, kLogWarn = 2, kLogInfo = 3, kLogDebug = 4, kLogTrace = 5 };
int logLevel();
void setLogLevel(int level);
void logLine(int level, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 4, 5)));
// Lines that scripts parse (bandwidth aggregates): printed whatever the level.
void logAlways(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

#define HL_LOG(level, ...)                                              \
  do {                                                                  \
    if ((level) <= ::hl::logLevel()) ::hl::logLine((level), __FILE__, __LINE__, __VA_ARGS__); \
  } while (0)
#define HL_ERR(...) HL_LOG(::hl::kLogError, __VA_ARGS__)
#define HL_WARN(...) HL_LOG(::hl::kLogWarn, __VA_ARGS__)
#define HL_INFO(...) HL_LOG(::hl::kLogInfo, __VA_ARGS__)
#define HL_DBG(...) HL_LOG(::hl::kLogDebug, __VA_ARGS__)

// ---------------------------------------------------------------- clocks
inline uint64_t nowNs() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}
inline uint64_t wallUs() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(
             std::chrono::system_clock::now().time_since_epoch())
      .count();
}
void cpuRelax();

// ---------------------------------------------------------------- env
// First variable of the list that is set wins; the list lets a reference
// spelling (PCCL_*, AMPCCL_*) act as an alias of the native HYLINK_* name.
const char* envFirst(std::initializer_list<const char*> names);
long long envInt(std::initializer_list<const char*> names, long long dflt);
double envDouble(std::initializer_list<const char*> names, double dflt);
bool envBool(std::initializer_list<const char*> names, bool dflt);
std::string envStr(std::initializer_list<const char*> names, const std::string& dflt);
// "64M", "2G", "4096" -> bytes.
long long parseBytes(const char* s, long long dflt);

struct Config {
  // --- PCIe path
  size_t host_buffer_bytes;      // per-NUMA pinned staging pool
  size_t internal_buffer_bytes;  // per-rank device scratch for schedules
  size_t subchunk_slice_bytes;   // 0 = derive from chunk size
  int host_ring_slots;
  size_t small_ir_max_bytes;
  size_t small_msg_threshold_bytes;
  bool small_msg_fastpath;
  int small_msg_timeout_ms;      // bound of a stream-ordered small call before the watchdog releases its flags
  int executor_queue_depth;
  int executor_timeout_ms;
  int barrier_timeout_ms;
  int remote_buffer_timeout_ms;
  bool skip_dma;
  bool warmup_kernel;
  bool disable_stream_mem_ops;
  int d2h_lead_window;
  int h2h_workers;
  int dma_lanes;                 // 0 = table
  std::string ir_path;
  std::string gpu_numa_map;
  bool force_pcie_switch;
  bool force_nvlink;
  bool host_reduce_simd;
  // --- NVLink path
  size_t symm_stage_bytes;       // staging region per direction
  int nvl_timeout_ms;            // bound of every device-side wait
  int nvls;                      // -1 auto, 0 off, 1 require
  std::string symm_mode;         // auto | vmm | ipc
  size_t symm_heap_bytes;        // registered-memory heap per rank (created at the first hlMemAlloc)
  bool zero_copy;                // use the zero-copy kernels when a call's buffers are registered
  bool ipc_close_on_finalize;    // CUDA-IPC fallback: close the peers' mappings at teardown (off: left to process exit)
  size_t oneshot_max_bytes;
  size_t pipe_min_bytes;         // from this size on the pipelined NVLS kernels are used (0 = by rank count)
  size_t push_min_bytes;         // with NVLS available: from this size on the stores-only kernels are used
  int nvls_min_ranks;            // NVLS kernels are preferred from this rank count on
  int nvl_max_blocks;
  // --- orchestrator
  bool orch_enable;
  std::string algo;              // static | tcp | split_ratio
  double static_alpha;
  size_t min_msg_bytes;          // below: NVLink only
  size_t min_msg_bytes_8;        // same, at 8 ranks
  size_t min_chunk_bytes;
  int node_scope_wait_ms;
  bool avg_bw_log;
  int avg_bw_warmup;
  bool fast_only_bw_log;
  bool pcie_child_comms;
  // --- host-side fault injection (tests): "copy_error@K", "stall_ms=V@K", optionally ",rank=R". The K-th
  // transfer this rank's executor issues fails with a device error, or is held back for V milliseconds. Nothing is
  // ever injected on a GPU: the failure is made where the host would have made the call.
  int fault_rank;                // -1 = every rank
  long fault_copy_error_at;      // 0 = off
  long fault_stall_at;           // 0 = off
  int fault_stall_ms;
  // --- diagnostics
  std::string trace_file;
  bool sigdump;
  std::string sigdump_file;
  static const Config& get();
  // Re-reads the environment (tests change it between communicators).
  static void reload();
};

// Size-dependent pipeline slice of the PCIe path: chunk/8 rounded down to a
// power of two inside [512 KiB, 4 MiB]; chunks of 512 MiB and more may grow to
// chunk/64 up to 16 MiB. Same rule as pcie-ccl-cuda/src/ir/ir.hpp:29-54.
size_t subchunkSliceFor(size_t chunk_bytes);

// Arms the SIGUSR1 stack dump when the configuration asks for it (idempotent).
void installSigdump();

}  // namespace hl
