// Chrome-trace ("chrome://tracing", Perfetto) event writer.
//
// Enabled at run time by HYLINK_TRACE_FILE (alias PCCL_TRACE_FILE); "%p" and
// "%r" in the name expand to the process id and the rank. Events are buffered
// per thread and appended to the file under a lock when a shard fills up or
// the process exits. Thread ids are deterministic (rank * 1000 + lane) so that
// traces of several runs line up, and a metadata record carries the wall-clock
// epoch of the monotonic timestamps for cross-process alignment.
//
// Parity: pcie-ccl-cuda/src/util/trace_writer.hpp:136-351,353-450,546-549
// (compile-time PCCL_TRACE there; a run-time switch here).
#pragma once
#include <cstdint>
#include <string>

namespace hl {

bool traceEnabled();
// Complete event ("ph":"X") from t0 to t1 (steady-clock nanoseconds).
// `bytes` (when >= 0) is recorded as the event's payload size, for per-size statistics.
void traceComplete(const char* category, const char* name, int lane, uint64_t t0_ns, uint64_t t1_ns, long long bytes = -1);
void traceInstant(const char* category, const char* name, int lane);
void traceCounter(const char* name, int lane, double value);
void traceFlush();
// Redirects tracing to `path` ("" switches it off); used by tests.
void traceOpen(const std::string& path, int rank);

// Named NVTX ranges (Nsight tools): on unless HYLINK_NVTX=0; every TraceScope is one.
bool nvtxEnabled();
void nvtxMark(const char* name);

class TraceScope {
 public:
  TraceScope(const char* category, const char* name, int lane);
  ~TraceScope();
  void setBytes(long long b) { bytes_ = b; }

 private:
  const char* cat_;
  const char* name_;
  int lane_;
  uint64_t t0_;
  bool nvtx_ = false;
  long long bytes_ = -1;
};

}  // namespace hl
