// Optional interposers of host-blocking CUDA runtime calls (part of
// libhylink_nccl.so, active with HYLINK_CUDA_BLOCK_SHIM=1).
//
// A thread that enters cudaStreamSynchronize / cudaDeviceSynchronize /
// cudaEventSynchronize / a synchronous cudaMemcpy / cudaMalloc / cudaFree may
// hold driver locks while it waits for a stream that is itself parked behind
// one of this library's doorbells; the CPU executor that would ring the
// doorbell needs the driver to issue its copies. Draining the executors before
// entering the blocking call removes the cycle.
//
// Parity: pcie-ccl-cuda/src/api/nccl_compat/cuda_block_shim.cpp:68-195 and
// src/util/inflight_drain.cpp; the reference interposes unconditionally, this
// build keeps it opt-in because the executor here never needs the driver to
// RELEASE a doorbell (a plain CPU store does that), which makes the cycle much
// rarer.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <atomic>

#include "core/core.h"

extern "C" void hlDrainAllExecutors(void);

namespace {
bool active() {
  static const bool on = hl::envBool({"HYLINK_CUDA_BLOCK_SHIM"}, false);
  return on;
}
template <typename F> F next(const char* name) {
  return reinterpret_cast<F>(dlsym(RTLD_NEXT, name));
}
thread_local int g_depth = 0;
struct Guard {
  Guard() {
    if (active() && g_depth++ == 0) hlDrainAllExecutors();
  }
  ~Guard() {
    if (active()) --g_depth;
  }
};
}  // namespace

extern "C" {

__attribute__((visibility("default"))) cudaError_t cudaStreamSynchronize(cudaStream_t s) {
  static auto fn = next<cudaError_t (*)(cudaStream_t)>("cudaStreamSynchronize");
  Guard g;
  return fn ? fn(s) : cudaErrorUnknown;
}
__attribute__((visibility("default"))) cudaError_t cudaDeviceSynchronize(void) {
  static auto fn = next<cudaError_t (*)(void)>("cudaDeviceSynchronize");
  Guard g;
  return fn ? fn() : cudaErrorUnknown;
}
__attribute__((visibility("default"))) cudaError_t cudaEventSynchronize(cudaEvent_t e) {
  static auto fn = next<cudaError_t (*)(cudaEvent_t)>("cudaEventSynchronize");
  Guard g;
  return fn ? fn(e) : cudaErrorUnknown;
}
__attribute__((visibility("default"))) cudaError_t cudaMemcpy(void* dst, const void* src, size_t n, cudaMemcpyKind k) {
  static auto fn = next<cudaError_t (*)(void*, const void*, size_t, cudaMemcpyKind)>("cudaMemcpy");
  Guard g;
  return fn ? fn(dst, src, n, k) : cudaErrorUnknown;
}
__attribute__((visibility("default"))) cudaError_t cudaMalloc(void** p, size_t n) {
  static auto fn = next<cudaError_t (*)(void**, size_t)>("cudaMalloc");
  Guard g;
  return fn ? fn(p, n) : cudaErrorUnknown;
}
__attribute__((visibility("default"))) cudaError_t cudaFree(void* p) {
  static auto fn = next<cudaError_t (*)(void*)>("cudaFree");
  Guard g;
  return fn ? fn(p) : cudaErrorUnknown;
}
__attribute__((visibility("default"))) cudaError_t cudaMallocHost(void** p, size_t n) {
  static auto fn = next<cudaError_t (*)(void**, size_t)>("cudaMallocHost");
  Guard g;
  return fn ? fn(p, n) : cudaErrorUnknown;
}
__attribute__((visibility("default"))) cudaError_t cudaFreeHost(void* p) {
  static auto fn = next<cudaError_t (*)(void*)>("cudaFreeHost");
  Guard g;
  return fn ? fn(p) : cudaErrorUnknown;
}

}  // extern "C"
