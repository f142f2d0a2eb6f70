// Optional interposers of host-blocking CUDA runtime calls (part of
// libhylink_nccl.so, active with HYLINK_CUDA_BLOCK_SHIM=1).
//
// A thread that enters cudaStreamSynchronize / cudaDeviceSynchronize /
// cudaEventSynchronize / a synchronous cudaMemcpy / cudaMemset / a cudaMemcpyAsync that touches
// pageable host memory / cudaMalloc / cudaFree / cudaMallocHost / cudaHostAlloc / cudaFreeHost may
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
std::atomic<unsigned long long> g_drains{0};
struct Guard {
  Guard() {
    if (active() && g_depth++ == 0) {
      hlDrainAllExecutors();
      g_drains.fetch_add(1, std::memory_order_relaxed);
    }
  }
  ~Guard() {
    if (active()) --g_depth;
  }
};
}  // namespace

extern "C" {

// How often a blocking call drained the executors first (0 while the shim is not active).
__attribute__((visibility("default"))) unsigned long long hlBlockShimDrains(void) { return g_drains.load(std::memory_order_relaxed); }

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
__attribute__((visibility("default"))) cudaError_t cudaHostAlloc(void** p, size_t n, unsigned int flags) {
  static auto fn = next<cudaError_t (*)(void**, size_t, unsigned int)>("cudaHostAlloc");
  Guard g;
  return fn ? fn(p, n, flags) : cudaErrorUnknown;
}
__attribute__((visibility("default"))) cudaError_t cudaMemset(void* p, int value, size_t n) {
  static auto fn = next<cudaError_t (*)(void*, int, size_t)>("cudaMemset");
  Guard g;
  return fn ? fn(p, value, n) : cudaErrorUnknown;
}
// An "asynchronous" copy between the device and PAGEABLE host memory blocks the calling thread inside the driver
// (`tensor.item()` and friends end here): it is drained for like the synchronous calls. Copies that involve only
// device or pinned memory return at once and pass straight through.
__attribute__((visibility("default"))) cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t n, cudaMemcpyKind k, cudaStream_t s) {
  static auto fn = next<cudaError_t (*)(void*, const void*, size_t, cudaMemcpyKind, cudaStream_t)>("cudaMemcpyAsync");
  if (!fn) return cudaErrorUnknown;
  if (!active() || k == cudaMemcpyDeviceToDevice) return fn(dst, src, n, k, s);
  const void* host = k == cudaMemcpyDeviceToHost ? dst : (k == cudaMemcpyHostToDevice ? src : nullptr);
  bool pageable = false;
  if (host) {
    cudaPointerAttributes at;
    static auto attr = next<cudaError_t (*)(cudaPointerAttributes*, const void*)>("cudaPointerGetAttributes");
    if (attr && attr(&at, host) == cudaSuccess) pageable = at.type == cudaMemoryTypeUnregistered;
    else pageable = true;
    static auto last = next<cudaError_t (*)(void)>("cudaGetLastError");
    if (last) last();   // an unregistered pointer may leave an error behind on older runtimes
  }
  if (!pageable) return fn(dst, src, n, k, s);
  Guard g;
  return fn(dst, src, n, k, s);
}
__attribute__((visibility("default"))) cudaError_t cudaFreeHost(void* p) {
  static auto fn = next<cudaError_t (*)(void*)>("cudaFreeHost");
  Guard g;
  return fn ? fn(p) : cudaErrorUnknown;
}

}  // extern "C"
