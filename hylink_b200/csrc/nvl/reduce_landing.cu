// Landing reduce, doorbell and warm-up kernels of the PCIe path (sm_100a).
//
// reduceLanding: dst = scale * op(src_0 .. src_{k-1}) (optionally with dst as
// an extra first operand). 16-byte vector accesses, four packets in flight per
// thread and per source, fp32 accumulation for fp16/bf16 with one rounding,
// up to eight sources reduced in ONE pass so that a batch of landed chunks is
// folded with a single read of each. A source may be pinned host memory: the
// kernel then reads the staging buffer over PCIe itself, fusing the H2D copy
// with the reduction.
//
// Parity: replaces D2DReduceTypedKernel<T>, D2DReduceHalfRawKernel and
// D2DReduceBfloat16RawKernel (pcie-ccl-cuda/kernels/wait_kernel.cu:255-360),
// which are scalar two-address grid-stride loops capped at 1024x256 threads;
// the doorbell replaces the 720 named one-thread spin kernels of
// wait_kernel.cu:13-109 with one kernel whose spin is bounded.
#include <cuda_runtime.h>

#include "nvl/nvl_device.cuh"
#include "nvl/nvl_launch.h"

namespace hl {
namespace dev {

constexpr int kRlThreads = 256;
constexpr int kRlUnroll = 4;

template <typename T>
__global__ void __launch_bounds__(kRlThreads) kReduceLanding(const __grid_constant__ nvl::ReduceLandingArgs a) {
  constexpr int N = Packet<T>::N;
  using Acc = typename Wire<T>::Acc;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
  bool vec = aligned16(a.dst);
  for (int s = 0; s < a.nsrc; ++s) vec = vec && aligned16(a.src[s]);
  const uint64_t np = vec ? a.count / N : 0;  // whole packets handled by the vector loop
  T* dst = reinterpret_cast<T*>(a.dst);
  for (uint64_t i = tid; i < np; i += nthreads * kRlUnroll) {
    Acc acc[kRlUnroll][N];
    bool have[kRlUnroll];
#pragma unroll
    for (int u = 0; u < kRlUnroll; ++u) {
      const uint64_t j = i + (uint64_t)u * nthreads;
      have[u] = j < np;
      if (have[u] && a.accumulate) Packet<T>::unpack(reinterpret_cast<const uint4*>(dst)[j], acc[u]);
    }
    for (int s = 0; s < a.nsrc; ++s) {
      uint4 v[kRlUnroll];
      const uint4* src = reinterpret_cast<const uint4*>(a.src[s]);
#pragma unroll
      for (int u = 0; u < kRlUnroll; ++u) {
        const uint64_t j = i + (uint64_t)u * nthreads;
        if (have[u]) v[u] = src[j];
      }
#pragma unroll
      for (int u = 0; u < kRlUnroll; ++u) {
        if (!have[u]) continue;
        if (s == 0 && !a.accumulate) {
          Packet<T>::unpack(v[u], acc[u]);
        } else {
          Acc b[N];
          Packet<T>::unpack(v[u], b);
#pragma unroll
          for (int e = 0; e < N; ++e) acc[u][e] = applyOp(a.op, acc[u][e], b[e]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kRlUnroll; ++u) {
      const uint64_t j = i + (uint64_t)u * nthreads;
      if (!have[u]) continue;
      finish<T>(acc[u], a.scale, 0);
      reinterpret_cast<uint4*>(dst)[j] = Packet<T>::pack(acc[u]);
    }
  }
  // ragged tail, or everything when some pointer is not 16-byte aligned
  for (uint64_t e = np * N + tid; e < a.count; e += nthreads) {
    Acc acc;
    int first = 0;
    if (a.accumulate) acc = Wire<T>::up(dst[e]);
    else { acc = Wire<T>::up(reinterpret_cast<const T*>(a.src[0])[e]); first = 1; }
    for (int s = first; s < a.nsrc; ++s) acc = applyOp(a.op, acc, Wire<T>::up(reinterpret_cast<const T*>(a.src[s])[e]));
    if constexpr (Wire<T>::kFloat) { if (a.scale != 1.0f) acc = (Acc)(acc * (Acc)a.scale); }
    dst[e] = Wire<T>::down(acc);
  }
}

// Plain device-to-device copy of whole 16-byte packets (the one-rank form of every collective). Eight packets per
// thread in flight; with kStream (HYLINK_COPY_STREAM_HINTS=1) the loads and stores carry the streaming cache hints,
// which keep a one-touch copy from displacing the L2 working set of the kernels around it but cost 5 % of the rate.
constexpr int kCopyThreads = 512;
constexpr int kCopyUnroll = 8;
template <bool kStream>
__global__ void __launch_bounds__(kCopyThreads) kCopyPackets(uint4* __restrict__ dst, const uint4* __restrict__ src, uint64_t packets) {
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = tid; i < packets; i += nthreads * kCopyUnroll) {
    uint4 v[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const uint64_t j = i + (uint64_t)u * nthreads;
      if (j < packets) v[u] = kStream ? __ldcs(src + j) : src[j];
    }
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const uint64_t j = i + (uint64_t)u * nthreads;
      if (j < packets) {
        if (kStream) __stcs(dst + j, v[u]);
        else dst[j] = v[u];
      }
    }
  }
}

__global__ void kWarmup(int* sink) {
  if (sink && threadIdx.x == 0) *sink = 1;
}

// Bounded doorbell: the profile shows `tag` through the launch's NVTX-free
// name argument instead of one symbol per (op, rank, slot).
__global__ void kDoorbell(volatile uint64_t* ready, uint64_t ready_value, volatile uint64_t* complete,
                          uint64_t wait_value, uint64_t timeout_ns, uint64_t* status, const char* tag) {
  (void)tag;
  if (ready) {
    *ready = ready_value;
    __threadfence_system();
  }
  if (!complete) return;
  const uint64_t t0 = globalTimerNs();
  uint32_t spins = 0;
  while (*complete < wait_value) {
    if ((++spins & 15u) == 0) {
      __nanosleep(200);
      if (globalTimerNs() - t0 > timeout_ns) {
        if (status) {
          *reinterpret_cast<volatile uint64_t*>(status) = HL_DEV_TIMEOUT;
          __threadfence_system();
        }
        return;
      }
    }
  }
}

}  // namespace dev

namespace nvl {

static const void* reduceLandingFn(int dt) {
  using namespace dev;
  switch (dt) {
    case hlInt8: return (const void*)kReduceLanding<int8_t>;
    case hlUint8: return (const void*)kReduceLanding<uint8_t>;
    case hlInt32: return (const void*)kReduceLanding<int32_t>;
    case hlUint32: return (const void*)kReduceLanding<uint32_t>;
    case hlInt64: return (const void*)kReduceLanding<long long>;
    case hlUint64: return (const void*)kReduceLanding<unsigned long long>;
    case hlFloat16: return (const void*)kReduceLanding<__half>;
    case hlFloat32: return (const void*)kReduceLanding<float>;
    case hlFloat64: return (const void*)kReduceLanding<double>;
    case hlBfloat16: return (const void*)kReduceLanding<__nv_bfloat16>;
    default: return nullptr;
  }
}

hlResult_t launchReduceLanding(const ReduceLandingArgs& a, int blocks, cudaStream_t stream) {
  const void* fn = reduceLandingFn(a.dtype);
  if (!fn) return fail(hlUnsupported, "reduce landing: unsupported dtype %d", a.dtype);
  if (a.nsrc < 1 || a.nsrc > 8) return fail(hlInvalidArgument, "reduce landing: nsrc %d out of [1,8]", a.nsrc);
  if (a.count == 0) return hlSuccess;
  const size_t es = hlTypeSize((hlDataType_t)a.dtype);
  const uint64_t packets = (a.count * es + 15) / 16;
  if (blocks <= 0) {
    // one packet-quad per thread up to four CTAs per SM of a 148-SM part
    uint64_t want = (packets + (uint64_t)dev::kRlThreads * dev::kRlUnroll - 1) / ((uint64_t)dev::kRlThreads * dev::kRlUnroll);
    blocks = (int)(want < 1 ? 1 : (want > 148 * 4 ? 148 * 4 : want));
  }
  ReduceLandingArgs copy = a;
  void* args[1] = {(void*)&copy};
  cudaError_t e = cudaLaunchKernel(fn, dim3((unsigned)blocks), dim3(dev::kRlThreads), args, 0, stream);
  if (e != cudaSuccess) return fail(hlDeviceError, "reduce landing launch: %s", cudaGetErrorString(e));
  return hlSuccess;
}

// dst and src 16-byte aligned, bytes a multiple of 16 (the caller sends anything else through launchReduceLanding).
hlResult_t launchCopy(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  const uint64_t packets = bytes / 16;
  if (!packets) return hlSuccess;
  static const int forced_blocks = (int)envInt({"HYLINK_COPY_BLOCKS"}, 0);
  static const bool stream_hints = envBool({"HYLINK_COPY_STREAM_HINTS"}, false);
  const uint64_t per_block = (uint64_t)dev::kCopyThreads * dev::kCopyUnroll;
  uint64_t want = (packets + per_block - 1) / per_block;
  // measured on B200 (1 GiB, copy rate): 2.91 TB/s with 4 CTAs per SM and streaming hints, 3.05-3.08 with 8 CTAs per
  // SM or without the hints (cudaMemcpyAsync: 3.21)
  const uint64_t cap = forced_blocks > 0 ? (uint64_t)forced_blocks : 148 * 8;
  const unsigned blocks = (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
  if (stream_hints) dev::kCopyPackets<true><<<blocks, dev::kCopyThreads, 0, stream>>>((uint4*)dst, (const uint4*)src, packets);
  else dev::kCopyPackets<false><<<blocks, dev::kCopyThreads, 0, stream>>>((uint4*)dst, (const uint4*)src, packets);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(hlDeviceError, "copy launch: %s", cudaGetErrorString(e));
  return hlSuccess;
}

hlResult_t prepareReduceLanding() {
  for (int dt = 0; dt < hlNumTypes; ++dt) {
    cudaFuncAttributes at;
    cudaError_t e = cudaFuncGetAttributes(&at, reduceLandingFn(dt));
    if (e != cudaSuccess) return fail(hlDeviceError, "cudaFuncGetAttributes: %s", cudaGetErrorString(e));
  }
  cudaFuncAttributes at;
  cudaFuncGetAttributes(&at, (const void*)dev::kCopyPackets<true>);
  cudaFuncGetAttributes(&at, (const void*)dev::kCopyPackets<false>);
  cudaFuncGetAttributes(&at, (const void*)dev::kDoorbell);
  cudaFuncGetAttributes(&at, (const void*)dev::kWarmup);
  return hlSuccess;
}

hlResult_t launchWarmup(cudaStream_t stream) {
  dev::kWarmup<<<1, 32, 0, stream>>>(nullptr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(hlDeviceError, "warm-up launch: %s", cudaGetErrorString(e));
  return hlSuccess;
}

hlResult_t launchDoorbell(volatile uint64_t* ready, uint64_t ready_value, volatile uint64_t* complete,
                          uint64_t wait_value, uint64_t timeout_ns, uint64_t* status, const char* tag,
                          cudaStream_t stream) {
  dev::kDoorbell<<<1, 1, 0, stream>>>(ready, ready_value, complete, wait_value, timeout_ns, status, tag);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(hlDeviceError, "doorbell launch: %s", cudaGetErrorString(e));
  return hlSuccess;
}

}  // namespace nvl
}  // namespace hl
