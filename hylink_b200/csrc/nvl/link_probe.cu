// Link probe: a bare copy kernel between this rank's symmetric staging and a
// peer's, with the launch shape, the unroll depth, the direction and the
// address layout as run-time choices. It answers the sizing questions of the
// collective kernels by measurement: how many CTAs and warps it takes to fill
// a link with posted stores, what a remote load costs, and what the same loop
// reaches inside local HBM.
//
// The kernel waits on nothing (no flags, no barriers): both ranks may run it at
// once, and the caller orders it against other work with the stream.
// There is no counterpart in the reference, which measures its links with
// host-side copy-engine tests only (pcie-ccl-cuda/tests/dev/test_gpu_dma_single.cpp).
#include "nvl/nvl_launch.h"

namespace hl {
namespace dev {

enum { kProbePush = 0, kProbePull = 1, kProbeLocal = 2, kProbeStoreOnly = 3, kProbeLoadOnly = 4 };

template <int U, int MAXT>
__global__ void __launch_bounds__(MAXT) kLinkProbe(const HlCommDev* comms, uint64_t packets, uint64_t dst_off, int mode, int peer,
                                                   int layout) {
  const HlCommDev& c = comms[0];
  const uint4* lsrc = reinterpret_cast<const uint4*>(c.stage[c.rank]);
  uint4* ldst = reinterpret_cast<uint4*>(c.stage[c.rank]) + dst_off;
  const uint4* rsrc = reinterpret_cast<const uint4*>(c.stage[peer]);
  uint4* rdst = reinterpret_cast<uint4*>(c.stage[peer]) + dst_off;
  const uint4* src = (mode == kProbePull || mode == kProbeLoadOnly) ? rsrc : lsrc;
  uint4* dst = (mode == kProbePush || mode == kProbeStoreOnly) ? rdst : ldst;
  // layout 0: the grid sweeps the buffer together (consecutive packets of a thread are a whole grid apart);
  // layout 1: every CTA owns one contiguous range and sweeps it alone.
  uint64_t first, stride, end;
  if (layout == 0) {
    first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    stride = (uint64_t)gridDim.x * blockDim.x;
    end = packets;
  } else {
    const uint64_t per = (packets + gridDim.x - 1) / gridDim.x;
    first = (uint64_t)blockIdx.x * per + threadIdx.x;
    stride = blockDim.x;
    end = first - threadIdx.x + per < packets ? first - threadIdx.x + per : packets;
  }
  uint4 acc = make_uint4(threadIdx.x, blockIdx.x, 3u, 4u);
  for (uint64_t i = first; i < end; i += stride * U) {
    uint4 v[U];
    if (mode != kProbeStoreOnly) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t j = i + (uint64_t)u * stride;
        if (j < end) v[u] = src[j];
      }
    }
    if (mode == kProbeLoadOnly) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t j = i + (uint64_t)u * stride;
        if (j < end) {
          acc.x ^= v[u].x;
          acc.y += v[u].y;
          acc.z ^= v[u].z;
          acc.w += v[u].w;
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t j = i + (uint64_t)u * stride;
        if (j < end) dst[j] = mode == kProbeStoreOnly ? acc : v[u];
      }
    }
  }
  // keeps the loads of the load-only mode alive; the branch is practically never taken
  if (mode == kProbeLoadOnly && acc.x == 0x9e3779b9u && acc.y == 0x7f4a7c15u) ldst[first < packets ? first : 0] = acc;
}

}  // namespace dev

namespace nvl {

hlResult_t launchLinkProbe(const HlCommDev* dcomm, int mode, int blocks, int threads, int unroll, int layout, uint64_t packets,
                           uint64_t dst_off, int peer, cudaStream_t stream) {
  if (mode < 0 || mode > 4 || blocks < 1 || blocks > 2048 || threads < 32 || threads > 1024 || threads % 32 || layout < 0 || layout > 1)
    return fail(hlInvalidArgument, "link probe: bad launch shape");
  const void* fn = nullptr;
  const bool big = threads > 512;
  switch (unroll) {
    case 2: fn = big ? (const void*)dev::kLinkProbe<2, 1024> : (const void*)dev::kLinkProbe<2, 512>; break;
    case 4: fn = big ? (const void*)dev::kLinkProbe<4, 1024> : (const void*)dev::kLinkProbe<4, 512>; break;
    case 8: fn = big ? (const void*)dev::kLinkProbe<8, 1024> : (const void*)dev::kLinkProbe<8, 512>; break;
    case 16: fn = big ? nullptr : (const void*)dev::kLinkProbe<16, 512>; break;
    default: break;
  }
  if (!fn) return fail(hlInvalidArgument, "link probe: unroll must be 2, 4, 8 (or 16 with at most 512 threads)");
  void* args[6] = {(void*)&dcomm, (void*)&packets, (void*)&dst_off, (void*)&mode, (void*)&peer, (void*)&layout};
  cudaError_t e = cudaLaunchKernel(fn, dim3((unsigned)blocks), dim3((unsigned)threads), args, 0, stream);
  if (e != cudaSuccess) return fail(hlDeviceError, "link probe launch failed: %s", cudaGetErrorString(e));
  return hlSuccess;
}

}  // namespace nvl
}  // namespace hl
