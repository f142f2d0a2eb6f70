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
#include <atomic>

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

// ---- the same copy driven by the bulk-copy engine ---------------------------------------------------------
// One thread per CTA runs a ring of kBulkStages shared-memory tiles: an asynchronous bulk load brings a tile of
// the LOCAL source into shared memory (completion counted in bytes on an mbarrier), an asynchronous bulk store
// sends it on to the destination (this rank's memory or the peer's), and stores are tracked as bulk groups so
// that a tile is only refilled once its store has finished reading it. No register or LSU traffic is involved:
// what is in flight per SM is set by the ring, not by the number of resident warps. Every wait is bounded; when
// one runs out the CTA records HL_DEV_TIMEOUT, drains its own stores and returns.
constexpr int kBulkStages = 8;
constexpr int kBulkLead = 4;   // tiles loaded ahead of the store stream

__device__ __forceinline__ uint32_t smemAddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbarWaitBounded(uint32_t bar, uint32_t parity, uint64_t timeout_ns) {
  uint64_t t0 = 0;
  for (uint32_t spins = 0;; ++spins) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spins & 63u) == 63u) {
      uint64_t now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      if (now - t0 > timeout_ns) return false;
    }
  }
}

__global__ void __launch_bounds__(128) kLinkProbeBulk(const HlCommDev* comms, uint64_t bytes, uint64_t dst_off_bytes, int to_peer,
                                                      int peer, uint32_t tile_bytes) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full[kBulkStages];
  const HlCommDev& c = comms[0];
  const uint8_t* src = c.stage[c.rank];
  uint8_t* dst = (to_peer ? c.stage[peer] : c.stage[c.rank]) + dst_off_bytes;
  if (threadIdx.x != 0) return;
  for (int s = 0; s < kBulkStages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&full[s])) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  const uint64_t ntiles = (bytes + tile_bytes - 1) / tile_bytes;
  // tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  const uint64_t mine = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  bool ok = true;
  for (uint64_t k = 0; k < mine + kBulkLead && ok; ++k) {
    if (k < mine) {
      // stage k % S was last read by the store of tile k - S; at most S - 1 - lead stores were issued after that one
      asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kBulkStages - 1 - kBulkLead) : "memory");
      const int s = (int)(k % kBulkStages);
      const uint64_t off = (blockIdx.x + k * gridDim.x) * (uint64_t)tile_bytes;
      const uint32_t len = (uint32_t)(bytes - off < tile_bytes ? bytes - off : tile_bytes);
      const uint32_t bar = smemAddr(&full[s]);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(len) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       smemAddr(ring + (size_t)s * tile_bytes)),
                   "l"(src + off), "r"(len), "r"(bar)
                   : "memory");
    }
    if (k >= kBulkLead) {
      const uint64_t j = k - kBulkLead;
      const int s = (int)(j % kBulkStages);
      const uint64_t off = (blockIdx.x + j * gridDim.x) * (uint64_t)tile_bytes;
      const uint32_t len = (uint32_t)(bytes - off < tile_bytes ? bytes - off : tile_bytes);
      if (!mbarWaitBounded(smemAddr(&full[s]), (uint32_t)((j / kBulkStages) & 1), c.timeout_ns)) {
        volatile uint64_t* st = c.status;
        st[1] = j;
        st[2] = blockIdx.x;
        st[0] = HL_DEV_TIMEOUT;
        ok = false;
        break;
      }
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + off),
                   "r"(smemAddr(ring + (size_t)s * tile_bytes)), "r"(len)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // this CTA's stores are complete when it exits
}

}  // namespace dev

namespace nvl {

hlResult_t launchLinkProbeBulk(const HlCommDev* dcomm, int to_peer, int blocks, uint32_t tile_bytes, uint64_t bytes, uint64_t dst_off_bytes,
                               int peer, cudaStream_t stream) {
  if (blocks < 1 || blocks > 2048 || tile_bytes < 1024 || tile_bytes > 24576 || tile_bytes % 128 || bytes % 16)
    return fail(hlInvalidArgument, "bulk link probe: tile must be 1 KiB..24 KiB in steps of 128 bytes, size a multiple of 16");
  const size_t smem = (size_t)dev::kBulkStages * tile_bytes;
  static std::atomic<size_t> granted{0};
  if (smem > 48 * 1024 && granted.load() < smem) {
    cudaError_t e = cudaFuncSetAttribute(dev::kLinkProbeBulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));
    if (e != cudaSuccess) return fail(hlDeviceError, "bulk link probe: cannot raise the shared memory limit: %s", cudaGetErrorString(e));
    granted.store(200 * 1024);
  }
  void* args[6] = {(void*)&dcomm, (void*)&bytes, (void*)&dst_off_bytes, (void*)&to_peer, (void*)&peer, (void*)&tile_bytes};
  cudaError_t e = cudaLaunchKernel((const void*)dev::kLinkProbeBulk, dim3((unsigned)blocks), dim3(128), args, smem, stream);
  if (e != cudaSuccess) return fail(hlDeviceError, "bulk link probe launch failed: %s", cudaGetErrorString(e));
  return hlSuccess;
}

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
