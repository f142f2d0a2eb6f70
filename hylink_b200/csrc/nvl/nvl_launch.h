// Host-side launch interface of the NVLink-path kernels and of the landing
// reduce kernel (the only parts of the library compiled by nvcc).
#pragma once
#include <cuda_runtime.h>

#include "core/core.h"
#include "nvl/nvl_types.h"

namespace hl {
namespace nvl {

// nranks picks the variant of the kernels that are compiled per rank-count class (<= 2, <= 4, <= 8).
const void* kernelFor(int kind, int wire_dt, int nranks = HL_MAX_RANKS);
const char* kernelName(int kind);
// The barrier-free small-message kernels live in a file of their own (nvl_ll_kernels.cu).
const void* lowLatencyKernelFor(int kind, int wire_dt);
// emu_ranks > 1: cooperative launch with one grid row per emulated rank.
hlResult_t launch(int kind, int wire_dt, const HlCommDev* dcomms, const HlEmuCalls& calls, int emu_ranks, int blocks,
                  cudaStream_t stream, int nranks = HL_MAX_RANKS);
hlResult_t prepareKernels();
// Bare copy between this rank's staging and `peer`'s (see link_probe.cu); mode 0 push, 1 pull, 2 local, 3 stores
// only, 4 loads only; `packets` 16-byte packets from offset 0 to offset dst_off.
hlResult_t launchLinkProbe(const HlCommDev* dcomm, int mode, int blocks, int threads, int unroll, int layout, uint64_t packets,
                           uint64_t dst_off, int peer, cudaStream_t stream);

// dst[i] = scale * op(src_0[i], ..., src_{k-1}[i]) with fp32 accumulation for
// 16-bit floats; when `accumulate` is set dst itself is the first operand.
// Sources may live in pinned host memory (zero-copy read over PCIe).
struct ReduceLandingArgs {
  void* dst;
  const void* src[8];
  int nsrc;
  int accumulate;
  uint64_t count;
  int dtype;      // element type of dst and of every source
  int op;
  float scale;
};
// The same copy through the bulk-copy engine: one thread per CTA, a ring of shared-memory tiles of `tile_bytes`.
hlResult_t launchLinkProbeBulk(const HlCommDev* dcomm, int to_peer, int blocks, uint32_t tile_bytes, uint64_t bytes, uint64_t dst_off_bytes,
                               int peer, cudaStream_t stream);
hlResult_t launchReduceLanding(const ReduceLandingArgs& a, int blocks, cudaStream_t stream);
// Device-to-device copy of whole 16-byte packets between 16-byte aligned buffers (streaming cache hints).
hlResult_t launchCopy(void* dst, const void* src, size_t bytes, cudaStream_t stream);
hlResult_t prepareReduceLanding();

// Context warm-up (one trivial kernel): a context whose first work is pure
// copy-engine traffic may stall (pcie-ccl-cuda/src/api/pccl_api.cpp:720-746).
hlResult_t launchWarmup(cudaStream_t stream);

// Doorbell fallback for drivers without stream memory operations: writes
// `ready_value` to a host-mapped word, then waits (bounded) until
// *complete >= wait_value. On expiry it writes HL_DEV_TIMEOUT to *status.
hlResult_t launchDoorbell(volatile uint64_t* ready, uint64_t ready_value, volatile uint64_t* complete,
                          uint64_t wait_value, uint64_t timeout_ns, uint64_t* status, const char* tag,
                          cudaStream_t stream);

}  // namespace nvl
}  // namespace hl
