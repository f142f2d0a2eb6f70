// sm_100a kernels of the dedicated-link path: all-reduce (one-shot, two-shot
// P2P, NVLS), reduce-scatter, all-gather, broadcast, all-to-all and barrier.
//
// Every kernel fuses, in one launch: the (converting) copy of the caller's
// buffer into peer-mapped symmetric staging, the cross-GPU flag exchange, the
// transfer itself (16-byte loads from peer memory issued by each CTA, or
// multimem.ld_reduce / multimem.st through NVSwitch), the reduction with fp32
// accumulation, the scale, and the converting store into the caller's output.
// Segment strides and a handled-prefix length are native arguments, so the
// orchestrator's "NVLink takes the first k elements of every segment" split
// needs no pack or merge copies.
//
// Protocol rules that make staging reuse safe without extra round trips:
//   A. EVERY kernel ends with a cross-GPU barrier that follows its last access
//      to any staging region, its own included (a kernel that finishes by
//      copying landed data out of its own staging is not exempt: a faster peer
//      would otherwise start the next call and push into slots that are still
//      being read);
//   B. launches of one communicator are stream-ordered on every rank, and all
//      ranks launch the same grid for the same call.
// With these, when any rank starts call k+1, all of its CTAs have left call k,
// so CTA b of every peer has arrived at call k's last barrier, for every b:
// no rank still reads or writes any staging of call k. A kernel of call k+1
// may therefore write into a peer's staging right at entry (the stores-only
// kernels do), and may stage locally before its first barrier.
//
// Block b of a rank only ever consumes data produced by block b of a peer
// (same in-segment packet residue class), so the barrier is per block.
//
// The reference delegates all of this to the vendor library
// (multipath-orchestrator/libampccl/core/virtual_collective.h:246-252 for
// all-reduce, :355-374 all-gather, :537-554 reduce-scatter, :740-757
// all-to-all) and packs/merges segment prefixes with extra D2D copies
// (virtual_collective.h:162-183).
#include <cuda_runtime.h>

#include "nvl/nvl_device.cuh"
#include "nvl/nvl_launch.h"

namespace hl {
namespace dev {

constexpr int kUnroll = 4;

struct Ctx {
  uint64_t g0;       // first in-segment packet index of this thread
  uint64_t gstride;  // packets covered by the whole grid per sweep
};
__device__ __forceinline__ Ctx makeCtx() {
  Ctx x;
  x.g0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  x.gstride = (uint64_t)gridDim.x * blockDim.x;
  return x;
}

// user segment -> staging (packets of this block's residue class)
template <typename S, typename W, bool kMc, int U = kUnroll>
__device__ __forceinline__ void segCopyIn(uint4* stage_seg, const S* src, uint64_t seg_count, const Ctx& x) {
  constexpr int N = Packet<W>::N;
  const uint64_t np = (seg_count + N - 1) / N;
  const bool vec = aligned16(src);
  for (uint64_t i = x.g0; i < np; i += x.gstride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t j = i + (uint64_t)u * x.gstride;
      if (j < np) v[u] = loadUserPacket<S, W>(src, j * N, seg_count, vec);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t j = i + (uint64_t)u * x.gstride;
      if (j < np) {
        if constexpr (kMc) multimemSt(stage_seg + j, v[u]);  // stage_seg is a multicast address
        else stage_seg[j] = v[u];
      }
    }
  }
}

// staging (local or peer) -> user segment
template <typename W, typename D, int U = kUnroll>
__device__ __forceinline__ void segCopyOut(D* dst, const uint4* stage_seg, uint64_t seg_count, const Ctx& x) {
  constexpr int N = Packet<W>::N;
  const uint64_t np = (seg_count + N - 1) / N;
  const bool vec = aligned16(dst);
  for (uint64_t i = x.g0; i < np; i += x.gstride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t j = i + (uint64_t)u * x.gstride;
      if (j < np) v[u] = stage_seg[j];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t j = i + (uint64_t)u * x.gstride;
      if (j < np) storeUserPacket<W, D>(dst, j * N, seg_count, vec, v[u]);
    }
  }
}

// Reduction over the same packet of every rank's staging, ranks visited in
// ascending order whatever the caller's rank: the sum order is fixed, so the
// result is bitwise identical on every rank and from run to run.
template <typename W, int MR = HL_MAX_RANKS>
__device__ __forceinline__ uint4 reducePackets(const uint4* v, int n, int op, float scale, int int_div) {
  constexpr int N = Packet<W>::N;
  typename Wire<W>::Acc acc[N], b[N];
  Packet<W>::unpack(v[0], acc);
#pragma unroll
  for (int q = 1; q < MR; ++q) {
    if (q < n) {
      Packet<W>::unpack(v[q], b);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = applyOp(op, acc[i], b[i]);
    }
  }
  finish<W>(acc, scale, int_div);
  return Packet<W>::pack(acc);
}

// Dispatch on the caller's element type. Conversions exist between fp32, fp16
// and bf16; every other wire type requires identical user types.
#define HL_USER_TYPE_SWITCH(W, dt, S, ...)                                    \
  do {                                                                        \
    if constexpr (IsFloatTrio<W>::value) {                                    \
      switch (dt) {                                                           \
        case hlFloat16: { using S = __half; __VA_ARGS__; } break;             \
        case hlBfloat16: { using S = __nv_bfloat16; __VA_ARGS__; } break;     \
        default: { using S = float; __VA_ARGS__; } break;                     \
      }                                                                       \
    } else {                                                                  \
      using S = W;                                                            \
      __VA_ARGS__;                                                            \
    }                                                                         \
  } while (0)

template <typename W, bool kMc = false, int U = kUnroll>
__device__ __forceinline__ void copyInAny(uint4* stage_seg, const void* src, int dt, uint64_t elem_off,
                                          uint64_t seg_count, const Ctx& x) {
  HL_USER_TYPE_SWITCH(W, dt, S, segCopyIn<S, W, kMc, U>(stage_seg, reinterpret_cast<const S*>(src) + elem_off, seg_count, x));
}
template <typename W, int U = kUnroll>
__device__ __forceinline__ void copyOutAny(void* dst, int dt, uint64_t elem_off, const uint4* stage_seg,
                                           uint64_t seg_count, const Ctx& x) {
  HL_USER_TYPE_SWITCH(W, dt, D, segCopyOut<W, D, U>(reinterpret_cast<D*>(dst) + elem_off, stage_seg, seg_count, x));
}

__device__ __forceinline__ uint64_t segElems(uint64_t count, uint64_t first, uint64_t span) {
  if (first >= count) return 0;
  const uint64_t left = count - first;
  return left < span ? left : span;
}

// ------------------------------------------------------------------ barrier
__global__ void __launch_bounds__(HL_NVL_THREADS) kBarrier(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  blockBarrier(c, a.seq + 1, 1);
  callDone(c, 0);
}

// ------------------------------------------------------------------ all-reduce, one-shot
// copy-in | barrier | every rank reduces all n copies of the whole message
// straight into its output | barrier (peers done reading).
template <typename W>
__global__ void __launch_bounds__(HL_NVL_THREADS) kAllReduceOneShot(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks;
  const Ctx x = makeCtx();
  const uint64_t np = (a.count + N - 1) / N;
  copyInAny<W>(reinterpret_cast<uint4*>(c.stage[c.rank]), a.in, a.in_dt, 0, a.count, x);
  if (!blockBarrier(c, a.seq + 1, 1)) return;
  const bool vec = aligned16(a.out);
  for (uint64_t i = x.g0; i < np; i += x.gstride) {
    uint4 v[HL_MAX_RANKS];
#pragma unroll
    for (int q = 0; q < HL_MAX_RANKS; ++q)
      if (q < n) v[q] = reinterpret_cast<const uint4*>(c.stage[q])[i];
    const uint4 r = reducePackets<W>(v, n, a.op, a.scale, a.int_div);
    HL_USER_TYPE_SWITCH(W, a.out_dt, D, storeUserPacket<W, D>(reinterpret_cast<D*>(a.out), i * N, a.count, vec, r));
  }
  blockBarrier(c, a.seq + 2, 2);
  callDone(c, 0);
}

// ------------------------------------------------------------------ all-reduce, two-shot over P2P
// copy-in | barrier | pull-reduce the owned shard from every peer, result
// written in place into the local staging shard | barrier | pull every shard
// from its owner straight into the output | barrier.
template <typename W>
__global__ void __launch_bounds__(HL_NVL_THREADS) kAllReduceTwoShot(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const Ctx x = makeCtx();
  const uint64_t np = (a.count + N - 1) / N;
  const uint64_t sp = (np + n - 1) / n;  // packets per shard
  uint4* mine = reinterpret_cast<uint4*>(c.stage[r]);
  for (int s = 0; s < n; ++s)
    copyInAny<W>(mine + s * sp, a.in, a.in_dt, s * sp * N, segElems(a.count, s * sp * N, sp * N), x);
  if (!blockBarrier(c, a.seq + 1, 1)) return;
  {
    const uint64_t first = (uint64_t)r * sp;
    const uint64_t shard_np = first >= np ? 0 : (np - first < sp ? np - first : sp);
    for (uint64_t i = x.g0; i < shard_np; i += x.gstride * 2) {
      uint4 v0[HL_MAX_RANKS], v1[HL_MAX_RANKS];
      const uint64_t j = i + x.gstride;
#pragma unroll
      for (int q = 0; q < HL_MAX_RANKS; ++q)
        if (q < n) {
          v0[q] = reinterpret_cast<const uint4*>(c.stage[q])[first + i];
          if (j < shard_np) v1[q] = reinterpret_cast<const uint4*>(c.stage[q])[first + j];
        }
      mine[first + i] = reducePackets<W>(v0, n, a.op, a.scale, a.int_div);
      if (j < shard_np) mine[first + j] = reducePackets<W>(v1, n, a.op, a.scale, a.int_div);
    }
  }
  if (!blockBarrier(c, a.seq + 2, 2)) return;
  for (int k = 0; k < n; ++k) {
    const int s = (r + k) % n;  // start at the local shard, then walk the peers
    copyOutAny<W>(a.out, a.out_dt, s * sp * N, reinterpret_cast<const uint4*>(c.stage[s]) + s * sp,
                  segElems(a.count, s * sp * N, sp * N), x);
  }
  blockBarrier(c, a.seq + 3, 3);
  callDone(c, 0);
}

// ------------------------------------------------------------------ all-reduce through NVSwitch (NVLS)
// copy-in | barrier | multimem.ld_reduce of the owned shard (the switch sums
// all ranks' copies, fp32 accumulate), scale, multimem.st back in place into
// every rank's staging | barrier | local copy-out.
template <typename W>
__global__ void __launch_bounds__(HL_NVL_THREADS) kAllReduceNvls(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const Ctx x = makeCtx();
  const uint64_t np = (a.count + N - 1) / N;
  const uint64_t sp = (np + n - 1) / n;
  uint4* mine = reinterpret_cast<uint4*>(c.stage[r]);
  for (int s = 0; s < n; ++s)
    copyInAny<W>(mine + s * sp, a.in, a.in_dt, s * sp * N, segElems(a.count, s * sp * N, sp * N), x);
  if (!blockBarrier(c, a.seq + 1, 1)) return;
  {
    const uint64_t first = (uint64_t)r * sp;
    const uint64_t shard_np = first >= np ? 0 : (np - first < sp ? np - first : sp);
    uint4* mc = reinterpret_cast<uint4*>(c.mc_stage) + first;
    for (uint64_t i = x.g0; i < shard_np; i += x.gstride * kUnroll) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint64_t j = i + (uint64_t)u * x.gstride;
        if (j < shard_np) v[u] = multimemLdReduceAdd<W>(mc + j);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint64_t j = i + (uint64_t)u * x.gstride;
        if (j < shard_np) {
          if (a.scale != 1.0f) {
            typename Wire<W>::Acc acc[N];
            Packet<W>::unpack(v[u], acc);
            finish<W>(acc, a.scale, 0);
            v[u] = Packet<W>::pack(acc);
          }
          multimemSt(mc + j, v[u]);
        }
      }
    }
  }
  if (!blockBarrier(c, a.seq + 2, 2)) return;
  for (int s = 0; s < n; ++s)
    copyOutAny<W>(a.out, a.out_dt, s * sp * N, mine + s * sp, segElems(a.count, s * sp * N, sp * N), x);
  blockBarrier(c, a.seq + 3, 3);   // rule A: a peer's next call may store into this staging
  callDone(c, 0);
}

// ------------------------------------------------------------------ pipelined all-reduce / reduce-scatter
// Large messages: the three phases of the two-shot scheme run CONCURRENTLY on
// different tiles. Each CTA is split into three warp groups,
//   A  copy-in:   caller's buffer -> symmetric staging (HBM traffic)
//   B  exchange:  reduce the owned part of the tile over NVLink
//                           (multimem.ld_reduce through the switch, or 16-byte
//                           pulls from every peer) and hand the result out
//                           (multimem.st / pushes to every peer)
//   C  copy-out:  staging -> caller's output (all-reduce only)
// and walks the tiles b, b+G, b+2G ... of the message. Tile k of block b is
// handed from group to group — and from GPU to GPU — by the same mechanism: a
// monotonically increasing word per (stage, block, source rank) in every rank's
// flag area, written with st.release.sys after a group-wide named barrier and
// polled (bounded) with ld.acquire.sys. While group B of a block moves tile k
// over NVLink, group A already stages tile k+1 from HBM and group C drains tile
// k-1, so the HBM copies hide behind the link time instead of adding to it.
// Staging is as large as the (sliced) message, so tiles never wait for space.
__device__ __forceinline__ void groupSync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// `lane` selects the flag word: the CTA index when the stages of a tile are warp groups of one CTA, the index of
// the CTA triple (or pair) when they are CTAs of their own.
__device__ __forceinline__ void tileSignal(const HlCommDev& c, int kind, uint64_t value, int gtid, unsigned lane) {
  if (gtid < c.nranks) {
    stReleaseSys(c.flags[gtid] + ((size_t)kind * HL_MAX_BLOCKS + lane) * HL_MAX_RANKS + c.rank, value);
  }
}

// Returns through *abort_flag (shared memory) whether the wait was abandoned.
__device__ __forceinline__ void tileWait(const HlCommDev& c, int kind, uint64_t value, int gtid, volatile int* abort_flag, int step,
                                         unsigned lane) {
  if (gtid < c.nranks) {
    const uint64_t* mine = c.flags[c.rank] + ((size_t)kind * HL_MAX_BLOCKS + lane) * HL_MAX_RANKS + gtid;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (ldAcquireSys(mine) < value) {
      if ((++spins & 31u) == 0) {
        const uint64_t now = globalTimerNs();
        if (t0 == 0) t0 = now;
        const bool aborted = *reinterpret_cast<volatile uint32_t*>(c.abort_word) != 0 || *abort_flag != 0;
        if (aborted || now - t0 > c.timeout_ns) {
          if (!aborted) {
            volatile uint64_t* st = c.status;
            st[1] = ((uint64_t)step << 32) | (uint64_t)gtid;
            st[2] = blockIdx.x;
            st[0] = HL_DEV_TIMEOUT;
            *reinterpret_cast<volatile uint32_t*>(c.abort_word) = 1;
            __threadfence_system();
          }
          *abort_flag = 1;
          break;
        }
      }
    }
  }
}

// Warp split A / B / C (four warps each).
template <bool kNvls> struct PipeShape {
  static constexpr int A = 4, B = 4, C = 4;
};
constexpr int kPipeCopyUnroll = 4;
constexpr int kPushUnroll = 8;      // 16-byte packets in flight per thread in the copy phases of the push kernels
constexpr int kPipeNvlsUnroll = 8;  // 16-byte multimem.ld_reduce in flight per exchange thread
constexpr int kPipeThreads = 384;  // 12 warps: leaves ~170 registers per thread for the deep unrolls

// Peer-pointer variant: every access that crosses NVLink is a posted STORE.
// A remote load stalls its thread for a full round trip through the switch
// (several microseconds under load), so a pull design needs megabytes in
// flight; pushes are fire-and-forget until the fence before the flag. Stage A
// therefore pushes, straight from the caller's buffer, the tile of every
// shard into slot `rank` of that shard's owner (no local staging copy at
// all); stage B folds the owner's own tile (read from the caller's buffer)
// with the landed slots — all local reads, ascending rank order — and pushes
// the result to every peer's result area (its own part goes directly to the
// caller's output); stage C copies the other owners' results out locally.
template <typename S, typename W, int U = kPipeCopyUnroll>
__device__ __forceinline__ void pushTile(uint4* remote_slot, const S* src, uint64_t cnt, const Ctx& x) {
  constexpr int N = Packet<W>::N;
  const uint64_t np = (cnt + N - 1) / N;
  const bool vec = aligned16(src);
  for (uint64_t i = x.g0; i < np; i += x.gstride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t j = i + (uint64_t)u * x.gstride;
      if (j < np) v[u] = loadUserPacket<S, W>(src, j * N, cnt, vec);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t j = i + (uint64_t)u * x.gstride;
      if (j < np) remote_slot[j] = v[u];
    }
  }
}

// U packets per thread and per source are in flight at once; MR bounds the rank count the
// unrolled source loop is compiled for (registers: U * MR * 4 for the landed packets).
template <typename S, typename W, typename D, bool kAllReduce, int U = 2, int MR = HL_MAX_RANKS>
__device__ __forceinline__ void foldTile(const HlCommDev& c, const HlCallArgs& a, const S* own, uint64_t own_cnt, D* out,
                                         uint64_t out_cnt, uint64_t sp, uint64_t p0, uint64_t tp, uint64_t res_off, const Ctx& x) {
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const uint4* slots = reinterpret_cast<const uint4*>(c.stage[r]);
  const bool vin = aligned16(own), vout = aligned16(out);
  for (uint64_t i = x.g0; i < tp; i += x.gstride * U) {
    uint4 v[U][MR];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t j = i + (uint64_t)u * x.gstride;
      if (j < tp) {
#pragma unroll
        for (int q = 0; q < MR; ++q)
          if (q < n) v[u][q] = q == r ? loadUserPacket<S, W>(own, j * N, own_cnt, vin) : slots[(uint64_t)q * sp + p0 + j];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t j = i + (uint64_t)u * x.gstride;
      if (j < tp) {
        const uint4 red = reducePackets<W, MR>(v[u], n, a.op, a.scale, a.int_div);
        storeUserPacket<W, D>(out, j * N, out_cnt, vout, red);
        if constexpr (kAllReduce) {
#pragma unroll
          for (int q = 0; q < MR; ++q)
            if (q < n && q != r) (reinterpret_cast<uint4*>(c.stage[q]) + res_off + (uint64_t)r * sp + p0)[j] = red;
        }
      }
    }
  }
}

template <typename W, bool kNvls, bool kAllReduce>
__global__ void __launch_bounds__(kPipeThreads) kPipelined(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const uint64_t np = (a.count + N - 1) / N;
  const uint64_t sp = kAllReduce ? (np + n - 1) / n : np;   // packets per shard (all-reduce) or per segment (reduce-scatter)
  const uint64_t tps = a.tile_packets;
  const uint64_t tiles = (sp + tps - 1) / tps;
  const uint64_t in_stride = kAllReduce ? sp * N : a.in_seg_stride;   // elements between shards / segments in the input
  const uint64_t seg_elems = a.count;                                 // reduce-scatter: valid elements per segment
  const int warp = threadIdx.x >> 5;
  constexpr int kPipeWarpsA = PipeShape<kNvls>::A, kPipeWarpsB = PipeShape<kNvls>::B, kPipeWarpsC = PipeShape<kNvls>::C;
  static_assert((kPipeWarpsA + kPipeWarpsB + kPipeWarpsC) * 32 == kPipeThreads, "warp groups must fill the CTA");
  const int role = warp < kPipeWarpsA ? 0 : (warp < kPipeWarpsA + kPipeWarpsB ? 1 : 2);
  const int gthreads = (role == 0 ? kPipeWarpsA : (role == 1 ? kPipeWarpsB : kPipeWarpsC)) * 32;
  const int gtid = threadIdx.x - (role == 0 ? 0 : (role == 1 ? kPipeWarpsA : kPipeWarpsA + kPipeWarpsB)) * 32;
  Ctx x;
  x.g0 = (uint64_t)gtid;
  x.gstride = (uint64_t)gthreads;
  uint4* mine = reinterpret_cast<uint4*>(c.stage[r]);
  // all-reduce over P2P keeps results in a second region so that peers never overwrite inputs still being pulled
  const uint64_t res_off = (kAllReduce && !kNvls) ? sp * (uint64_t)n : 0;
  uint64_t k = 0;
  for (uint64_t t = blockIdx.x; t < tiles; t += gridDim.x, ++k) {
    const uint64_t target = a.pipe_seq + k + 1;
    const uint64_t p0 = t * tps;                                   // first packet of the tile inside a shard
    const uint64_t tp = sp - p0 < tps ? sp - p0 : tps;             // packets of this tile inside a shard
    if (role == 0) {
      for (int k2 = 0; k2 < n; ++k2) {
        const int s = kNvls ? k2 : (r + 1 + k2) % n;               // pushes start at the next rank to spread the load
        // elements of shard / segment s that fall into this tile
        uint64_t e0 = p0 * N, cnt;
        if constexpr (kAllReduce) {
          const uint64_t g0e = (uint64_t)s * in_stride + e0;       // global element index
          cnt = g0e >= a.count ? 0 : (a.count - g0e < tp * N ? a.count - g0e : tp * N);
        } else {
          cnt = e0 >= seg_elems ? 0 : (seg_elems - e0 < tp * N ? seg_elems - e0 : tp * N);
        }
        if constexpr (kNvls) {
          copyInAny<W, false, kPipeCopyUnroll>(mine + (uint64_t)s * sp + p0, a.in, a.in_dt, (uint64_t)s * in_stride + e0, cnt, x);
        } else {
          if (s == r) continue;                                    // the owner reads its own tile from the caller's buffer
          uint4* slot = reinterpret_cast<uint4*>(c.stage[s]) + (uint64_t)r * sp + p0;
          pushTile<W, W>(slot, reinterpret_cast<const W*>(a.in) + (uint64_t)s * in_stride + e0, cnt, x);
        }
      }
      groupSync(1, gthreads);
      tileSignal(c, 1, target, gtid, blockIdx.x);
    } else if (role == 1) {
      tileWait(c, 1, target, gtid, &s_abort, 1, blockIdx.x);
      groupSync(2, gthreads);
      if (s_abort) break;
      const uint64_t first = (uint64_t)r * sp + p0;
      if constexpr (kNvls) {
        uint4* mc = reinterpret_cast<uint4*>(c.mc_stage) + first;
        for (uint64_t i = x.g0; i < tp; i += x.gstride * kPipeNvlsUnroll) {
          uint4 v[kPipeNvlsUnroll];
#pragma unroll
          for (int u = 0; u < kPipeNvlsUnroll; ++u) {
            const uint64_t j = i + (uint64_t)u * x.gstride;
            if (j < tp) v[u] = multimemLdReduceAdd<W>(mc + j);
          }
#pragma unroll
          for (int u = 0; u < kPipeNvlsUnroll; ++u) {
            const uint64_t j = i + (uint64_t)u * x.gstride;
            if (j < tp) {
              if (a.scale != 1.0f) {
                typename Wire<W>::Acc acc[N];
                Packet<W>::unpack(v[u], acc);
                finish<W>(acc, a.scale, 0);
                v[u] = Packet<W>::pack(acc);
              }
              if constexpr (kAllReduce) {
                multimemSt(mc + j, v[u]);
              } else {
                HL_USER_TYPE_SWITCH(W, a.out_dt, D, storeUserPacket<W, D>(reinterpret_cast<D*>(a.out), (p0 + j) * N, a.count, aligned16(a.out), v[u]));
              }
            }
          }
        }
      } else {
        const uint64_t e0 = p0 * N;
        const uint64_t own_first = (uint64_t)r * in_stride + e0;   // element index of the owned tile in the input
        uint64_t own_cnt, out_first, out_cnt;
        if constexpr (kAllReduce) {
          own_cnt = own_first >= a.count ? 0 : (a.count - own_first < tp * N ? a.count - own_first : tp * N);
          out_first = own_first;
          out_cnt = own_cnt;
        } else {
          own_cnt = e0 >= seg_elems ? 0 : (seg_elems - e0 < tp * N ? seg_elems - e0 : tp * N);
          out_first = e0;
          out_cnt = own_cnt;
        }
        const uint64_t tpk = (own_cnt + N - 1) / N;                // packets that hold valid elements
        // the push variant moves the caller's element type unchanged (the host side
        // routes converting calls to the staged kernels)
        foldTile<W, W, W, kAllReduce>(c, a, reinterpret_cast<const W*>(a.in) + own_first, own_cnt,
                                      reinterpret_cast<W*>(a.out) + out_first, out_cnt, sp, p0, tpk, res_off, x);
      }
      if constexpr (kAllReduce) {
        groupSync(2, gthreads);
        tileSignal(c, 2, target, gtid, blockIdx.x);
      }
    } else {
      if constexpr (kAllReduce) {
        tileWait(c, 2, target, gtid, &s_abort, 2, blockIdx.x);
        groupSync(3, gthreads);
        if (s_abort) break;
        for (int s = 0; s < n; ++s) {
          if (!kNvls && s == r) continue;                          // written by the exchange stage already
          const uint64_t e0 = p0 * N;
          const uint64_t g0e = (uint64_t)s * in_stride + e0;
          uint64_t cnt = g0e >= a.count ? 0 : (a.count - g0e < tp * N ? a.count - g0e : tp * N);
          const uint64_t shard_left = sp * N - e0;
          if (cnt > shard_left) cnt = shard_left;
          copyOutAny<W, kPipeCopyUnroll>(a.out, a.out_dt, g0e, mine + res_off + (uint64_t)s * sp + p0, cnt, x);
        }
      }
    }
  }
  // rule A. Reduce-scatter: peers pull from this rank's staging in their exchange stage. All-reduce: the copy-out
  // stage reads this rank's own staging, which a peer's next call may store into.
  blockBarrier(c, a.seq + 1, 3);
  callDone(c, (tiles + gridDim.x - 1) / gridDim.x);
}

// ------------------------------------------------------------------ pipelined push all-reduce / reduce-scatter, one CTA per stage
// The stores-only scheme of kPush below, cut into tiles whose stages run at the same time on CTAs of their own.
// Measured on the link (2 GPUs, both directions loaded): posted 16-byte stores from 16 to 37 CTAs already fill a
// direction (~690 GB/s) and a fold is HBM-bound, so a stage gains nothing from more than a third of the SMs, while
// the phases of kPush — push | wait | fold | wait | copy-out, each with the whole grid — leave the link idle for a
// fifth (all-reduce) to a third (reduce-scatter) of the call. CTAs form lanes of three (all-reduce: push, fold,
// copy-out) or two (reduce-scatter: push, fold); lane L handles tiles L, L + lanes, ...; its stages hand a tile
// on — across GPUs — through the tile flag words [kind][lane][source rank], exactly as the warp groups of
// kPipelined do. Nothing waits for space (staging holds the whole sliced message), so the only waits are for data.
// Valid elements of a shard (all-reduce: it starts at element `shard_first` of the buffer) or of a segment
// (reduce-scatter: `count` elements each) that fall into the tile of `tp` packets starting at packet p0.
template <bool kAllReduce, int N>
__device__ __forceinline__ uint64_t tileElems(uint64_t count, uint64_t shard_first, uint64_t p0, uint64_t tp) {
  const uint64_t e0 = p0 * N;
  const uint64_t g = kAllReduce ? shard_first + e0 : e0;
  return g >= count ? 0 : (count - g < tp * N ? count - g : tp * N);
}

// The fold of one tile of the owned shard. MR bounds the rank count the unrolled source loop is compiled for; one
// kernel carries one such variant (three of them side by side push the register allocator into local memory).
template <typename W, bool kAllReduce, int MR>
__device__ __forceinline__ void foldStage(const HlCommDev& c, const HlCallArgs& a, uint64_t in_stride, uint64_t sp, uint64_t p0, uint64_t tp,
                                       uint64_t res_off, const Ctx& x) {
  constexpr int N = Packet<W>::N;
  const int r = c.rank;
  const uint64_t cnt = tileElems<kAllReduce, N>(a.count, (uint64_t)r * in_stride, p0, tp);
  const W* own = reinterpret_cast<const W*>(a.in) + (uint64_t)r * in_stride + p0 * N;
  W* res = reinterpret_cast<W*>(a.out) + (kAllReduce ? (uint64_t)r * in_stride : 0) + p0 * N;
  const uint64_t tpk = (cnt + N - 1) / N;
  constexpr int U = MR <= 2 ? 6 : (MR <= 4 ? 3 : 2);   // about a dozen landed packets per thread in flight
  foldTile<W, W, W, kAllReduce, U, MR>(c, a, own, cnt, res, cnt, sp, p0, tpk, res_off, x);
}

__device__ __forceinline__ void barArrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Hand-off without a stall. The release store that announces a tile has to see the CTA's posted stores acknowledged;
// under load that takes longer than pushing a 128 KiB tile (measured: 8 us against 5 us), and a CTA that does it
// itself idles its share of the link meanwhile. Stages that announce tiles therefore give up their last warp as a
// signaller: the working warps arrive on named barrier 1 when a tile's stores are issued and go on with the next
// tile; the signaller picks the tile up there, acknowledges the pick-up on named barrier 2 (the workers wait for
// that before they arrive again, so the two never run more than one tile apart) and only then pays for the release.
template <typename W, bool kAllReduce, int MR>
__global__ void __launch_bounds__(HL_NVL_THREADS, 1) kPipeCta(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  __shared__ int s_abort;
  __shared__ unsigned long long s_stop_at;   // tile (ordinal within this lane) at which the workers gave up
  if (threadIdx.x == 0) {
    s_abort = 0;
    s_stop_at = ~0ull;
  }
  __syncthreads();
  constexpr int N = Packet<W>::N;
  // CTAs per lane. All-reduce: push, fold (which pushes the result on), copy-out. Reduce-scatter: one pusher and
  // three folders that each take a third of the tile — 16 to 37 CTAs of posted stores fill the link, while the
  // fold is the stage that needs the SMs (measured with one folder per pusher: push 183 us, fold 247 us).
  const unsigned kFoldParts = kAllReduce ? 1u : (unsigned)(a.lane_parts >= 1 && a.lane_parts <= 7 ? a.lane_parts : 3);
  const unsigned kRoles = kAllReduce ? 3u : 1u + kFoldParts;
  const int n = c.nranks, r = c.rank;
  const uint64_t np = (a.count + N - 1) / N;
  const uint64_t sp = kAllReduce ? (np + n - 1) / n : np;   // packets per shard (all-reduce) or per segment (reduce-scatter)
  const uint64_t tps = a.tile_packets;
  const uint64_t tiles = (sp + tps - 1) / tps;
  const uint64_t in_stride = kAllReduce ? sp * N : a.in_seg_stride;
  const uint64_t res_off = sp * (uint64_t)n;                // results live behind the n slots
  const unsigned member = blockIdx.x % kRoles, lane = blockIdx.x / kRoles, lanes = gridDim.x / kRoles;
  const unsigned role = kAllReduce ? member : (member == 0 ? 0u : 1u);   // 0 push, 1 fold, 2 copy-out
  const unsigned part = kAllReduce ? 0u : (member == 0 ? 0u : member - 1);
  const bool announces = role == 0 || (kAllReduce && role == 1);
  const int workers = announces ? (int)blockDim.x - 32 : (int)blockDim.x;
  const bool signaller = announces && (int)threadIdx.x >= workers;
  const int gtid = (int)threadIdx.x;
  const uint64_t my_tiles = lane < lanes && lane < tiles ? (tiles - lane + lanes - 1) / lanes : 0;
  Ctx x;
  x.g0 = threadIdx.x;
  x.gstride = (uint64_t)workers;
  const W* in = reinterpret_cast<const W*>(a.in);
  W* out = reinterpret_cast<W*>(a.out);
  // Kernel timeline: thread 0 adds up what this CTA spent waiting for a tile, held back by the hand-off and
  // working; the sums land in stamp slots 1 to 3 at exit.
  const bool timed = c.timeline != nullptr && threadIdx.x == 0;
  uint64_t t_wait = 0, t_hand = 0, t_work = 0, t_mark = timed ? globalTimerNs() : 0;
  auto lap = [&](uint64_t& sum) {
    if (timed) {
      const uint64_t now = globalTimerNs();
      sum += now - t_mark;
      t_mark = now;
    }
  };
  if (signaller) {
    const int kind = role == 0 ? 1 : 2;
    for (uint64_t k = 0; k < my_tiles; ++k) {
      groupSync(1, (int)blockDim.x);                          // tile k's stores are issued (or the workers gave up at k)
      // not s_abort: that may already be set for tile k + 1 while tile k still has to be picked up and announced
      if (*reinterpret_cast<volatile unsigned long long*>(&s_stop_at) == k) break;
      if (k + 1 < my_tiles) barArrive(2, (int)blockDim.x);    // picked up: the workers may announce the next one
      tileSignal(c, kind, a.pipe_seq + k + 1, gtid - workers, lane);
    }
  } else {
    for (uint64_t k = 0; k < my_tiles; ++k) {
      const uint64_t t = lane + k * lanes;
      const uint64_t target = a.pipe_seq + k + 1;
      const uint64_t p0 = t * tps;
      const uint64_t tp = sp - p0 < tps ? sp - p0 : tps;
      bool gave_up = false;
      if (role == 0) {
        for (int k2 = 1; k2 < n; ++k2) {
          const int s = (r + k2) % n;   // start at the next rank: the owners are loaded evenly
          pushTile<W, W, kPipeCopyUnroll>(reinterpret_cast<uint4*>(c.stage[s]) + (uint64_t)r * sp + p0, in + (uint64_t)s * in_stride + p0 * N,
                                          tileElems<kAllReduce, N>(a.count, (uint64_t)s * in_stride, p0, tp), x);
        }
        lap(t_work);
      } else if (role == 1) {
        tileWait(c, 1, target, gtid, &s_abort, 1, lane);
        groupSync(3, workers);
        lap(t_wait);
        gave_up = s_abort != 0;
        if (!gave_up) {
          const uint64_t chunk = (tp + kFoldParts - 1) / kFoldParts;   // this folder's share of the tile
          const uint64_t f0 = (uint64_t)part * chunk;
          if (f0 < tp) foldStage<W, kAllReduce, MR>(c, a, in_stride, sp, p0 + f0, tp - f0 < chunk ? tp - f0 : chunk, res_off, x);
        }
        lap(t_work);
      } else {
        tileWait(c, 2, target, gtid, &s_abort, 2, lane);
        groupSync(3, workers);
        lap(t_wait);
        if (s_abort) break;
        const uint4* mine = reinterpret_cast<const uint4*>(c.stage[r]);
        for (int k2 = 1; k2 < n; ++k2) {
          const int s = (r + k2) % n;
          segCopyOut<W, W, kPipeCopyUnroll>(out + (uint64_t)s * in_stride + p0 * N, mine + res_off + (uint64_t)s * sp + p0,
                                            tileElems<kAllReduce, N>(a.count, (uint64_t)s * in_stride, p0, tp), x);
        }
        lap(t_work);
      }
      if (announces) {
        if (k > 0) groupSync(2, (int)blockDim.x);             // the signaller has picked up tile k - 1
        if (gave_up && threadIdx.x == 0) s_stop_at = k;       // ordered before the arrival below
        barArrive(1, (int)blockDim.x);                        // tile k is ready (or: nothing more comes)
        lap(t_hand);
      }
      if (gave_up) break;
    }
  }
  // rule A: a pusher of the next call may overwrite slots that a slower peer is still folding (or, all-reduce,
  // result areas that it is still copying out): nobody leaves before every peer's CTA of the same index is through
  blockBarrier(c, a.seq + 1, 3);
  if (timed && blockIdx.x < HL_TL_BLOCKS) {
    lap(t_work);
    // slots 1..3 hold entry + duration, so that "time since entry" reads as the three sums; slot 4 carries the
    // stage (0 push, 1 fold, 2 copy-out) the same way, in milliseconds
    uint64_t* st = c.timeline + (((a.seq / HL_SEQ_STRIDE) % HL_TL_CALLS) * HL_TL_BLOCKS + blockIdx.x) * HL_TL_PHASES;
    const uint64_t e = st[0];
    st[1] = e + t_wait;
    st[2] = e + t_hand;
    st[3] = e + t_work;
    st[4] = e + (uint64_t)role * 1000000ull;
  }
  callDone(c, lanes ? (tiles + lanes - 1) / lanes : 0);
}

// ------------------------------------------------------------------ push all-reduce / reduce-scatter over peer pointers
// Every NVLink access is a posted store and every load is local:
//   1. push: each rank streams, straight from the caller's buffer, shard s of
//      its input into slot `rank` of shard s's owner (nothing is staged locally);
//   barrier
//   2. fold: the owner adds its own shard (read from the caller's buffer) and
//      the n-1 landed slots in ascending rank order, writes its part of the
//      result to the caller's output and (all-reduce) pushes it into every
//      peer's result area;
//   barrier
//   3. (all-reduce) copy the other owners' results from the local result area
//      to the caller's output.
// All 512 threads of every CTA work in every phase, so each phase has the
// whole grid's loads and stores in flight. The caller's element type is the
// wire type (converting calls use the staged kernels).
template <typename W, bool kAllReduce>
__global__ void __launch_bounds__(HL_NVL_THREADS) kPush(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const Ctx x = makeCtx();
  const uint64_t np = (a.count + N - 1) / N;
  const uint64_t sp = kAllReduce ? (np + n - 1) / n : np;
  const uint64_t in_stride = kAllReduce ? sp * N : a.in_seg_stride;
  const uint64_t res_off = sp * (uint64_t)n;
  const W* in = reinterpret_cast<const W*>(a.in);
  W* out = reinterpret_cast<W*>(a.out);
  auto shardElems = [&](int s) -> uint64_t {
    if constexpr (kAllReduce) return segElems(a.count, (uint64_t)s * sp * N, sp * N);
    else return a.count;
  };
  for (int k = 1; k < n; ++k) {
    const int s = (r + k) % n;
    pushTile<W, W, kPushUnroll>(reinterpret_cast<uint4*>(c.stage[s]) + (uint64_t)r * sp, in + (uint64_t)s * in_stride, shardElems(s), x);
  }
  if (!blockBarrier(c, a.seq + 1, 1)) return;
  {
    const uint64_t cnt = shardElems(r);
    const uint64_t first = kAllReduce ? (uint64_t)r * sp * N : 0;
    // about a dozen landed packets per thread in flight whatever the rank count (more spills registers)
    if (n <= 2)
      foldTile<W, W, W, kAllReduce, 6, 2>(c, a, in + (uint64_t)r * in_stride, cnt, out + first, cnt, sp, 0, (cnt + N - 1) / N, res_off, x);
    else if (n <= 4)
      foldTile<W, W, W, kAllReduce, 3, 4>(c, a, in + (uint64_t)r * in_stride, cnt, out + first, cnt, sp, 0, (cnt + N - 1) / N, res_off, x);
    else
      foldTile<W, W, W, kAllReduce, 2, HL_MAX_RANKS>(c, a, in + (uint64_t)r * in_stride, cnt, out + first, cnt, sp, 0, (cnt + N - 1) / N, res_off, x);
  }
  if (!blockBarrier(c, a.seq + 2, 2)) return;
  if constexpr (kAllReduce) {
    const uint4* mine = reinterpret_cast<const uint4*>(c.stage[r]);
    for (int k = 1; k < n; ++k) {
      const int s = (r + k) % n;
      segCopyOut<W, W, kPushUnroll>(out + (uint64_t)s * sp * N, mine + res_off + (uint64_t)s * sp, shardElems(s), x);
    }
    // rule A: the result areas just read are where a peer's next (larger) call pushes its slots
    blockBarrier(c, a.seq + 3, 3);
  }
  callDone(c, 0);
}

// ------------------------------------------------------------------ reduce-scatter
// `in` holds n segments (stride in_seg_stride); the first `count` elements of
// each are handled. copy-in | barrier | pull-reduce segment r from every peer
// straight into the output | barrier.
template <typename W, bool kNvls>
__global__ void __launch_bounds__(HL_NVL_THREADS) kReduceScatter(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const Ctx x = makeCtx();
  const uint64_t sp = (a.count + N - 1) / N;
  uint4* mine = reinterpret_cast<uint4*>(c.stage[r]);
  for (int s = 0; s < n; ++s) copyInAny<W>(mine + s * sp, a.in, a.in_dt, s * a.in_seg_stride, a.count, x);
  if (!blockBarrier(c, a.seq + 1, 1)) return;
  const bool vec = aligned16(a.out);
  const uint64_t first = (uint64_t)r * sp;
  if constexpr (kNvls) {
    const uint4* mc = reinterpret_cast<const uint4*>(c.mc_stage) + first;
    for (uint64_t i = x.g0; i < sp; i += x.gstride * kUnroll) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint64_t j = i + (uint64_t)u * x.gstride;
        if (j < sp) v[u] = multimemLdReduceAdd<W>(mc + j);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint64_t j = i + (uint64_t)u * x.gstride;
        if (j < sp) {
          if (a.scale != 1.0f) {
            typename Wire<W>::Acc acc[N];
            Packet<W>::unpack(v[u], acc);
            finish<W>(acc, a.scale, 0);
            v[u] = Packet<W>::pack(acc);
          }
          HL_USER_TYPE_SWITCH(W, a.out_dt, D,
                              storeUserPacket<W, D>(reinterpret_cast<D*>(a.out), j * N, a.count, vec, v[u]));
        }
      }
    }
  } else {
    for (uint64_t i = x.g0; i < sp; i += x.gstride * 2) {
      uint4 v0[HL_MAX_RANKS], v1[HL_MAX_RANKS];
      const uint64_t j = i + x.gstride;
#pragma unroll
      for (int q = 0; q < HL_MAX_RANKS; ++q)
        if (q < n) {
          v0[q] = reinterpret_cast<const uint4*>(c.stage[q])[first + i];
          if (j < sp) v1[q] = reinterpret_cast<const uint4*>(c.stage[q])[first + j];
        }
      const uint4 r0 = reducePackets<W>(v0, n, a.op, a.scale, a.int_div);
      HL_USER_TYPE_SWITCH(W, a.out_dt, D, storeUserPacket<W, D>(reinterpret_cast<D*>(a.out), i * N, a.count, vec, r0));
      if (j < sp) {
        const uint4 r1 = reducePackets<W>(v1, n, a.op, a.scale, a.int_div);
        HL_USER_TYPE_SWITCH(W, a.out_dt, D, storeUserPacket<W, D>(reinterpret_cast<D*>(a.out), j * N, a.count, vec, r1));
      }
    }
  }
  blockBarrier(c, a.seq + 2, 2);
  callDone(c, 0);
}

// ------------------------------------------------------------------ all-gather
// P2P: copy-in of the local prefix | barrier | pull every rank's prefix into
// out + q*out_seg_stride | barrier.
// NVLS: barrier | multimem.st of the local prefix from the caller's buffer into
// slot r of every rank's staging (one store, n destinations) | barrier | local
// copy-out of all n slots.
template <typename W, bool kNvls>
__global__ void __launch_bounds__(HL_NVL_THREADS) kAllGather(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const Ctx x = makeCtx();
  const uint64_t sp = (a.count + N - 1) / N;
  uint4* mine = reinterpret_cast<uint4*>(c.stage[r]);
  if constexpr (kNvls) {
    if (!blockBarrier(c, a.seq + 1, 1)) return;
    uint4* mc = reinterpret_cast<uint4*>(c.mc_stage) + (uint64_t)r * sp;
    copyInAny<W, true>(mc, a.in, a.in_dt, 0, a.count, x);
    if (!blockBarrier(c, a.seq + 2, 2)) return;
    for (int q = 0; q < n; ++q) copyOutAny<W>(a.out, a.out_dt, q * a.out_seg_stride, mine + q * sp, a.count, x);
    blockBarrier(c, a.seq + 3, 3);   // rule A
  } else {
    copyInAny<W>(mine, a.in, a.in_dt, 0, a.count, x);
    if (!blockBarrier(c, a.seq + 1, 1)) return;
    for (int k = 0; k < n; ++k) {
      const int q = (r + k) % n;
      copyOutAny<W>(a.out, a.out_dt, q * a.out_seg_stride, reinterpret_cast<const uint4*>(c.stage[q]), a.count, x);
    }
    blockBarrier(c, a.seq + 2, 2);
  }
  callDone(c, 0);
}

// Stores-only all-gather over peer pointers: every rank pushes its prefix straight from the caller's buffer into
// slot `rank` of every peer's staging (no local staging copy, and posted stores run ~7 % above loads from a peer on
// this link), copies its own prefix to its place in the output while the peers' data is on its way, and after the
// barrier copies the landed slots out locally. The caller's element type is the wire type.
template <typename W>
__global__ void __launch_bounds__(HL_NVL_THREADS) kAllGatherPush(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const Ctx x = makeCtx();
  const uint64_t sp = (a.count + N - 1) / N;
  const W* in = reinterpret_cast<const W*>(a.in);
  W* out = reinterpret_cast<W*>(a.out);
  for (int k = 1; k < n; ++k) {
    const int s = (r + k) % n;
    pushTile<W, W, kPushUnroll>(reinterpret_cast<uint4*>(c.stage[s]) + (uint64_t)r * sp, in, a.count, x);
  }
  W* own = out + (uint64_t)r * a.out_seg_stride;
  if (own != in) {  // in place (the input already sits in its segment of the output): nothing to copy
    const bool vin = aligned16(in), vout = aligned16(own);
    for (uint64_t i = x.g0; i < sp; i += x.gstride * kPipeCopyUnroll) {
      uint4 v[kPipeCopyUnroll];
#pragma unroll
      for (int u = 0; u < kPipeCopyUnroll; ++u) {
        const uint64_t j = i + (uint64_t)u * x.gstride;
        if (j < sp) v[u] = loadUserPacket<W, W>(in, j * N, a.count, vin);
      }
#pragma unroll
      for (int u = 0; u < kPipeCopyUnroll; ++u) {
        const uint64_t j = i + (uint64_t)u * x.gstride;
        if (j < sp) storeUserPacket<W, W>(own, j * N, a.count, vout, v[u]);
      }
    }
  }
  if (!blockBarrier(c, a.seq + 1, 1)) return;
  const uint4* mine = reinterpret_cast<const uint4*>(c.stage[r]);
  for (int k = 1; k < n; ++k) {
    const int s = (r + k) % n;
    segCopyOut<W, W, kPushUnroll>(out + (uint64_t)s * a.out_seg_stride, mine + (uint64_t)s * sp, a.count, x);
  }
  // the peers' next pushes may land in these slots: nobody leaves before every peer has copied out
  blockBarrier(c, a.seq + 2, 2);
  callDone(c, 0);
}

// The stores-only all-gather cut into tiles, with the link stage and the HBM stage on CTAs of their own (see
// kPipeCta): per lane one pusher — its last warp is the signaller — and three copiers that each take a third of
// every tile: they copy the own segment's part to its place, wait for the tile from all peers, and copy the landed
// parts out. The link never waits for a copy.
template <typename W>
__global__ void __launch_bounds__(HL_NVL_THREADS, 1) kAllGatherLanes(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  constexpr int N = Packet<W>::N;
  const unsigned kParts = (unsigned)(a.lane_parts >= 1 && a.lane_parts <= 7 ? a.lane_parts : 3);
  const unsigned kMembers = 1 + kParts;
  const int n = c.nranks, r = c.rank;
  const uint64_t sp = (a.count + N - 1) / N;
  const uint64_t tps = a.tile_packets;
  const uint64_t tiles = (sp + tps - 1) / tps;
  const unsigned member = blockIdx.x % kMembers, lane = blockIdx.x / kMembers, lanes = gridDim.x / kMembers;
  const bool pusher = member == 0;
  const int workers = pusher ? (int)blockDim.x - 32 : (int)blockDim.x;
  const bool signaller = pusher && (int)threadIdx.x >= workers;
  const int gtid = (int)threadIdx.x;
  const uint64_t my_tiles = lane < lanes && lane < tiles ? (tiles - lane + lanes - 1) / lanes : 0;
  Ctx x;
  x.g0 = threadIdx.x;
  x.gstride = (uint64_t)workers;
  const W* in = reinterpret_cast<const W*>(a.in);
  W* out = reinterpret_cast<W*>(a.out);
  W* own = out + (uint64_t)r * a.out_seg_stride;
  if (signaller) {
    for (uint64_t k = 0; k < my_tiles; ++k) {
      groupSync(1, (int)blockDim.x);                          // tile k's stores are issued
      if (k + 1 < my_tiles) barArrive(2, (int)blockDim.x);    // picked up
      tileSignal(c, 1, a.pipe_seq + k + 1, gtid - workers, lane);
    }
  } else {
    for (uint64_t k = 0; k < my_tiles; ++k) {
      const uint64_t p0 = (lane + k * lanes) * tps;
      const uint64_t tp = sp - p0 < tps ? sp - p0 : tps;
      if (pusher) {
        const uint64_t cnt = tileElems<false, N>(a.count, 0, p0, tp);
        for (int k2 = 1; k2 < n; ++k2) {
          const int s = (r + k2) % n;
          pushTile<W, W, kPipeCopyUnroll>(reinterpret_cast<uint4*>(c.stage[s]) + (uint64_t)r * sp + p0, in + p0 * N, cnt, x);
        }
        if (k > 0) groupSync(2, (int)blockDim.x);             // the signaller has picked up tile k - 1
        barArrive(1, (int)blockDim.x);
      } else {
        const uint64_t chunk = (tp + kParts - 1) / kParts;
        const uint64_t f0 = (uint64_t)(member - 1) * chunk;
        const uint64_t len = f0 >= tp ? 0 : (tp - f0 < chunk ? tp - f0 : chunk);
        const uint64_t q0 = p0 + f0;
        const uint64_t cnt = len ? tileElems<false, N>(a.count, 0, q0, len) : 0;
        if (cnt && own != in) {  // not in place: the own segment's part, while the peers' data is on its way
          const bool vin = aligned16(in), vout = aligned16(own);
          const uint64_t pk = (cnt + N - 1) / N;
          for (uint64_t i = x.g0; i < pk; i += x.gstride * kPipeCopyUnroll) {
            uint4 v[kPipeCopyUnroll];
#pragma unroll
            for (int u = 0; u < kPipeCopyUnroll; ++u) {
              const uint64_t j = i + (uint64_t)u * x.gstride;
              if (j < pk) v[u] = loadUserPacket<W, W>(in, (q0 + j) * N, a.count, vin);
            }
#pragma unroll
            for (int u = 0; u < kPipeCopyUnroll; ++u) {
              const uint64_t j = i + (uint64_t)u * x.gstride;
              if (j < pk) storeUserPacket<W, W>(own, (q0 + j) * N, a.count, vout, v[u]);
            }
          }
        }
        tileWait(c, 1, a.pipe_seq + k + 1, gtid, &s_abort, 1, lane);
        groupSync(3, workers);
        if (s_abort) break;
        const uint4* mine = reinterpret_cast<const uint4*>(c.stage[r]);
        for (int k2 = 1; k2 < n && cnt; ++k2) {
          const int s = (r + k2) % n;
          segCopyOut<W, W, kPipeCopyUnroll>(out + (uint64_t)s * a.out_seg_stride + q0 * N, mine + (uint64_t)s * sp + q0, cnt, x);
        }
      }
    }
  }
  // the peers' next pushes may land in these slots: nobody leaves before every peer's CTA of the same index is through
  blockBarrier(c, a.seq + 1, 3);
  callDone(c, lanes ? (tiles + lanes - 1) / lanes : 0);
}

// ------------------------------------------------------------------ broadcast
template <typename W, bool kNvls>
__global__ void __launch_bounds__(HL_NVL_THREADS) kBroadcast(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int r = c.rank;
  const Ctx x = makeCtx();
  uint4* mine = reinterpret_cast<uint4*>(c.stage[r]);
  if constexpr (kNvls) {
    if (!blockBarrier(c, a.seq + 1, 1)) return;
    if (r == a.root) {
      uint4* mc = reinterpret_cast<uint4*>(c.mc_stage);
      copyInAny<W, true>(mc, a.in, a.in_dt, 0, a.count, x);
    }
    if (!blockBarrier(c, a.seq + 2, 2)) return;
    if (r != a.root || a.out != a.in) copyOutAny<W>(a.out, a.out_dt, 0, mine, a.count, x);
    blockBarrier(c, a.seq + 3, 3);   // rule A
  } else {
    if (r == a.root) copyInAny<W>(mine, a.in, a.in_dt, 0, a.count, x);
    if (!blockBarrier(c, a.seq + 1, 1)) return;
    if (r != a.root || a.out != a.in)
      copyOutAny<W>(a.out, a.out_dt, 0, reinterpret_cast<const uint4*>(c.stage[a.root]), a.count, x);
    blockBarrier(c, a.seq + 2, 2);
  }
  callDone(c, 0);
}

// ------------------------------------------------------------------ all-to-all
// Segment q of `in` goes to rank q; segment q of `out` comes from rank q.
template <typename W>
__global__ void __launch_bounds__(HL_NVL_THREADS) kAllToAll(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const Ctx x = makeCtx();
  const uint64_t sp = (a.count + N - 1) / N;
  uint4* mine = reinterpret_cast<uint4*>(c.stage[r]);
  for (int s = 0; s < n; ++s) copyInAny<W>(mine + s * sp, a.in, a.in_dt, s * a.in_seg_stride, a.count, x);
  if (!blockBarrier(c, a.seq + 1, 1)) return;
  for (int k = 0; k < n; ++k) {
    const int q = (r + k) % n;
    copyOutAny<W>(a.out, a.out_dt, q * a.out_seg_stride, reinterpret_cast<const uint4*>(c.stage[q]) + (uint64_t)r * sp,
                  a.count, x);
  }
  blockBarrier(c, a.seq + 2, 2);
  callDone(c, 0);
}

// ------------------------------------------------------------------ zero-copy kernels on registered memory
// Buffers that the library's allocator handed out lie in a symmetric heap: same offset on every rank, every
// peer's heap mapped here, and (with NVLS) one multicast alias of all of them. These kernels read the peers'
// inputs and write the peers' outputs IN PLACE — nothing is staged, no byte is copied twice:
//   all-reduce      NVLS: multimem.ld_reduce of the owned shard straight from all ranks' inputs, scale,
//                         multimem.st straight into all ranks' outputs.
//                   P2P:  16-byte loads of the owned shard from every peer's input (ascending rank order, fp32
//                         accumulate), the result stored into every peer's output.
//   reduce-scatter  the same loads for segment `rank`, result stored locally.
//   all-gather      the local input stored into segment `rank` of every rank's output (one multimem.st, or n stores).
//   broadcast       the root stores into every rank's output.
// Protocol: announce the heap offsets of this call to every peer | barrier (every peer has entered the call: its
// input is complete and its output may be overwritten) | check that all ranks use the same offsets | the transfer |
// barrier (every store has landed; nobody still reads this rank's input). The reference reads registered user
// buffers of its peers in place as well, but only with copy-engine transfers on its PCIe path
// (pcie-ccl-cuda/src/core/process_state.cpp:329-510).
enum ZcColl { kZcAllReduce = 0, kZcReduceScatter = 1, kZcAllGather = 2, kZcBroadcast = 3 };
constexpr int kZcNvlsUnroll = 8;

__device__ __forceinline__ bool zcHandshake(const HlCommDev& c, const HlCallArgs& a) {
  const int t = threadIdx.x;
  if (t < c.nranks) {
    // plain stores: the release store of the barrier below (same thread) orders them before the flag
    volatile uint64_t* slot = c.flags[t] + HL_ZC_ARGS_WORD_OFF + 2 * c.rank;
    slot[0] = a.zc_in_off;
    slot[1] = a.zc_out_off;
  }
  if (!blockBarrier(c, a.seq + 1, 1)) return false;
  __shared__ int s_sym;
  if (t == 0) s_sym = 1;
  __syncthreads();
  if (t < c.nranks) {
    const volatile uint64_t* got = c.flags[c.rank] + HL_ZC_ARGS_WORD_OFF + 2 * t;
    if (got[0] != a.zc_in_off || got[1] != a.zc_out_off) {
      // a peer passed a buffer at another heap offset: touching anything would read or overwrite the wrong memory
      volatile uint64_t* st = c.status;
      st[1] = ((uint64_t)9 << 32) | (uint64_t)t;
      st[2] = blockIdx.x;
      st[0] = HL_DEV_ASYMMETRIC;
      *reinterpret_cast<volatile uint32_t*>(c.abort_word) = 1;
      __threadfence_system();
      s_sym = 0;
    }
  }
  __syncthreads();
  return s_sym != 0;
}

template <typename W>
__device__ __forceinline__ uint4 zcScale(uint4 v, float scale) {
  if (scale != 1.0f) {
    constexpr int N = Packet<W>::N;
    typename Wire<W>::Acc acc[N];
    Packet<W>::unpack(v, acc);
    finish<W>(acc, scale, 0);
    v = Packet<W>::pack(acc);
  }
  return v;
}

// `count` is a whole number of 16-byte packets and every buffer is 16-byte aligned (the host side sends anything
// else through the staged kernels).
template <typename W, int kColl, bool kNvls, int MR>
__global__ void __launch_bounds__(HL_NVL_THREADS) kZeroCopy(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const Ctx x = makeCtx();
  if (!zcHandshake(c, a)) return;
  const uint64_t np = a.count / N;
  if constexpr (kColl == kZcAllReduce || kColl == kZcReduceScatter) {
    // all-reduce: the owned shard of the buffer; reduce-scatter: segment r of the input
    uint64_t first, cnt;
    if constexpr (kColl == kZcAllReduce) {
      const uint64_t sp = (np + n - 1) / n;
      first = (uint64_t)r * sp;
      cnt = first >= np ? 0 : (np - first < sp ? np - first : sp);
    } else {
      first = (uint64_t)r * (a.in_seg_stride / N);
      cnt = np;
    }
    uint4* out_local = reinterpret_cast<uint4*>(a.out);
    if constexpr (kNvls) {
      const uint4* mi = reinterpret_cast<const uint4*>(c.mc_heap + a.zc_in_off) + first;
      uint4* mo = reinterpret_cast<uint4*>(c.mc_heap + a.zc_out_off) + first;
      for (uint64_t i = x.g0; i < cnt; i += x.gstride * kZcNvlsUnroll) {
        uint4 v[kZcNvlsUnroll];
#pragma unroll
        for (int u = 0; u < kZcNvlsUnroll; ++u) {
          const uint64_t j = i + (uint64_t)u * x.gstride;
          if (j < cnt) v[u] = multimemLdReduceAdd<W>(mi + j);
        }
#pragma unroll
        for (int u = 0; u < kZcNvlsUnroll; ++u) {
          const uint64_t j = i + (uint64_t)u * x.gstride;
          if (j < cnt) {
            const uint4 red = zcScale<W>(v[u], a.scale);
            if constexpr (kColl == kZcAllReduce) multimemSt(mo + j, red);
            else out_local[j] = red;
          }
        }
      }
    } else {
      constexpr int U = MR <= 2 ? 6 : (MR <= 4 ? 3 : 2);
      for (uint64_t i = x.g0; i < cnt; i += x.gstride * U) {
        uint4 v[U][MR];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint64_t j = i + (uint64_t)u * x.gstride;
          if (j < cnt) {
#pragma unroll
            for (int q = 0; q < MR; ++q)
              if (q < n) v[u][q] = (reinterpret_cast<const uint4*>(c.heap[q] + a.zc_in_off) + first)[j];
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint64_t j = i + (uint64_t)u * x.gstride;
          if (j < cnt) {
            const uint4 red = reducePackets<W, MR>(v[u], n, a.op, a.scale, a.int_div);
            if constexpr (kColl == kZcAllReduce) {
#pragma unroll
              for (int q = 0; q < MR; ++q)
                if (q < n) (reinterpret_cast<uint4*>(c.heap[(r + q) % n] + a.zc_out_off) + first)[j] = red;
            } else {
              out_local[j] = red;
            }
          }
        }
      }
    }
  } else {
    // all-gather: this rank's input goes to segment r of every output; broadcast: the root's input to every output
    const bool sender = kColl == kZcAllGather || r == a.root;
    const uint64_t seg_first = kColl == kZcAllGather ? (uint64_t)r * (a.out_seg_stride / N) : 0;
    if (sender) {
      const uint4* in = reinterpret_cast<const uint4*>(a.in);
      constexpr int U = kPushUnroll;
      for (uint64_t i = x.g0; i < np; i += x.gstride * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint64_t j = i + (uint64_t)u * x.gstride;
          if (j < np) v[u] = in[j];
        }
        if constexpr (kNvls) {
          uint4* mo = reinterpret_cast<uint4*>(c.mc_heap + a.zc_out_off) + seg_first;
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint64_t j = i + (uint64_t)u * x.gstride;
            if (j < np) multimemSt(mo + j, v[u]);
          }
        } else {
          for (int k = 0; k < n; ++k) {
            uint4* po = reinterpret_cast<uint4*>(c.heap[(r + k) % n] + a.zc_out_off) + seg_first;
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint64_t j = i + (uint64_t)u * x.gstride;
              if (j < np) po[j] = v[u];
            }
          }
        }
      }
    }
  }
  blockBarrier(c, a.seq + 2, 2);
  callDone(c, 0);
}

}  // namespace dev

// ====================================================================== host
namespace nvl {

template <typename W>
static const void* pickKernelT(int kind, int nranks) {
  using namespace dev;
  switch (kind) {
    case kNvlAllReduceOneShot: return (const void*)kAllReduceOneShot<W>;
    case kNvlAllReduceTwoShot: return (const void*)kAllReduceTwoShot<W>;
    case kNvlReduceScatter: return (const void*)kReduceScatter<W, false>;
    case kNvlAllGather: return (const void*)kAllGather<W, false>;
    case kNvlBroadcast: return (const void*)kBroadcast<W, false>;
    case kNvlAllToAll: return (const void*)kAllToAll<W>;
    case kNvlAllGatherNvls: return (const void*)kAllGather<W, true>;
    case kNvlBroadcastNvls: return (const void*)kBroadcast<W, true>;
    case kNvlAllReducePush: return (const void*)kPush<W, true>;
    case kNvlReduceScatterPush: return (const void*)kPush<W, false>;
    case kNvlAllGatherPush: return (const void*)kAllGatherPush<W>;
    case kNvlAllGatherLanes: return (const void*)kAllGatherLanes<W>;
    case kNvlAllReducePipeP2p:   // one variant per rank-count class (the unrolled source loop of the fold)
      return nranks <= 2 ? (const void*)kPipeCta<W, true, 2> : (nranks <= 4 ? (const void*)kPipeCta<W, true, 4> : (const void*)kPipeCta<W, true, HL_MAX_RANKS>);
    case kNvlReduceScatterPipeP2p:
      return nranks <= 2 ? (const void*)kPipeCta<W, false, 2> : (nranks <= 4 ? (const void*)kPipeCta<W, false, 4> : (const void*)kPipeCta<W, false, HL_MAX_RANKS>);
    case kNvlZcAllReduceP2p:
      return nranks <= 2 ? (const void*)kZeroCopy<W, kZcAllReduce, false, 2> : (nranks <= 4 ? (const void*)kZeroCopy<W, kZcAllReduce, false, 4> : (const void*)kZeroCopy<W, kZcAllReduce, false, HL_MAX_RANKS>);
    case kNvlZcReduceScatterP2p:
      return nranks <= 2 ? (const void*)kZeroCopy<W, kZcReduceScatter, false, 2> : (nranks <= 4 ? (const void*)kZeroCopy<W, kZcReduceScatter, false, 4> : (const void*)kZeroCopy<W, kZcReduceScatter, false, HL_MAX_RANKS>);
    case kNvlZcAllGatherP2p: return (const void*)kZeroCopy<W, kZcAllGather, false, 2>;
    case kNvlZcBroadcastP2p: return (const void*)kZeroCopy<W, kZcBroadcast, false, 2>;
    case kNvlZcAllGatherNvls: return (const void*)kZeroCopy<W, kZcAllGather, true, 2>;     // multimem.st moves bits: any type
    case kNvlZcBroadcastNvls: return (const void*)kZeroCopy<W, kZcBroadcast, true, 2>;
    default: break;
  }
  if constexpr (dev::IsFloatTrio<W>::value) {
    switch (kind) {
      case kNvlAllReduceNvls: return (const void*)kAllReduceNvls<W>;
      case kNvlReduceScatterNvls: return (const void*)kReduceScatter<W, true>;
      case kNvlAllReducePipeNvls: return (const void*)kPipelined<W, true, true>;
      case kNvlReduceScatterPipeNvls: return (const void*)kPipelined<W, true, false>;
      case kNvlZcAllReduceNvls: return (const void*)kZeroCopy<W, kZcAllReduce, true, 2>;
      case kNvlZcReduceScatterNvls: return (const void*)kZeroCopy<W, kZcReduceScatter, true, 2>;
      default: break;
    }
  }
  return nullptr;
}

const void* kernelFor(int kind, int wire_dt, int nranks) {
  if (kind == kNvlBarrier) return (const void*)dev::kBarrier;
  if (kind == kNvlLlAllReduce || kind == kNvlLlReduceScatter || kind == kNvlLlAllGather || kind == kNvlLlAllToAll) return lowLatencyKernelFor(kind, wire_dt);
  switch (wire_dt) {
    case hlInt8: return pickKernelT<int8_t>(kind, nranks);
    case hlUint8: return pickKernelT<uint8_t>(kind, nranks);
    case hlInt32: return pickKernelT<int32_t>(kind, nranks);
    case hlUint32: return pickKernelT<uint32_t>(kind, nranks);
    case hlInt64: return pickKernelT<long long>(kind, nranks);
    case hlUint64: return pickKernelT<unsigned long long>(kind, nranks);
    case hlFloat16: return pickKernelT<__half>(kind, nranks);
    case hlFloat32: return pickKernelT<float>(kind, nranks);
    case hlFloat64: return pickKernelT<double>(kind, nranks);
    case hlBfloat16: return pickKernelT<__nv_bfloat16>(kind, nranks);
    default: return nullptr;
  }
}

const char* kernelName(int kind) {
  switch (kind) {
    case kNvlBarrier: return "barrier";
    case kNvlAllReduceOneShot: return "allreduce_oneshot";
    case kNvlAllReduceTwoShot: return "allreduce_twoshot_p2p";
    case kNvlAllReduceNvls: return "allreduce_nvls";
    case kNvlReduceScatter: return "reducescatter_p2p";
    case kNvlReduceScatterNvls: return "reducescatter_nvls";
    case kNvlAllGather: return "allgather_p2p";
    case kNvlBroadcast: return "broadcast_p2p";
    case kNvlAllToAll: return "alltoall_p2p";
    case kNvlAllGatherNvls: return "allgather_nvls";
    case kNvlBroadcastNvls: return "broadcast_nvls";
    case kNvlAllReducePush: return "allreduce_push";
    case kNvlReduceScatterPush: return "reducescatter_push";
    case kNvlAllGatherPush: return "allgather_push";
    case kNvlAllGatherLanes: return "allgather_lanes";
    case kNvlAllReducePipeP2p: return "allreduce_pipelined_p2p";
    case kNvlAllReducePipeNvls: return "allreduce_pipelined_nvls";
    case kNvlReduceScatterPipeP2p: return "reducescatter_pipelined_p2p";
    case kNvlReduceScatterPipeNvls: return "reducescatter_pipelined_nvls";
    case kNvlZcAllReduceNvls: return "allreduce_zerocopy_nvls";
    case kNvlZcAllReduceP2p: return "allreduce_zerocopy_p2p";
    case kNvlZcReduceScatterNvls: return "reducescatter_zerocopy_nvls";
    case kNvlZcReduceScatterP2p: return "reducescatter_zerocopy_p2p";
    case kNvlZcAllGatherNvls: return "allgather_zerocopy_nvls";
    case kNvlZcAllGatherP2p: return "allgather_zerocopy_p2p";
    case kNvlZcBroadcastNvls: return "broadcast_zerocopy_nvls";
    case kNvlZcBroadcastP2p: return "broadcast_zerocopy_p2p";
    case kNvlLlAllReduce: return "allreduce_lowlatency";
    case kNvlLlReduceScatter: return "reducescatter_lowlatency";
    case kNvlLlAllGather: return "allgather_lowlatency";
    case kNvlLlAllToAll: return "alltoall_lowlatency";
    default: return "?";
  }
}

hlResult_t launch(int kind, int wire_dt, const HlCommDev* dcomms, const HlEmuCalls& calls, int emu_ranks, int blocks,
                  cudaStream_t stream, int nranks) {
  const void* fn = kernelFor(kind, wire_dt, nranks);
  if (!fn) return fail(hlUnsupported, "no %s kernel for wire type %d", kernelName(kind), wire_dt);
  if (blocks < 1) blocks = 1;
  if (blocks > HL_MAX_BLOCKS) blocks = HL_MAX_BLOCKS;
  dim3 grid((unsigned)blocks, (unsigned)(emu_ranks > 1 ? emu_ranks : 1), 1);
  const bool pipe = kind == kNvlAllReducePipeNvls || kind == kNvlReduceScatterPipeNvls;  // warp-group stages: 384 threads
  dim3 block(pipe ? dev::kPipeThreads : HL_NVL_THREADS, 1, 1);
  void* args[2] = {(void*)&dcomms, (void*)&calls};
  cudaError_t e;
  if (emu_ranks > 1) {
    // The emulated ranks wait on one another: all their blocks must be
    // co-resident, which only a cooperative launch guarantees (it fails
    // cleanly instead of deadlocking when they would not fit).
    e = cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream);
  } else {
    e = cudaLaunchKernel(fn, grid, block, args, 0, stream);
  }
  if (e != cudaSuccess) return fail(hlDeviceError, "launch of %s failed: %s", kernelName(kind), cudaGetErrorString(e));
  return hlSuccess;
}

hlResult_t prepareKernels() {
  // Resolve every variant once on the init thread: lazy module loading plus
  // concurrent first launches from several threads can deadlock in the driver
  // (same cure as pcie-ccl-cuda/kernels/wait_kernel.cu:216-234,400-432).
  static const int kinds[] = {kNvlBarrier, kNvlAllReduceOneShot, kNvlAllReduceTwoShot, kNvlAllReduceNvls,
                              kNvlReduceScatter, kNvlReduceScatterNvls, kNvlAllGather, kNvlBroadcast,
                              kNvlAllToAll, kNvlAllGatherNvls, kNvlBroadcastNvls, kNvlAllReducePipeP2p,
                              kNvlAllReducePipeNvls, kNvlReduceScatterPipeP2p, kNvlReduceScatterPipeNvls, kNvlAllReducePush,
                              kNvlReduceScatterPush, kNvlAllGatherPush, kNvlAllGatherLanes, kNvlZcAllReduceNvls,
                              kNvlZcAllReduceP2p, kNvlZcReduceScatterNvls, kNvlZcReduceScatterP2p, kNvlZcAllGatherNvls,
                              kNvlZcAllGatherP2p, kNvlZcBroadcastNvls, kNvlZcBroadcastP2p, kNvlLlAllReduce,
                              kNvlLlReduceScatter, kNvlLlAllGather, kNvlLlAllToAll};
  for (int k : kinds)
    for (int dt = 0; dt < hlNumTypes; ++dt) {
      for (int nr : {2, 4, HL_MAX_RANKS}) {   // rank-count classes (only the pipelined push kernels differ by it)
        const void* fn = kernelFor(k, dt, nr);
        if (!fn) continue;
        cudaFuncAttributes at;
        cudaError_t e = cudaFuncGetAttributes(&at, fn);
        if (e != cudaSuccess) return fail(hlDeviceError, "cudaFuncGetAttributes: %s", cudaGetErrorString(e));
      }
      if (k == kNvlBarrier) break;
    }
  return hlSuccess;
}

}  // namespace nvl
}  // namespace hl
