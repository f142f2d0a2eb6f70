// Low-latency kernels of the dedicated-link path for small messages: all-reduce, reduce-scatter, all-gather and
// all-to-all with NO cross-GPU barrier at all.
//
// The barrier-based kernels (nvl_kernels.cu) pay two flag round trips per call — about 3 to 8 microseconds each
// once the stores in front of them have to be acknowledged — which is most of the time of a message of a few MiB.
// Here every 16-byte store carries its own arrival flag: 8 data bytes and two copies of a 32-bit call tag
// ({d0, tag, d1, tag}, one st.volatile.v4, so each 8-byte half validates itself), written straight into the
// receiver's low-latency region; the receiver spins on the packet itself until all tags match. One network
// traversal per hop, no fence, no second trip. The price is half the link bandwidth, so the host side uses these
// kernels only while latency decides (measured limits in NvlPath::lowLatencyChoice). An all-reduce in the case
// of np < n packets still ends only after some shard owner heard from every rank, which keeps the argument below.
//
// Region (per rank, behind the flag words of the symmetric region): [2 parities][2 phases][HL_MAX_RANKS sources]
// slots of ll_slot_bytes. A call uses the parity of its call index, so the slots it writes were last used two calls
// ago. That reuse is safe without any handshake: in each of these collectives every rank receives from every other
// rank (directly, or through a shard owner that did), so a rank can only FINISH call k+1 after every peer has
// STARTED sending in call k+1, i.e. after every peer has left call k (launches of one communicator are
// stream-ordered); barrier-based kernels in between synchronise all ranks anyway. The tag is the call index + 1 (never 0, the value of cleared memory) and differs from the tag
// that the same slot held two calls earlier.
//
// all-to-all:      send segment q to rank q       | receive segment s from rank s into slot s of the output
// all-gather:      send own segment to every peer | receive the others' segments into the output
// reduce-scatter:  send segment q to rank q       | receive n-1 contributions, add in rank order, store
// all-reduce:      reduce-scatter of the n shards (phase 0), then all-gather of the reduced shards (phase 1)
//
// Buffers: any device memory, any alignment, any element count; no type conversion. Sum order is by rank index on every rank: results are bitwise identical
// across ranks and runs.
//
// The reference has no kernels of its own on this path (it calls the vendor library:
// multipath-orchestrator/libampccl/core/virtual_collective.h:246-252); the protocol is the classic flag-in-data
// scheme of vendor collective libraries, written here from its description.
#include <cuda_runtime.h>

#include "nvl/nvl_device.cuh"
#include "nvl/nvl_launch.h"

namespace hl {
namespace dev {

constexpr int kLlAllReduce = 0, kLlReduceScatter = 1, kLlAllGather = 2, kLlAllToAll = 3;

__device__ __forceinline__ uint8_t* llSlot(const HlCommDev& c, int owner, int parity, int phase, int src) {
  return c.ll[owner] + ((size_t)((parity * 2 + phase) * HL_MAX_RANKS + src)) * c.ll_slot_bytes;
}

// One 16-byte data packet = two flagged 16-byte stores. Packets are laid out in groups of 32 (one warp): the 32
// first halves side by side (512 bytes), then the 32 second halves, so that each of the two store instructions of
// a warp — and each of the two polling loads — covers 512 contiguous bytes instead of every other 16.
__device__ __forceinline__ uint64_t llOffset(uint64_t j) { return (j >> 5) * 1024 + (j & 31) * 16; }

__device__ __forceinline__ void llSend(uint8_t* slot, uint64_t j, const uint4& v, uint32_t tag) {
  uint8_t* p = slot + llOffset(j);
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(tag), "r"(v.y), "r"(tag) : "memory");
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p + 512), "r"(v.z), "r"(tag), "r"(v.w), "r"(tag) : "memory");
}

struct LlWait {
  uint64_t t0;
  bool ok;
};

// Spins until both halves of packet j carry the tag. Bounded: after timeout_ns (or when the communicator is
// poisoned) it records where it gave up, poisons the communicator and returns false; the caller leaves the kernel.
__device__ __forceinline__ bool llRecv(const HlCommDev& c, const uint8_t* slot, uint64_t j, uint32_t tag, int src, LlWait& w, uint4* out) {
  const uint8_t* p = slot + llOffset(j);
  uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
  uint32_t spins = 0;
  for (;;) {
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "l"(p) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "l"(p + 512) : "memory");
    if (a1 == tag && a3 == tag && b1 == tag && b3 == tag) break;
    // a late peer (milliseconds, when the call overlaps with compute) must not have thousands of threads hammer L2
    // (an ordinary wait is a handful of polls and never gets here)
    if (++spins > 64) __nanosleep(spins > 1024 ? 400 : 50);
    if ((spins & 63u) == 0) {
      const uint64_t now = globalTimerNs();
      if (w.t0 == 0) w.t0 = now;
      const bool aborted = *reinterpret_cast<volatile uint32_t*>(c.abort_word) != 0;
      if (aborted || now - w.t0 > c.timeout_ns) {
        if (!aborted) {
          volatile uint64_t* st = c.status;
          st[1] = ((uint64_t)8 << 32) | (uint64_t)src;   // step 8: a low-latency packet that never arrived
          st[2] = blockIdx.x;
          st[0] = HL_DEV_TIMEOUT;
          *reinterpret_cast<volatile uint32_t*>(c.abort_word) = 1;
          __threadfence_system();
        }
        w.ok = false;
        return false;
      }
    }
  }
  *out = make_uint4(a0, a2, b0, b2);
  return true;
}

template <typename W>
__device__ __forceinline__ uint4 llReduce(const uint4* v, int n, int op, float scale, int int_div) {
  constexpr int N = Packet<W>::N;
  typename Wire<W>::Acc acc[N], b[N];
  Packet<W>::unpack(v[0], acc);
#pragma unroll
  for (int q = 1; q < HL_MAX_RANKS; ++q) {
    if (q < n) {
      Packet<W>::unpack(v[q], b);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = applyOp(op, acc[i], b[i]);
    }
  }
  finish<W>(acc, scale, int_div);
  return Packet<W>::pack(acc);
}

// `count`: elements of the whole buffer (all-reduce) or of one segment (the others). User buffers may have any
// alignment and any element count: packets are loaded and stored through loadUserPacket / storeUserPacket (vector
// accesses when the segment is 16-byte aligned and the packet whole, element by element otherwise; lanes past the
// end travel as zeros and are never stored). Whether a call takes these kernels therefore depends on sizes and
// types only, which are the same on every rank - never on a pointer, which need not be.
// Every thread keeps the same packet indices in every loop of the kernel, which is what makes the in-place forms
// safe (a location is read by the thread that later overwrites it, earlier in program order).
template <typename W, int kColl>
__global__ void __launch_bounds__(HL_NVL_THREADS) kLowLatency(const HlCommDev* comms, HlEmuCalls calls) {
  const HlCommDev& c = comms[blockIdx.y];
  HlCallArgs a = calls.c[blockIdx.y];
  if (!entryOk(c, a)) return;
  constexpr int N = Packet<W>::N;
  const int n = c.nranks, r = c.rank;
  const uint64_t g0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, gstride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t call = a.seq / HL_SEQ_STRIDE;
  const uint32_t tag = (uint32_t)(call % 0xfffffffeull) + 1u;
  const int parity = (int)(call & 1);
  const W* in = reinterpret_cast<const W*>(a.in);
  W* out = reinterpret_cast<W*>(a.out);
  const uint64_t cnt = a.count;
  const uint64_t np = (cnt + N - 1) / N;
  // packet j of the segment that starts at element `base` of a buffer
  auto ld = [&](const W* seg, uint64_t j) { return loadUserPacket<W, W>(seg, j * N, cnt, aligned16(seg)); };
  auto st = [&](W* seg, uint64_t j, const uint4& v) { storeUserPacket<W, W>(seg, j * N, cnt, aligned16(seg), v); };
  LlWait w;
  w.t0 = 0;
  w.ok = true;
  if constexpr (kColl == kLlAllGather) {
    for (uint64_t j = g0; j < np; j += gstride) {
      const uint4 v = ld(in, j);
      for (int k = 1; k < n; ++k) llSend(llSlot(c, (r + k) % n, parity, 0, r), j, v, tag);
      st(out + (uint64_t)r * a.out_seg_stride, j, v);
    }
    for (uint64_t j = g0; j < np && w.ok; j += gstride)
      for (int k = 1; k < n; ++k) {
        const int s = (r + n - k) % n;
        uint4 v;
        if (!llRecv(c, llSlot(c, r, parity, 0, s), j, tag, s, w, &v)) break;
        st(out + (uint64_t)s * a.out_seg_stride, j, v);
      }
  } else if constexpr (kColl == kLlAllToAll) {
    for (uint64_t j = g0; j < np; j += gstride) {
      uint4 own;
      for (int k = 0; k < n; ++k) {
        const int q = (r + k) % n;
        const uint4 v = ld(in + (uint64_t)q * a.in_seg_stride, j);
        if (k == 0) own = v;
        else llSend(llSlot(c, q, parity, 0, r), j, v, tag);
      }
      st(out + (uint64_t)r * a.out_seg_stride, j, own);   // after every read of this thread's column: in place is safe
    }
    for (uint64_t j = g0; j < np && w.ok; j += gstride)
      for (int k = 1; k < n; ++k) {
        const int s = (r + n - k) % n;
        uint4 v;
        if (!llRecv(c, llSlot(c, r, parity, 0, s), j, tag, s, w, &v)) break;
        st(out + (uint64_t)s * a.out_seg_stride, j, v);
      }
  } else if constexpr (kColl == kLlReduceScatter) {
    for (uint64_t j = g0; j < np; j += gstride)
      for (int k = 1; k < n; ++k) {
        const int q = (r + k) % n;
        llSend(llSlot(c, q, parity, 0, r), j, ld(in + (uint64_t)q * a.in_seg_stride, j), tag);
      }
    for (uint64_t j = g0; j < np && w.ok; j += gstride) {
      uint4 v[HL_MAX_RANKS];   // indexed by compile-time constants only: stays in registers
#pragma unroll
      for (int q = 0; q < HL_MAX_RANKS; ++q)
        if (q < n) {
          if (q == r) v[q] = ld(in + (uint64_t)r * a.in_seg_stride, j);
          else if (w.ok) llRecv(c, llSlot(c, r, parity, 0, q), j, tag, q, w, &v[q]);
        }
      if (!w.ok) break;
      st(out, j, llReduce<W>(v, n, a.op, a.scale, a.int_div));
    }
  } else {
    // shard q = packets [q * sp, min(np, (q + 1) * sp)) of the whole buffer; rank q reduces it
    const uint64_t sp = (np + n - 1) / n;
    const uint64_t first = (uint64_t)r * sp;
    const uint64_t mine = first >= np ? 0 : (np - first < sp ? np - first : sp);
    for (uint64_t j = g0; j < sp; j += gstride)
      for (int k = 1; k < n; ++k) {
        const int q = (r + k) % n;
        const uint64_t e = (uint64_t)q * sp + j;
        if (e < np) llSend(llSlot(c, q, parity, 0, r), j, ld(in, e), tag);
      }
    for (uint64_t j = g0; j < mine && w.ok; j += gstride) {
      uint4 v[HL_MAX_RANKS];
#pragma unroll
      for (int q = 0; q < HL_MAX_RANKS; ++q)
        if (q < n) {
          if (q == r) v[q] = ld(in, first + j);
          else if (w.ok) llRecv(c, llSlot(c, r, parity, 0, q), j, tag, q, w, &v[q]);
        }
      if (!w.ok) break;
      const uint4 red = llReduce<W>(v, n, a.op, a.scale, a.int_div);
      for (int k = 1; k < n; ++k) llSend(llSlot(c, (r + k) % n, parity, 1, r), j, red, tag);
      st(out, first + j, red);
    }
    for (uint64_t j = g0; j < sp && w.ok; j += gstride)
      for (int k = 1; k < n; ++k) {
        const int s = (r + n - k) % n;
        const uint64_t e = (uint64_t)s * sp + j;
        if (e >= np) continue;
        uint4 v;
        if (!llRecv(c, llSlot(c, r, parity, 1, s), j, tag, s, w, &v)) break;
        st(out, e, v);
      }
  }
  // a thread that gave up has poisoned the communicator; the others find the abort word in their own waits
  callDone(c, 0);
}

}  // namespace dev

namespace nvl {

template <typename W>
static const void* pickLl(int kind) {
  using namespace dev;
  switch (kind) {
    case kNvlLlAllReduce: return (const void*)kLowLatency<W, kLlAllReduce>;
    case kNvlLlReduceScatter: return (const void*)kLowLatency<W, kLlReduceScatter>;
    case kNvlLlAllGather: return (const void*)kLowLatency<W, kLlAllGather>;
    case kNvlLlAllToAll: return (const void*)kLowLatency<W, kLlAllToAll>;
    default: return nullptr;
  }
}

const void* lowLatencyKernelFor(int kind, int wire_dt) {
  switch (wire_dt) {
    case hlInt8: return pickLl<int8_t>(kind);
    case hlUint8: return pickLl<uint8_t>(kind);
    case hlInt32: return pickLl<int32_t>(kind);
    case hlUint32: return pickLl<uint32_t>(kind);
    case hlInt64: return pickLl<long long>(kind);
    case hlUint64: return pickLl<unsigned long long>(kind);
    case hlFloat16: return pickLl<__half>(kind);
    case hlFloat32: return pickLl<float>(kind);
    case hlFloat64: return pickLl<double>(kind);
    case hlBfloat16: return pickLl<__nv_bfloat16>(kind);
    default: return nullptr;
  }
}

}  // namespace nvl
}  // namespace hl
