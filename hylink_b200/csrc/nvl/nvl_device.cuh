// Device-side building blocks of the NVLink/NVSwitch kernels (sm_100a).
//
//  * wire packets: every kernel moves 16-byte packets of the wire type W;
//    16-bit floats are widened to fp32 for the arithmetic and rounded once.
//  * user-memory accessors that convert between the caller's element type and
//    the wire type on the fly (the fused cast) and fall back to element-wise
//    access for unaligned pointers or ragged tails.
//  * the cross-GPU block barrier: block b of every rank exchanges one 8-byte
//    flag with block b of every peer through peer-mapped memory. Every wait is
//    bounded by %globaltimer; a wait that runs out records a status word and
//    the kernel returns, so no launch can spin forever.
//  * NVSwitch multimem load-reduce / store.
//
// The reference has no device-side collective code at all: its dedicated-link
// path is the vendor library (multipath-orchestrator/libampccl/backend/
// fast_backend.cc:15-25) and its only kernels are scalar element-wise reduces
// and one-thread doorbells (pcie-ccl-cuda/kernels/wait_kernel.cu:13-30,255-360).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <type_traits>

#include "hylink/hylink.h"
#include "nvl/nvl_types.h"

namespace hl {
namespace dev {

// ------------------------------------------------------------ wire types
template <typename T> struct Wire {
  using Acc = T;
  static __device__ __forceinline__ Acc up(T v) { return v; }
  static __device__ __forceinline__ T down(Acc v) { return v; }
  static constexpr bool kFloat = false;
};
template <> struct Wire<float> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(float v) { return v; }
  static __device__ __forceinline__ float down(Acc v) { return v; }
  static constexpr bool kFloat = true;
};
template <> struct Wire<double> {
  using Acc = double;
  static __device__ __forceinline__ Acc up(double v) { return v; }
  static __device__ __forceinline__ double down(Acc v) { return v; }
  static constexpr bool kFloat = true;
};
template <> struct Wire<__half> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half down(Acc v) { return __float2half_rn(v); }
  static constexpr bool kFloat = true;
};
template <> struct Wire<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ Acc up(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 down(Acc v) { return __float2bfloat16_rn(v); }
  static constexpr bool kFloat = true;
};

template <typename T> struct IsFloatTrio { static constexpr bool value = false; };
template <> struct IsFloatTrio<float> { static constexpr bool value = true; };
template <> struct IsFloatTrio<__half> { static constexpr bool value = true; };
template <> struct IsFloatTrio<__nv_bfloat16> { static constexpr bool value = true; };

template <typename A> __device__ __forceinline__ A applyOp(int op, A a, A b) {
  switch (op) {
    case hlProd: return a * b;
    case hlMax: return a > b ? a : b;
    case hlMin: return a < b ? a : b;
    default: return a + b;  // hlSum, hlAvg
  }
}

template <typename W> struct Packet {
  static constexpr int N = 16 / (int)sizeof(W);
  using Acc = typename Wire<W>::Acc;
  static __device__ __forceinline__ void unpack(const uint4& p, Acc* a) {
    alignas(16) W w[N];
    *reinterpret_cast<uint4*>(w) = p;
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = Wire<W>::up(w[i]);
  }
  static __device__ __forceinline__ uint4 pack(const Acc* a) {
    alignas(16) W w[N];
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = Wire<W>::down(a[i]);
    return *reinterpret_cast<uint4*>(w);
  }
};

// Final scaling of a reduced packet: multiply floating values by `scale`
// (1/world for an average, or a loss-scale factor), divide integers for hlAvg.
template <typename W>
__device__ __forceinline__ void finish(typename Wire<W>::Acc* a, float scale, int int_div) {
  constexpr int N = Packet<W>::N;
  if constexpr (Wire<W>::kFloat) {
    if (scale != 1.0f) {
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = (typename Wire<W>::Acc)(a[i] * (typename Wire<W>::Acc)scale);
    }
  } else {
    if (int_div > 1) {
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = (typename Wire<W>::Acc)(a[i] / (typename Wire<W>::Acc)int_div);
    }
  }
}

// ------------------------------------------------------------ conversions
template <typename D, typename S> __device__ __forceinline__ D cvt(S v) {
  if constexpr (std::is_same<D, S>::value) {
    return v;
  } else {
    return Wire<D>::down((typename Wire<D>::Acc)Wire<S>::up(v));
  }
}

// Loads the wire packet that starts at element e0 of a user segment of
// `count` elements of type S; elements past the end read as zero.
template <typename S, typename W>
__device__ __forceinline__ uint4 loadUserPacket(const S* base, uint64_t e0, uint64_t count, bool vec_ok) {
  constexpr int N = Packet<W>::N;
  alignas(16) W w[N];
  if (vec_ok && e0 + N <= count) {
    constexpr int kBytes = N * (int)sizeof(S);
    alignas(16) S s[N];
    if constexpr (kBytes == 8) {
      *reinterpret_cast<uint2*>(s) = *reinterpret_cast<const uint2*>(base + e0);
    } else if constexpr (kBytes == 16) {
      *reinterpret_cast<uint4*>(s) = *reinterpret_cast<const uint4*>(base + e0);
    } else {
      static_assert(kBytes == 32, "unexpected packet ratio");
      const uint4* p = reinterpret_cast<const uint4*>(base + e0);
      reinterpret_cast<uint4*>(s)[0] = p[0];
      reinterpret_cast<uint4*>(s)[1] = p[1];
    }
#pragma unroll
    for (int i = 0; i < N; ++i) w[i] = cvt<W, S>(s[i]);
  } else {
    *reinterpret_cast<uint4*>(w) = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (e0 + i < count) w[i] = cvt<W, S>(base[e0 + i]);
  }
  return *reinterpret_cast<uint4*>(w);
}

template <typename W, typename D>
__device__ __forceinline__ void storeUserPacket(D* base, uint64_t e0, uint64_t count, bool vec_ok, const uint4& pkt) {
  constexpr int N = Packet<W>::N;
  alignas(16) W w[N];
  *reinterpret_cast<uint4*>(w) = pkt;
  if (vec_ok && e0 + N <= count) {
    constexpr int kBytes = N * (int)sizeof(D);
    alignas(16) D d[N];
#pragma unroll
    for (int i = 0; i < N; ++i) d[i] = cvt<D, W>(w[i]);
    if constexpr (kBytes == 8) {
      *reinterpret_cast<uint2*>(base + e0) = *reinterpret_cast<uint2*>(d);
    } else if constexpr (kBytes == 16) {
      *reinterpret_cast<uint4*>(base + e0) = *reinterpret_cast<uint4*>(d);
    } else {
      static_assert(kBytes == 32, "unexpected packet ratio");
      uint4* p = reinterpret_cast<uint4*>(base + e0);
      p[0] = reinterpret_cast<uint4*>(d)[0];
      p[1] = reinterpret_cast<uint4*>(d)[1];
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (e0 + i < count) base[e0 + i] = cvt<D, W>(w[i]);
  }
}

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ------------------------------------------------------------ signalling
__device__ __forceinline__ void stReleaseSys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ldAcquireSys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Kernel timeline: thread 0 of the first HL_TL_BLOCKS CTAs records when it passes a phase boundary.
__device__ __forceinline__ void timelineStamp(const HlCommDev& c, uint64_t seq, int phase) {
  if (c.timeline != nullptr && threadIdx.x == 0 && blockIdx.x < HL_TL_BLOCKS) {
    const uint64_t slot = (seq / HL_SEQ_STRIDE) % HL_TL_CALLS;
    c.timeline[(slot * HL_TL_BLOCKS + blockIdx.x) * HL_TL_PHASES + phase] = globalTimerNs();
  }
}

// Uniform entry: a poisoned communicator (an earlier wait ran out) makes every
// later kernel a no-op instead of a second hang candidate. The call's flag
// bases are read here from device memory rather than passed by the host, so a
// launch carries no per-call counter and can be captured in a CUDA graph and
// replayed: each replay picks up where the previous launch left off.
__device__ __forceinline__ bool entryOk(const HlCommDev& c, HlCallArgs& a) {
  __shared__ int s_entry;
  __shared__ uint64_t s_seq[2];
  if (threadIdx.x == 0) {
    s_entry = (*reinterpret_cast<volatile uint32_t*>(c.abort_word) == 0) ? 1 : 0;
    s_seq[0] = reinterpret_cast<volatile uint64_t*>(c.seq_words)[0];
    s_seq[1] = reinterpret_cast<volatile uint64_t*>(c.seq_words)[1];
  }
  __syncthreads();
  a.seq = s_seq[0];
  a.pipe_seq = s_seq[1];
  if (c.timeline != nullptr && threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      uint64_t* meta = c.timeline + (size_t)HL_TL_CALLS * HL_TL_BLOCKS * HL_TL_PHASES + ((a.seq / HL_SEQ_STRIDE) % HL_TL_CALLS) * 4;
      meta[0] = a.seq;
      meta[1] = ((uint64_t)(uint32_t)a.kind << 32) | gridDim.x;
      meta[2] = a.count;
      meta[3] = 0;
    }
    timelineStamp(c, a.seq, 0);
  }
  return s_entry != 0;
}

// Normal exit of a call: the last CTA to get here advances the bases for the
// next launch. No CTA of this launch can still be about to read them: every
// CTA reads at entry and counts itself here.
__device__ __forceinline__ void callDone(const HlCommDev& c, uint64_t pipe_tiles) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (c.timeline != nullptr) timelineStamp(c, reinterpret_cast<volatile uint64_t*>(c.seq_words)[0], 7);  // still this call's base
    __threadfence();
    const unsigned long long prev = atomicAdd(reinterpret_cast<unsigned long long*>(c.seq_words + 2), 1ull);
    if (prev + 1 == gridDim.x) {
      volatile uint64_t* w = c.seq_words;
      w[2] = 0;
      w[0] = w[0] + HL_SEQ_STRIDE;
      w[1] = w[1] + pipe_tiles;
      __threadfence();
    }
  }
}

// Cross-GPU barrier of block blockIdx.x with the same block of every peer.
// `target` = seq + k for the k-th barrier of the call; flags only grow, so a
// peer that is already one barrier ahead still satisfies the test.
// Returns false (uniformly for the block) when the wait was abandoned.
__device__ __forceinline__ bool blockBarrier(const HlCommDev& c, uint64_t target, int step) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();  // also orders every thread's earlier accesses before the signal below
  if (step >= 1 && step <= 3) timelineStamp(c, target, 2 * step - 1);  // target / HL_SEQ_STRIDE == base / HL_SEQ_STRIDE
  const int t = threadIdx.x;
  if (t < c.nranks) {
    // st.release.sys orders this thread's earlier accesses — and, through the
    // bar.sync above, those of the whole CTA — before the flag; no separate
    // (sequentially consistent) fence is needed.
    uint64_t* remote = c.flags[t] + (size_t)blockIdx.x * HL_MAX_RANKS + c.rank;
    stReleaseSys(remote, target);
    const uint64_t* mine = c.flags[c.rank] + (size_t)blockIdx.x * HL_MAX_RANKS + t;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (ldAcquireSys(mine) < target) {
      if ((++spins & 31u) == 0) {
        const uint64_t now = globalTimerNs();
        if (t0 == 0) t0 = now;
        const bool aborted = *reinterpret_cast<volatile uint32_t*>(c.abort_word) != 0;
        if (aborted || now - t0 > c.timeout_ns) {
          if (!aborted) {
            volatile uint64_t* st = c.status;
            st[1] = ((uint64_t)step << 32) | (uint64_t)t;
            st[2] = blockIdx.x;
            st[0] = HL_DEV_TIMEOUT;
            *reinterpret_cast<volatile uint32_t*>(c.abort_word) = 1;
            __threadfence_system();
          }
          s_ok = 0;
          break;
        }
      }
    }
  }
  __syncthreads();
  if (step >= 1 && step <= 3) timelineStamp(c, target, 2 * step);
  return s_ok != 0;
}

// ------------------------------------------------------------ NVSwitch multimem
// Sum of the packet at the same offset of every rank bound to the multicast
// object, reduced inside the switch; 16-bit inputs accumulate in fp32.
template <typename W> __device__ __forceinline__ uint4 multimemLdReduceAdd(const void* mc);
template <> __device__ __forceinline__ uint4 multimemLdReduceAdd<float>(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
template <> __device__ __forceinline__ uint4 multimemLdReduceAdd<__nv_bfloat16>(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
template <> __device__ __forceinline__ uint4 multimemLdReduceAdd<__half>(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
// One store lands in the same offset of every rank's memory.
__device__ __forceinline__ void multimemSt(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}

}  // namespace dev
}  // namespace hl
