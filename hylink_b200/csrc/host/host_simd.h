// Host-side copy and reduction kernels of the PCIe path.
//
// hostCopy: streaming (non-temporal) or cached memcpy, AVX-512 / AVX2 / scalar
// chosen at run time. hostReduce: three-address dst = op(a, b) for all ten
// element types and sum / prod / max / min; fp16 and bf16 are widened to fp32,
// combined and rounded to nearest-even once — the same arithmetic as the
// device kernels, so host-reduced and device-reduced schedules agree bitwise.
//
// Parity: pcie-ccl-cuda/src/hal/host_rt.hpp:45-61 with
// impl/avx512_host_rt_impl.hpp:18-198 provides float-only SIMD copy/reduce and
// the engine itself reduces with a scalar loop that rejects fp16/bf16
// (src/executor/h2h_engine.cpp:35-89).
#pragma once
#include <cstddef>
#include <cstdint>

#include "hylink/hylink.h"

namespace hl {

enum class SimdLevel { Scalar = 0, Avx2 = 1, Avx512 = 2 };
SimdLevel simdLevel();               // best level the CPU supports (HYLINK_HOST_SIMD=scalar|avx2|avx512 caps it)
const char* simdLevelName(SimdLevel l);

void hostCopy(void* dst, const void* src, size_t bytes, bool non_temporal);
// Returns false for an unknown dtype/op pair. `level_cap` < 0: use simdLevel().
bool hostReduce(void* dst, const void* a, const void* b, size_t count, hlDataType_t t, hlRedOp_t op, int level_cap = -1);
// dst *= scale for floating types (used for hlAvg and fused scaling on the host path).
bool hostScale(void* dst, size_t count, hlDataType_t t, double scale);

// software conversions (round to nearest even), exposed for tests
float bf16ToFloat(uint16_t v);
uint16_t floatToBf16(float f);
float halfToFloat(uint16_t v);
uint16_t floatToHalf(float f);

}  // namespace hl
