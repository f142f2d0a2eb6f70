#include "host/host_simd.h"

#include <immintrin.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "core/core.h"

namespace hl {

// ------------------------------------------------------------ conversions
float bf16ToFloat(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t floatToBf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float halfToFloat(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t floatToHalf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const uint32_t abs = u & 0x7fffffffu;
  if (abs > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
  if (abs >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);  // overflow -> inf (also inf)
  if (abs < 0x33000001u) return (uint16_t)sign;               // underflow -> 0
  int exp = (int)(abs >> 23) - 127;
  uint32_t man = (abs & 0x7fffffu) | 0x800000u;
  uint32_t shift, half;
  if (exp < -14) {
    shift = (uint32_t)(13 + (-14 - exp));
    half = 0;
  } else {
    shift = 13;
    half = (uint32_t)(exp + 15) << 10;
  }
  const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
  uint32_t q = man >> shift;
  if (exp >= -14) q &= 0x3ffu;
  uint32_t r = half + q;
  if (rem > halfway || (rem == halfway && (r & 1u))) ++r;
  return (uint16_t)(sign | r);
}

// ------------------------------------------------------------ dispatch level
static SimdLevel detect() {
  SimdLevel best = SimdLevel::Scalar;
#if defined(__x86_64__)
  __builtin_cpu_init();
  if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c")) best = SimdLevel::Avx2;
  if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl"))
    best = SimdLevel::Avx512;
#endif
  const char* cap = getenv("HYLINK_HOST_SIMD");
  if (cap) {
    if (!strcmp(cap, "scalar")) best = SimdLevel::Scalar;
    else if (!strcmp(cap, "avx2") && best >= SimdLevel::Avx2) best = SimdLevel::Avx2;
  }
  return best;
}
SimdLevel simdLevel() {
  static const SimdLevel l = detect();
  return l;
}
const char* simdLevelName(SimdLevel l) {
  return l == SimdLevel::Avx512 ? "avx512" : (l == SimdLevel::Avx2 ? "avx2" : "scalar");
}

// ------------------------------------------------------------ copy
#if defined(__x86_64__)
__attribute__((target("avx512f"))) static void copyNt512(char* d, const char* s, size_t n) {
  // 256 bytes per iteration, prefetch two KiB ahead, streaming stores
  while (n >= 256) {
    _mm_prefetch(s + 2048, _MM_HINT_NTA);
    __m512i a = _mm512_loadu_si512((const void*)(s));
    __m512i b = _mm512_loadu_si512((const void*)(s + 64));
    __m512i c = _mm512_loadu_si512((const void*)(s + 128));
    __m512i e = _mm512_loadu_si512((const void*)(s + 192));
    _mm512_stream_si512((__m512i*)(d), a);
    _mm512_stream_si512((__m512i*)(d + 64), b);
    _mm512_stream_si512((__m512i*)(d + 128), c);
    _mm512_stream_si512((__m512i*)(d + 192), e);
    s += 256; d += 256; n -= 256;
  }
  while (n >= 64) {
    _mm512_stream_si512((__m512i*)d, _mm512_loadu_si512((const void*)s));
    s += 64; d += 64; n -= 64;
  }
  _mm_sfence();
  if (n) memcpy(d, s, n);
}
__attribute__((target("avx2"))) static void copyNt256(char* d, const char* s, size_t n) {
  while (n >= 128) {
    _mm_prefetch(s + 1024, _MM_HINT_NTA);
    __m256i a = _mm256_loadu_si256((const __m256i*)(s));
    __m256i b = _mm256_loadu_si256((const __m256i*)(s + 32));
    __m256i c = _mm256_loadu_si256((const __m256i*)(s + 64));
    __m256i e = _mm256_loadu_si256((const __m256i*)(s + 96));
    _mm256_stream_si256((__m256i*)(d), a);
    _mm256_stream_si256((__m256i*)(d + 32), b);
    _mm256_stream_si256((__m256i*)(d + 64), c);
    _mm256_stream_si256((__m256i*)(d + 96), e);
    s += 128; d += 128; n -= 128;
  }
  _mm_sfence();
  if (n) memcpy(d, s, n);
}
#endif

void hostCopy(void* dst, const void* src, size_t bytes, bool non_temporal) {
  if (!bytes || dst == src) return;
#if defined(__x86_64__)
  if (non_temporal && bytes >= 4096) {
    char* d = (char*)dst;
    const char* s = (const char*)src;
    // streaming stores need an aligned destination: peel the head
    const size_t mis = (64 - ((uintptr_t)d & 63)) & 63;
    if (mis) {
      memcpy(d, s, mis);
      d += mis; s += mis; bytes -= mis;
    }
    if (simdLevel() == SimdLevel::Avx512) return copyNt512(d, s, bytes);
    if (simdLevel() == SimdLevel::Avx2) return copyNt256(d, s, bytes);
  }
#endif
  memcpy(dst, src, bytes);
}

// ------------------------------------------------------------ scalar reduce
template <typename T> static inline T applyOp(hlRedOp_t op, T a, T b) {
  switch (op) {
    case hlProd: return (T)(a * b);
    case hlMax: return a > b ? a : b;
    case hlMin: return a < b ? a : b;
    default: return (T)(a + b);
  }
}
template <typename T> static void reduceScalar(T* d, const T* a, const T* b, size_t n, hlRedOp_t op) {
  for (size_t i = 0; i < n; ++i) d[i] = applyOp<T>(op, a[i], b[i]);
}
static void reduceScalarBf16(uint16_t* d, const uint16_t* a, const uint16_t* b, size_t n, hlRedOp_t op) {
  for (size_t i = 0; i < n; ++i) d[i] = floatToBf16(applyOp<float>(op, bf16ToFloat(a[i]), bf16ToFloat(b[i])));
}
static void reduceScalarHalf(uint16_t* d, const uint16_t* a, const uint16_t* b, size_t n, hlRedOp_t op) {
  for (size_t i = 0; i < n; ++i) d[i] = floatToHalf(applyOp<float>(op, halfToFloat(a[i]), halfToFloat(b[i])));
}

#if defined(__x86_64__)
// ------------------------------------------------------------ AVX-512
#define HL_T512 __attribute__((target("avx512f,avx512bw,avx512vl,avx512dq")))
HL_T512 static inline __m512 op512(hlRedOp_t op, __m512 x, __m512 y) {
  switch (op) {
    case hlProd: return _mm512_mul_ps(x, y);
    case hlMax: return _mm512_max_ps(x, y);
    case hlMin: return _mm512_min_ps(x, y);
    default: return _mm512_add_ps(x, y);
  }
}
HL_T512 static void reduceF32_512(float* d, const float* a, const float* b, size_t n, hlRedOp_t op) {
  size_t i = 0;
  for (; i + 64 <= n; i += 64) {
    _mm_prefetch((const char*)(a + i) + 2048, _MM_HINT_NTA);
    _mm_prefetch((const char*)(b + i) + 2048, _MM_HINT_NTA);
    __m512 r0 = op512(op, _mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i));
    __m512 r1 = op512(op, _mm512_loadu_ps(a + i + 16), _mm512_loadu_ps(b + i + 16));
    __m512 r2 = op512(op, _mm512_loadu_ps(a + i + 32), _mm512_loadu_ps(b + i + 32));
    __m512 r3 = op512(op, _mm512_loadu_ps(a + i + 48), _mm512_loadu_ps(b + i + 48));
    _mm512_storeu_ps(d + i, r0);
    _mm512_storeu_ps(d + i + 16, r1);
    _mm512_storeu_ps(d + i + 32, r2);
    _mm512_storeu_ps(d + i + 48, r3);
  }
  for (; i + 16 <= n; i += 16) _mm512_storeu_ps(d + i, op512(op, _mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i)));
  if (i < n) {
    const __mmask16 m = (__mmask16)((1u << (n - i)) - 1);
    _mm512_mask_storeu_ps(d + i, m, op512(op, _mm512_maskz_loadu_ps(m, a + i), _mm512_maskz_loadu_ps(m, b + i)));
  }
}
HL_T512 static void reduceF64_512(double* d, const double* a, const double* b, size_t n, hlRedOp_t op) {
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    __m512d x = _mm512_loadu_pd(a + i), y = _mm512_loadu_pd(b + i), r;
    switch (op) {
      case hlProd: r = _mm512_mul_pd(x, y); break;
      case hlMax: r = _mm512_max_pd(x, y); break;
      case hlMin: r = _mm512_min_pd(x, y); break;
      default: r = _mm512_add_pd(x, y); break;
    }
    _mm512_storeu_pd(d + i, r);
  }
  reduceScalar<double>(d + i, a + i, b + i, n - i, op);
}
HL_T512 static void reduceI32_512(int32_t* d, const int32_t* a, const int32_t* b, size_t n, hlRedOp_t op) {
  size_t i = 0;
  for (; i + 16 <= n; i += 16) {
    __m512i x = _mm512_loadu_si512(a + i), y = _mm512_loadu_si512(b + i), r;
    switch (op) {
      case hlProd: r = _mm512_mullo_epi32(x, y); break;
      case hlMax: r = _mm512_max_epi32(x, y); break;
      case hlMin: r = _mm512_min_epi32(x, y); break;
      default: r = _mm512_add_epi32(x, y); break;
    }
    _mm512_storeu_si512(d + i, r);
  }
  reduceScalar<int32_t>(d + i, a + i, b + i, n - i, op);
}
HL_T512 static inline __m512 bf16x16ToF32(__m256i v) { return _mm512_castsi512_ps(_mm512_slli_epi32(_mm512_cvtepu16_epi32(v), 16)); }
HL_T512 static inline __m256i f32ToBf16x16(__m512 f) {
  const __m512i u = _mm512_castps_si512(f);
  const __m512i lsb = _mm512_and_si512(_mm512_srli_epi32(u, 16), _mm512_set1_epi32(1));
  __m512i r = _mm512_srli_epi32(_mm512_add_epi32(u, _mm512_add_epi32(lsb, _mm512_set1_epi32(0x7fff))), 16);
  // NaN stays NaN (the rounding add could carry it into infinity's encoding)
  const __mmask16 nan = _mm512_cmp_ps_mask(f, f, _CMP_UNORD_Q);
  r = _mm512_mask_mov_epi32(r, nan, _mm512_or_si512(_mm512_srli_epi32(u, 16), _mm512_set1_epi32(0x40)));
  return _mm512_cvtepi32_epi16(r);
}
HL_T512 static void reduceBf16_512(uint16_t* d, const uint16_t* a, const uint16_t* b, size_t n, hlRedOp_t op) {
  size_t i = 0;
  for (; i + 32 <= n; i += 32) {
    _mm_prefetch((const char*)(a + i) + 1024, _MM_HINT_NTA);
    _mm_prefetch((const char*)(b + i) + 1024, _MM_HINT_NTA);
    __m512 r0 = op512(op, bf16x16ToF32(_mm256_loadu_si256((const __m256i*)(a + i))), bf16x16ToF32(_mm256_loadu_si256((const __m256i*)(b + i))));
    __m512 r1 = op512(op, bf16x16ToF32(_mm256_loadu_si256((const __m256i*)(a + i + 16))), bf16x16ToF32(_mm256_loadu_si256((const __m256i*)(b + i + 16))));
    _mm256_storeu_si256((__m256i*)(d + i), f32ToBf16x16(r0));
    _mm256_storeu_si256((__m256i*)(d + i + 16), f32ToBf16x16(r1));
  }
  for (; i + 16 <= n; i += 16) {
    __m512 r = op512(op, bf16x16ToF32(_mm256_loadu_si256((const __m256i*)(a + i))), bf16x16ToF32(_mm256_loadu_si256((const __m256i*)(b + i))));
    _mm256_storeu_si256((__m256i*)(d + i), f32ToBf16x16(r));
  }
  reduceScalarBf16(d + i, a + i, b + i, n - i, op);
}
HL_T512 static void reduceHalf_512(uint16_t* d, const uint16_t* a, const uint16_t* b, size_t n, hlRedOp_t op) {
  size_t i = 0;
  for (; i + 16 <= n; i += 16) {
    __m512 x = _mm512_cvtph_ps(_mm256_loadu_si256((const __m256i*)(a + i)));
    __m512 y = _mm512_cvtph_ps(_mm256_loadu_si256((const __m256i*)(b + i)));
    _mm256_storeu_si256((__m256i*)(d + i), _mm512_cvtps_ph(op512(op, x, y), _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
  }
  reduceScalarHalf(d + i, a + i, b + i, n - i, op);
}

// ------------------------------------------------------------ AVX2
#define HL_T256 __attribute__((target("avx2,fma,f16c")))
HL_T256 static inline __m256 op256(hlRedOp_t op, __m256 x, __m256 y) {
  switch (op) {
    case hlProd: return _mm256_mul_ps(x, y);
    case hlMax: return _mm256_max_ps(x, y);
    case hlMin: return _mm256_min_ps(x, y);
    default: return _mm256_add_ps(x, y);
  }
}
HL_T256 static void reduceF32_256(float* d, const float* a, const float* b, size_t n, hlRedOp_t op) {
  size_t i = 0;
  for (; i + 8 <= n; i += 8) _mm256_storeu_ps(d + i, op256(op, _mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i)));
  reduceScalar<float>(d + i, a + i, b + i, n - i, op);
}
HL_T256 static void reduceHalf_256(uint16_t* d, const uint16_t* a, const uint16_t* b, size_t n, hlRedOp_t op) {
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    __m256 x = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(a + i)));
    __m256 y = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(b + i)));
    _mm_storeu_si128((__m128i*)(d + i), _mm256_cvtps_ph(op256(op, x, y), _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
  }
  reduceScalarHalf(d + i, a + i, b + i, n - i, op);
}
#endif  // __x86_64__

bool hostReduce(void* dst, const void* a, const void* b, size_t n, hlDataType_t t, hlRedOp_t op, int level_cap) {
  if ((int)op < 0 || op >= hlNumOps) return false;
  SimdLevel lv = simdLevel();
  if (level_cap >= 0 && level_cap < (int)lv) lv = (SimdLevel)level_cap;
  if (!Config::get().host_reduce_simd) lv = SimdLevel::Scalar;
  switch (t) {
    case hlFloat32:
#if defined(__x86_64__)
      if (lv == SimdLevel::Avx512) return reduceF32_512((float*)dst, (const float*)a, (const float*)b, n, op), true;
      if (lv == SimdLevel::Avx2) return reduceF32_256((float*)dst, (const float*)a, (const float*)b, n, op), true;
#endif
      return reduceScalar<float>((float*)dst, (const float*)a, (const float*)b, n, op), true;
    case hlFloat64:
#if defined(__x86_64__)
      if (lv == SimdLevel::Avx512) return reduceF64_512((double*)dst, (const double*)a, (const double*)b, n, op), true;
#endif
      return reduceScalar<double>((double*)dst, (const double*)a, (const double*)b, n, op), true;
    case hlBfloat16:
#if defined(__x86_64__)
      if (lv == SimdLevel::Avx512) return reduceBf16_512((uint16_t*)dst, (const uint16_t*)a, (const uint16_t*)b, n, op), true;
#endif
      return reduceScalarBf16((uint16_t*)dst, (const uint16_t*)a, (const uint16_t*)b, n, op), true;
    case hlFloat16:
#if defined(__x86_64__)
      if (lv == SimdLevel::Avx512) return reduceHalf_512((uint16_t*)dst, (const uint16_t*)a, (const uint16_t*)b, n, op), true;
      if (lv == SimdLevel::Avx2) return reduceHalf_256((uint16_t*)dst, (const uint16_t*)a, (const uint16_t*)b, n, op), true;
#endif
      return reduceScalarHalf((uint16_t*)dst, (const uint16_t*)a, (const uint16_t*)b, n, op), true;
    case hlInt32:
#if defined(__x86_64__)
      if (lv == SimdLevel::Avx512) return reduceI32_512((int32_t*)dst, (const int32_t*)a, (const int32_t*)b, n, op), true;
#endif
      return reduceScalar<int32_t>((int32_t*)dst, (const int32_t*)a, (const int32_t*)b, n, op), true;
    case hlUint32: return reduceScalar<uint32_t>((uint32_t*)dst, (const uint32_t*)a, (const uint32_t*)b, n, op), true;
    case hlInt64: return reduceScalar<int64_t>((int64_t*)dst, (const int64_t*)a, (const int64_t*)b, n, op), true;
    case hlUint64: return reduceScalar<uint64_t>((uint64_t*)dst, (const uint64_t*)a, (const uint64_t*)b, n, op), true;
    case hlInt8: return reduceScalar<int8_t>((int8_t*)dst, (const int8_t*)a, (const int8_t*)b, n, op), true;
    case hlUint8: return reduceScalar<uint8_t>((uint8_t*)dst, (const uint8_t*)a, (const uint8_t*)b, n, op), true;
    default: return false;
  }
}

bool hostScale(void* dst, size_t n, hlDataType_t t, double scale) {
  switch (t) {
    case hlFloat32: { float* p = (float*)dst; const float s = (float)scale; for (size_t i = 0; i < n; ++i) p[i] *= s; return true; }
    case hlFloat64: { double* p = (double*)dst; for (size_t i = 0; i < n; ++i) p[i] *= scale; return true; }
    case hlBfloat16: { uint16_t* p = (uint16_t*)dst; const float s = (float)scale; for (size_t i = 0; i < n; ++i) p[i] = floatToBf16(bf16ToFloat(p[i]) * s); return true; }
    case hlFloat16: { uint16_t* p = (uint16_t*)dst; const float s = (float)scale; for (size_t i = 0; i < n; ++i) p[i] = floatToHalf(halfToFloat(p[i]) * s); return true; }
    default: return false;
  }
}

}  // namespace hl

extern "C" {
// ctypes entry points for tests and benchmarks
int hlHostReduce(void* dst, const void* a, const void* b, size_t count, int dtype, int op, int level_cap) {
  return hl::hostReduce(dst, a, b, count, (hlDataType_t)dtype, (hlRedOp_t)op, level_cap) ? 0 : 1;
}
void hlHostCopy(void* dst, const void* src, size_t bytes, int non_temporal) { hl::hostCopy(dst, src, bytes, non_temporal != 0); }
int hlHostSimdLevel(void) { return (int)hl::simdLevel(); }
}
