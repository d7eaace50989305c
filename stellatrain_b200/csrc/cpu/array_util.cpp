#include "array_util.h"

#include <immintrin.h>

#include <cmath>
#include <cstdlib>
#include <cstring>

namespace stc {

Isa best_isa() {
  static const Isa cached = [] {
    Isa isa = Isa::Scalar;
    __builtin_cpu_init();
    if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma") && __builtin_cpu_supports("f16c"))
      isa = Isa::Avx2;
    if (isa == Isa::Avx2 && __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
        __builtin_cpu_supports("avx512vl"))
      isa = Isa::Avx512;
    if (const char* cap = std::getenv("STELLATRAIN_ISA")) {
      if (!std::strcmp(cap, "scalar")) isa = Isa::Scalar;
      else if (!std::strcmp(cap, "avx2") && isa != Isa::Scalar) isa = Isa::Avx2;
    }
    return isa;
  }();
  return cached;
}

const char* isa_name(Isa isa) {
  switch (isa) {
    case Isa::Avx512: return "avx512";
    case Isa::Avx2: return "avx2";
    default: return "scalar";
  }
}

// ---------------------------------------------------------------- add
__attribute__((target("avx512f"))) static void add_avx512(float* dst, const float* a, const float* b, size_t n) {
  size_t i = 0;
  for (; i + 64 <= n; i += 64) {
    _mm512_storeu_ps(dst + i, _mm512_add_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i)));
    _mm512_storeu_ps(dst + i + 16, _mm512_add_ps(_mm512_loadu_ps(a + i + 16), _mm512_loadu_ps(b + i + 16)));
    _mm512_storeu_ps(dst + i + 32, _mm512_add_ps(_mm512_loadu_ps(a + i + 32), _mm512_loadu_ps(b + i + 32)));
    _mm512_storeu_ps(dst + i + 48, _mm512_add_ps(_mm512_loadu_ps(a + i + 48), _mm512_loadu_ps(b + i + 48)));
  }
  for (; i + 16 <= n; i += 16) _mm512_storeu_ps(dst + i, _mm512_add_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i)));
  for (; i < n; ++i) dst[i] = a[i] + b[i];
}

__attribute__((target("avx2"))) static void add_avx2(float* dst, const float* a, const float* b, size_t n) {
  size_t i = 0;
  for (; i + 32 <= n; i += 32) {
    _mm256_storeu_ps(dst + i, _mm256_add_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i)));
    _mm256_storeu_ps(dst + i + 8, _mm256_add_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8)));
    _mm256_storeu_ps(dst + i + 16, _mm256_add_ps(_mm256_loadu_ps(a + i + 16), _mm256_loadu_ps(b + i + 16)));
    _mm256_storeu_ps(dst + i + 24, _mm256_add_ps(_mm256_loadu_ps(a + i + 24), _mm256_loadu_ps(b + i + 24)));
  }
  for (; i + 8 <= n; i += 8) _mm256_storeu_ps(dst + i, _mm256_add_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i)));
  for (; i < n; ++i) dst[i] = a[i] + b[i];
}

void add_arrays_to(float* dst, const float* a, const float* b, size_t n) {
  switch (best_isa()) {
    case Isa::Avx512: add_avx512(dst, a, b, n); return;
    case Isa::Avx2: add_avx2(dst, a, b, n); return;
    default:
      for (size_t i = 0; i < n; ++i) dst[i] = a[i] + b[i];
  }
}

void add_arrays(float* dst, const float* src, size_t n) { add_arrays_to(dst, dst, src, n); }

__attribute__((target("avx512f"))) static void add_nan0_avx512(float* dst, const float* a, const float* b, size_t n) {
  size_t i = 0;
  for (; i + 16 <= n; i += 16) {
    const __m512 s = _mm512_add_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i));
    _mm512_storeu_ps(dst + i, _mm512_maskz_mov_ps(_mm512_cmp_ps_mask(s, s, _CMP_ORD_Q), s));   // NaN lanes become 0
  }
  for (; i < n; ++i) {
    const float s = a[i] + b[i];
    dst[i] = s == s ? s : 0.f;
  }
}

__attribute__((target("avx2"))) static void add_nan0_avx2(float* dst, const float* a, const float* b, size_t n) {
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 s = _mm256_add_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i));
    _mm256_storeu_ps(dst + i, _mm256_and_ps(s, _mm256_cmp_ps(s, s, _CMP_ORD_Q)));
  }
  for (; i < n; ++i) {
    const float s = a[i] + b[i];
    dst[i] = s == s ? s : 0.f;
  }
}

void add_arrays_nan_to_zero(float* dst, const float* a, const float* b, size_t n) {
  switch (best_isa()) {
    case Isa::Avx512: add_nan0_avx512(dst, a, b, n); return;
    case Isa::Avx2: add_nan0_avx2(dst, a, b, n); return;
    default:
      for (size_t i = 0; i < n; ++i) {
        const float s = a[i] + b[i];
        dst[i] = s == s ? s : 0.f;
      }
  }
}

// ---------------------------------------------------------------- block L1 norms
// The reduction tree matches the GPU kernel: ((|x0|+|x1|)+(|x2|+|x3|)) per group of four, then
// (g0+g1)+(g2+g3); scores are therefore bit-identical across tiers.
static inline float block16_l1_scalar(const float* x, size_t valid) {
  float g[4];
  for (int q = 0; q < 4; ++q) {
    float v[4];
    for (int j = 0; j < 4; ++j) {
      const size_t i = (size_t)q * 4 + j;
      v[j] = i < valid ? std::fabs(x[i]) : 0.f;
    }
    g[q] = (v[0] + v[1]) + (v[2] + v[3]);
  }
  return (g[0] + g[1]) + (g[2] + g[3]);
}

__attribute__((target("avx2"))) static void block_l1_avx2(const float* x, size_t blocks, float* out) {
  const __m256 sign = _mm256_set1_ps(-0.0f);
  for (size_t b = 0; b < blocks; ++b) {
    const __m256 lo = _mm256_andnot_ps(sign, _mm256_loadu_ps(x + 16 * b));       // x0..x7
    const __m256 hi = _mm256_andnot_ps(sign, _mm256_loadu_ps(x + 16 * b + 8));   // x8..x15
    // hadd(lo,hi): [x0+x1, x2+x3, x8+x9, x10+x11 | x4+x5, x6+x7, x12+x13, x14+x15]
    const __m256 p = _mm256_hadd_ps(lo, hi);
    // hadd(p,p): [g0, g2, g0, g2 | g1, g3, g1, g3]
    const __m256 q = _mm256_hadd_ps(p, p);
    const __m128 ql = _mm256_castps256_ps128(q), qh = _mm256_extractf128_ps(q, 1);
    const __m128 s = _mm_add_ps(ql, qh);   // [g0+g1, g2+g3, ...]
    out[b] = _mm_cvtss_f32(s) + _mm_cvtss_f32(_mm_shuffle_ps(s, s, 1));
  }
}

void block_l1_norms(const float* x, size_t n, float* out) {
  const size_t full = n / 16;
  if (best_isa() != Isa::Scalar) block_l1_avx2(x, full, out);
  else
    for (size_t b = 0; b < full; ++b) out[b] = block16_l1_scalar(x + 16 * b, 16);
  if (n % 16) out[full] = block16_l1_scalar(x + 16 * full, n % 16);
}

float max_abs(const float* x, size_t n) {
  float m = 0.f;
  for (size_t i = 0; i < n; ++i) {
    const float a = std::fabs(x[i]);
    if (a > m) m = a;
  }
  return m;
}

bool has_nan(const float* x, size_t n) {
  for (size_t i = 0; i < n; ++i)
    if (x[i] != x[i]) return true;
  return false;
}

// ---------------------------------------------------------------- casts
__attribute__((target("avx2"))) static void narrow_avx2(const uint32_t* src, uint16_t* dst, size_t n) {
  size_t i = 0;
  for (; i + 16 <= n; i += 16) {
    const __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(src + i));
    const __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(src + i + 8));
    // unsigned saturating pack; lanes come out interleaved per 128-bit half, fix with a permute
    const __m256i p = _mm256_permute4x64_epi64(_mm256_packus_epi32(a, b), 0xD8);
    _mm256_storeu_si256(reinterpret_cast<__m256i*>(dst + i), p);
  }
  for (; i < n; ++i) dst[i] = static_cast<uint16_t>(src[i]);
}

void narrow_u32_to_u16(const uint32_t* src, uint16_t* dst, size_t n) {
  if (best_isa() != Isa::Scalar) narrow_avx2(src, dst, n);
  else
    for (size_t i = 0; i < n; ++i) dst[i] = static_cast<uint16_t>(src[i]);
}

__attribute__((target("avx2"))) static void widen_avx2(const uint16_t* src, uint32_t* dst, size_t n) {
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m128i a = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i));
    _mm256_storeu_si256(reinterpret_cast<__m256i*>(dst + i), _mm256_cvtepu16_epi32(a));   // zero extension
  }
  for (; i < n; ++i) dst[i] = src[i];
}

void widen_u16_to_u32(const uint16_t* src, uint32_t* dst, size_t n) {
  if (best_isa() != Isa::Scalar) widen_avx2(src, dst, n);
  else
    for (size_t i = 0; i < n; ++i) dst[i] = src[i];
}

static inline uint16_t f32_to_f16_scalar(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = static_cast<int32_t>((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0u));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return static_cast<uint16_t>(sign | h);
  }
  uint32_t h = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return static_cast<uint16_t>(sign | h);
}

static inline float f16_to_f32_scalar(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, x;
  if (exp == 0) {
    if (man == 0) x = sign;
    else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      x = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) x = sign | 0x7f800000u | (man << 13);
  else x = sign | ((exp - 15 + 127) << 23) | (man << 13);
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

__attribute__((target("avx2,f16c"))) static void f32_to_f16_avx2(const float* src, uint16_t* dst, size_t n) {
  size_t i = 0;
  for (; i + 8 <= n; i += 8)
    _mm_storeu_si128(reinterpret_cast<__m128i*>(dst + i),
                     _mm256_cvtps_ph(_mm256_loadu_ps(src + i), _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
  for (; i < n; ++i) dst[i] = f32_to_f16_scalar(src[i]);
}

__attribute__((target("avx2,f16c"))) static void f16_to_f32_avx2(const uint16_t* src, float* dst, size_t n) {
  size_t i = 0;
  for (; i + 8 <= n; i += 8)
    _mm256_storeu_ps(dst + i, _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i))));
  for (; i < n; ++i) dst[i] = f16_to_f32_scalar(src[i]);
}

void f32_to_f16(const float* src, uint16_t* dst, size_t n) {
  if (best_isa() != Isa::Scalar) f32_to_f16_avx2(src, dst, n);
  else
    for (size_t i = 0; i < n; ++i) dst[i] = f32_to_f16_scalar(src[i]);
}

void f16_to_f32(const uint16_t* src, float* dst, size_t n) {
  if (best_isa() != Isa::Scalar) f16_to_f32_avx2(src, dst, n);
  else
    for (size_t i = 0; i < n; ++i) dst[i] = f16_to_f32_scalar(src[i]);
}

void f32_to_bf16(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    uint32_t x;
    std::memcpy(&x, src + i, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) { dst[i] = static_cast<uint16_t>((x >> 16) | 0x40u); continue; }   // NaN
    x += 0x7fffu + ((x >> 16) & 1u);
    dst[i] = static_cast<uint16_t>(x >> 16);
  }
}

void bf16_to_f32(const uint16_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    const uint32_t x = static_cast<uint32_t>(src[i]) << 16;
    std::memcpy(dst + i, &x, 4);
  }
}

}  // namespace stc
