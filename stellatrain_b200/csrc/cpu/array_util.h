// Dense array helpers of the CPU tier with run-time ISA dispatch (AVX-512F / AVX2 / scalar).
//
// The reference selects its vector paths at compile time and ships with -march=broadwell, which
// leaves its AVX-512 code unreachable (backend/CMakeLists.txt:28-29, backend/src/misc/array_util.h:12-52).
// Here every function carries target attributes and the best supported variant is picked once.
#pragma once
#include <cstddef>
#include <cstdint>

namespace stc {

enum class Isa : int { Scalar = 0, Avx2 = 1, Avx512 = 2 };
Isa best_isa();                 // highest level the running CPU supports (env STELLATRAIN_ISA caps it)
const char* isa_name(Isa isa);

// dst[i] += src[i]
void add_arrays(float* dst, const float* src, size_t n);
// dst[i] = a[i] + b[i]
void add_arrays_to(float* dst, const float* a, const float* b, size_t n);
// dst = a + b with every NaN replaced by zero (the accumulate step of error feedback: a NaN gradient is
// dropped instead of poisoning the residual).
void add_arrays_nan_to_zero(float* dst, const float* a, const float* b, size_t n);
// sum of |x[i]| over aligned blocks of 16: out[b] = sum_{j<16} |x[16 b + j]| (tail block zero padded)
void block_l1_norms(const float* x, size_t n, float* out);
float max_abs(const float* x, size_t n);
bool has_nan(const float* x, size_t n);

// Wire casts (the reference's versions are in backend/src/engine/comm_manager.cpp:487-571; its
// u32->u16 pack saturates as signed and corrupts 32768..65535, this one is unsigned).
void narrow_u32_to_u16(const uint32_t* src, uint16_t* dst, size_t n);
void widen_u16_to_u32(const uint16_t* src, uint32_t* dst, size_t n);
void f32_to_f16(const float* src, uint16_t* dst, size_t n);
void f16_to_f32(const uint16_t* src, float* dst, size_t n);
void f32_to_bf16(const float* src, uint16_t* dst, size_t n);   // round to nearest even
void bf16_to_f32(const uint16_t* src, float* dst, size_t n);

}  // namespace stc
