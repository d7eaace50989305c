// Vectorised xorshift128+ generators for random-k sampling.  Same role as the reference's
// backend/src/misc/simdxorshift128plus.{c,h} (4 lanes with AVX2, 8 with AVX-512); written here as
// a plain lane array that the compiler vectorises, plus a scalar generator and bounded sampling.
#pragma once
#include <cstddef>
#include <cstdint>

namespace stc {

struct XorShift128Plus {
  uint64_t s0, s1;
  explicit XorShift128Plus(uint64_t seed);
  uint64_t next();
  void jump();                           // advance by 2^64 calls: independent sub-streams
  uint32_t bounded(uint32_t bound);      // unbiased value in [0, bound)
};

template <int Lanes>
struct XorShift128PlusLanes {
  uint64_t s0[Lanes], s1[Lanes];
  explicit XorShift128PlusLanes(uint64_t seed);
  void next(uint64_t* out);              // Lanes results
};

extern template struct XorShift128PlusLanes<4>;
extern template struct XorShift128PlusLanes<8>;

// k distinct indices out of [0, n) by partial Fisher-Yates on a virtual array (k << n friendly).
void sample_without_replacement(uint32_t n, uint32_t k, uint64_t seed, uint32_t* out);
// Fisher-Yates shuffle of an index array.
void shuffle_u32(uint32_t* data, size_t n, uint64_t seed);

}  // namespace stc
