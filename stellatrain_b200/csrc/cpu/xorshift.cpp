#include "xorshift.h"

#include <unordered_map>
#include <utility>

namespace stc {

static inline uint64_t splitmix64(uint64_t& x) {
  uint64_t z = (x += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

XorShift128Plus::XorShift128Plus(uint64_t seed) {
  s0 = splitmix64(seed);
  s1 = splitmix64(seed);
  if ((s0 | s1) == 0) s1 = 1;
}

uint64_t XorShift128Plus::next() {
  uint64_t a = s0;
  const uint64_t b = s1;
  s0 = b;
  a ^= a << 23;
  s1 = a ^ b ^ (a >> 18) ^ (b >> 5);
  return s1 + b;
}

void XorShift128Plus::jump() {
  static const uint64_t kJump[2] = {0x8a5cd789635d2dffull, 0x121fd2155c472f96ull};
  uint64_t j0 = 0, j1 = 0;
  for (int i = 0; i < 2; ++i)
    for (int b = 0; b < 64; ++b) {
      if (kJump[i] & (1ull << b)) { j0 ^= s0; j1 ^= s1; }
      next();
    }
  s0 = j0;
  s1 = j1;
}

uint32_t XorShift128Plus::bounded(uint32_t bound) {
  // Lemire's multiply-shift with rejection of the biased zone
  uint64_t m = (next() >> 32) * static_cast<uint64_t>(bound);
  uint32_t low = static_cast<uint32_t>(m);
  if (low < bound) {
    const uint32_t thresh = (0u - bound) % bound;
    while (low < thresh) {
      m = (next() >> 32) * static_cast<uint64_t>(bound);
      low = static_cast<uint32_t>(m);
    }
  }
  return static_cast<uint32_t>(m >> 32);
}

template <int Lanes>
XorShift128PlusLanes<Lanes>::XorShift128PlusLanes(uint64_t seed) {
  XorShift128Plus g(seed);
  for (int l = 0; l < Lanes; ++l) {
    s0[l] = g.s0;
    s1[l] = g.s1;
    g.jump();
  }
}

template <int Lanes>
void XorShift128PlusLanes<Lanes>::next(uint64_t* out) {
  for (int l = 0; l < Lanes; ++l) {   // straight-line per lane: auto-vectorised
    uint64_t a = s0[l];
    const uint64_t b = s1[l];
    s0[l] = b;
    a ^= a << 23;
    s1[l] = a ^ b ^ (a >> 18) ^ (b >> 5);
    out[l] = s1[l] + b;
  }
}

template struct XorShift128PlusLanes<4>;
template struct XorShift128PlusLanes<8>;

void sample_without_replacement(uint32_t n, uint32_t k, uint64_t seed, uint32_t* out) {
  XorShift128Plus g(seed);
  std::unordered_map<uint32_t, uint32_t> moved;   // sparse view of the partially shuffled identity array
  moved.reserve(static_cast<size_t>(k) * 2);
  for (uint32_t i = 0; i < k; ++i) {
    const uint32_t j = i + g.bounded(n - i);
    auto itj = moved.find(j);
    const uint32_t vj = itj == moved.end() ? j : itj->second;
    auto iti = moved.find(i);
    const uint32_t vi = iti == moved.end() ? i : iti->second;
    out[i] = vj;
    moved[j] = vi;
  }
}

void shuffle_u32(uint32_t* data, size_t n, uint64_t seed) {
  XorShift128Plus g(seed);
  for (size_t i = n; i > 1; --i) {
    const uint32_t j = g.bounded(static_cast<uint32_t>(i));
    std::swap(data[i - 1], data[j]);
  }
}

}  // namespace stc
