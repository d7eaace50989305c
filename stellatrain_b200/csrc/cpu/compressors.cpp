#include "compressors.h"

#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <stdexcept>

#include "../core/threadpool.h"
#include "array_util.h"
#include "xorshift.h"

namespace stc {

namespace {

constexpr size_t kGrain = 1 << 16;     // elements per parallel range
constexpr int kBins = 2048;
constexpr int kShift = 20;

inline uint32_t key_of(float x) {
  uint32_t b;
  std::memcpy(&b, &x, 4);
  return b & 0x7fffffffu;
}

inline float as_float(uint32_t b) {
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}

void run_ranges(ThreadPool* pool, size_t n, const std::function<void(size_t, size_t, size_t)>& fn, size_t& parts_out) {
  // fixed partition so that per-range results can be combined in order
  const size_t parts = std::max<size_t>(1, std::min<size_t>(pool ? pool->size() + 1 : 1, (n + kGrain - 1) / kGrain));
  const size_t step = (n + parts - 1) / parts;
  parts_out = parts;
  if (parts == 1 || pool == nullptr) {
    for (size_t p = 0; p < parts; ++p) fn(p, p * step, std::min(n, (p + 1) * step));
    return;
  }
  pool->parallel_for(parts, 1, [&](size_t pb, size_t pe) {
    for (size_t p = pb; p < pe; ++p) fn(p, p * step, std::min(n, (p + 1) * step));
  });
}

// Exact top-k over keys produced by key(i); result positions ascending.  Returns the k-th key.
template <typename KeyFn>
uint32_t select_top_generic(size_t n, size_t k, ThreadPool* pool, KeyFn key, std::vector<uint32_t>& out_pos) {
  out_pos.clear();
  if (k == 0 || n == 0) return 0;
  k = std::min(k, n);
  size_t parts = 1;
  std::vector<std::vector<uint32_t>> hists;
  hists.assign(pool ? pool->size() + 1 : 1, std::vector<uint32_t>());
  run_ranges(pool, n, [&](size_t p, size_t b, size_t e) {
    auto& h = hists[p];
    h.assign(kBins, 0);
    for (size_t i = b; i < e; ++i) ++h[key(i) >> kShift];
  }, parts);
  std::vector<uint64_t> hist(kBins, 0);
  for (size_t p = 0; p < parts; ++p)
    for (int b = 0; b < kBins; ++b) hist[b] += hists[p][b];
  uint64_t above = 0;
  int thr_bin = kBins - 1;
  for (; thr_bin >= 0; --thr_bin) {
    if (above + hist[thr_bin] >= k) break;
    above += hist[thr_bin];
  }
  const size_t k_rem = k - above;
  // One more pass: positions whose bin lies above the threshold bin (ascending inside a range, ranges are
  // ascending themselves) and the candidates inside the bin.
  std::vector<std::vector<uint32_t>> above_parts(parts);
  std::vector<std::vector<std::pair<uint32_t, uint32_t>>> cparts(parts);   // (key, pos)
  run_ranges(pool, n, [&](size_t p, size_t b, size_t e) {
    auto& up = above_parts[p];
    auto& c = cparts[p];
    up.reserve((e - b) / 64 + 16);
    for (size_t i = b; i < e; ++i) {
      const uint32_t kx = key(i);
      const int bin = static_cast<int>(kx >> kShift);
      if (bin < thr_bin) continue;
      if (bin > thr_bin) up.push_back(static_cast<uint32_t>(i));
      else c.emplace_back(kx, static_cast<uint32_t>(i));
    }
  }, parts);
  std::vector<std::pair<uint32_t, uint32_t>> cand;
  for (auto& c : cparts) cand.insert(cand.end(), c.begin(), c.end());
  auto better = [](const std::pair<uint32_t, uint32_t>& a, const std::pair<uint32_t, uint32_t>& b) {
    return a.first != b.first ? a.first > b.first : a.second < b.second;
  };
  // after nth_element the first k_rem candidates are the k_rem best: larger key first, ties towards the lower position
  std::nth_element(cand.begin(), cand.begin() + (k_rem - 1), cand.end(), better);
  const uint32_t t_key = cand[k_rem - 1].first;
  std::vector<uint32_t> from_bin(k_rem);
  for (size_t j = 0; j < k_rem; ++j) from_bin[j] = cand[j].second;
  std::sort(from_bin.begin(), from_bin.end());
  std::vector<uint32_t> from_above;
  from_above.reserve(above);
  for (auto& up : above_parts) from_above.insert(from_above.end(), up.begin(), up.end());
  out_pos.resize(from_above.size() + from_bin.size());
  std::merge(from_above.begin(), from_above.end(), from_bin.begin(), from_bin.end(), out_pos.begin());
  return t_key;
}

}  // namespace

uint32_t select_top_keys(const uint32_t* keys, size_t n, size_t k, ThreadPool* pool, std::vector<uint32_t>& out_pos) {
  return select_top_generic(n, k, pool, [keys](size_t i) { return keys[i]; }, out_pos);
}

// ---------------------------------------------------------------- state
ThresholdState Compressor::load_state(const std::string& tensor) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = state_.find(tensor);
  return it == state_.end() ? ThresholdState{} : it->second;
}

void Compressor::store_state(const std::string& tensor, const ThresholdState& st) {
  std::lock_guard<std::mutex> lk(mu_);
  state_[tensor] = st;
}

std::map<std::string, ThresholdState> Compressor::export_state() {
  std::lock_guard<std::mutex> lk(mu_);
  return state_;
}

void Compressor::import_state(const std::map<std::string, ThresholdState>& st) {
  std::lock_guard<std::mutex> lk(mu_);
  state_ = st;
}

// ---------------------------------------------------------------- top-k
size_t TopkCompressor::compress(const std::string&, const float* src, size_t n, uint32_t k, uint32_t* dst_idx,
                                float* dst_val, int32_t idx_offset) {
  std::vector<uint32_t> pos;
  select_top_generic(n, k, pool_, [src](size_t i) { return key_of(src[i]); }, pos);
  for (size_t j = 0; j < pos.size(); ++j) {
    dst_idx[j] = pos[j] + idx_offset;
    dst_val[j] = src[pos[j]];
  }
  return pos.size();
}

// ---------------------------------------------------------------- threshold-v
namespace {

// Ordered compaction of |x| >= tau into dst, at most cap entries; returns (found, written).
__attribute__((target("avx512f"))) size_t filter_avx512(const float* src, size_t b, size_t e, float tau, uint32_t* dst_idx,
                                                        float* dst_val, size_t cap, int32_t idx_offset) {
  size_t w = 0, i = b;
  const __m512 vt = _mm512_set1_ps(tau);
  const __m512i lane = _mm512_setr_epi32(0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15);
  for (; i + 16 <= e && w + 16 <= cap; i += 16) {
    const __m512 v = _mm512_loadu_ps(src + i);
    const __mmask16 m = _mm512_cmp_ps_mask(_mm512_abs_ps(v), vt, _CMP_GE_OQ);
    if (!m) continue;
    const __m512i idx = _mm512_add_epi32(lane, _mm512_set1_epi32(static_cast<int>(i) + idx_offset));
    _mm512_mask_compressstoreu_ps(dst_val + w, m, v);
    _mm512_mask_compressstoreu_epi32(dst_idx + w, m, idx);
    w += static_cast<size_t>(__builtin_popcount(m));
  }
  for (; i < e && w < cap; ++i)
    if (std::fabs(src[i]) >= tau) {
      dst_idx[w] = static_cast<uint32_t>(i) + idx_offset;
      dst_val[w] = src[i];
      ++w;
    }
  return w;
}

size_t filter_scalar(const float* src, size_t b, size_t e, float tau, uint32_t* dst_idx, float* dst_val, size_t cap,
                     int32_t idx_offset) {
  size_t w = 0;
  for (size_t i = b; i < e && w < cap; ++i)
    if (std::fabs(src[i]) >= tau) {
      dst_idx[w] = static_cast<uint32_t>(i) + idx_offset;
      dst_val[w] = src[i];
      ++w;
    }
  return w;
}

}  // namespace

size_t ThresholdvCompressor::compress(const std::string& tensor, const float* src, size_t n, uint32_t k,
                                      uint32_t* dst_idx, float* dst_val, int32_t idx_offset) {
  if (k == 0 || n == 0) return 0;
  ThresholdState st = load_state(tensor);
  size_t parts = 1;
  std::vector<float> maxes(pool_ ? pool_->size() + 1 : 1, 0.f);
  if (!st.inited) {
    // first call: exact top-k gives the starting threshold (the reference runs nth_element,
    // thresholdv.cpp:27-37), followed by the first AIMD step as if one element too many was found
    std::vector<uint32_t> pos;
    const uint32_t t_key = select_top_generic(n, k, pool_, [src](size_t i) { return key_of(src[i]); }, pos);
    const float mx = max_abs(src, n);
    for (size_t j = 0; j < pos.size(); ++j) {
      dst_idx[j] = pos[j] + idx_offset;
      dst_val[j] = src[pos[j]];
    }
    st.tau = as_float(t_key) + (0.01f * (static_cast<float>(k + 1) / static_cast<float>(k))) * mx;
    st.tau_inc = 0.f;
    st.inited = true;
    store_state(tensor, st);
    return pos.size();
  }
  const float tau = st.tau;
  std::vector<size_t> counts(pool_ ? pool_->size() + 1 : 1, 0);
  run_ranges(pool_, n, [&](size_t p, size_t b, size_t e) {
    size_t c = 0;
    float m = 0.f;
    for (size_t i = b; i < e; ++i) {
      const float a = std::fabs(src[i]);
      c += a >= tau;
      m = a > m ? a : m;
    }
    counts[p] = c;
    maxes[p] = m;
  }, parts);
  std::vector<size_t> offs(parts + 1, 0);
  float mx = 0.f;
  for (size_t p = 0; p < parts; ++p) {
    offs[p + 1] = offs[p] + counts[p];
    mx = std::max(mx, maxes[p]);
  }
  const size_t found = offs[parts];
  const size_t step = (n + parts - 1) / parts;
  const bool v512 = best_isa() == Isa::Avx512;
  run_ranges(pool_, n, [&](size_t p, size_t b, size_t e) {
    if (offs[p] >= k) return;
    const size_t cap = std::min<size_t>(k - offs[p], counts[p]);
    (void)step;
    if (v512) filter_avx512(src, b, e, tau, dst_idx + offs[p], dst_val + offs[p], cap, idx_offset);
    else filter_scalar(src, b, e, tau, dst_idx + offs[p], dst_val + offs[p], cap, idx_offset);
  }, parts);
  if (k > found) st.tau = st.tau * 0.99f;
  else if (k < found) st.tau = st.tau + (0.01f * (static_cast<float>(found) / static_cast<float>(k))) * mx;
  store_state(tensor, st);
  return std::min<size_t>(found, k);
}

// ---------------------------------------------------------------- threshold-v16
size_t Thresholdv16Compressor::compress(const std::string& tensor, const float* src, size_t n, uint32_t k,
                                        uint32_t* dst_idx, float* dst_val, int32_t idx_offset) {
  if (k == 0 || n == 0) return 0;
  const size_t blocks = (n + 15) / 16;
  const size_t kb = (static_cast<size_t>(k) + 15) / 16;
  std::vector<float> score(blocks);
  size_t parts = 1;
  run_ranges(pool_, blocks, [&](size_t, size_t b, size_t e) {
    const size_t lo = b * 16, hi = std::min(n, e * 16);
    block_l1_norms(src + lo, hi - lo, score.data() + b);
  }, parts);
  ThresholdState st = load_state(tensor);
  std::vector<uint32_t> chosen;    // block ids in emission order; the last one may be truncated
  auto top_blocks = [&]() -> uint32_t {
    std::vector<uint32_t> pos;
    const uint32_t t_key = select_top_generic(blocks, kb, pool_, [&](size_t i) { return key_of(score[i]); }, pos);
    // the lowest-ranked block (smallest score, highest id among equals) goes last
    size_t last = 0;
    for (size_t j = 0; j < pos.size(); ++j)
      if (key_of(score[pos[j]]) == t_key) last = j;
    chosen.assign(pos.begin(), pos.end());
    if (!chosen.empty()) {
      const uint32_t lb = chosen[last];
      chosen.erase(chosen.begin() + static_cast<long>(last));
      chosen.push_back(lb);
    }
    return t_key;
  };
  if (!st.inited) {
    const float t0 = as_float(top_blocks());
    st.tau_inc = 0.01f * t0;
    st.tau = t0 + st.tau_inc;
    st.inited = true;
  } else {
    size_t flagged = 0;
    for (size_t b = 0; b < blocks; ++b) flagged += score[b] >= st.tau;
    if (flagged * 16 >= k) {
      chosen.reserve(kb);
      for (size_t b = 0; b < blocks && chosen.size() < kb; ++b)
        if (score[b] >= st.tau) chosen.push_back(static_cast<uint32_t>(b));
      st.tau = st.tau + st.tau_inc;
    } else {
      top_blocks();
      st.tau = st.tau * 0.99f;
    }
  }
  store_state(tensor, st);
  size_t w = 0, logical = 0;   // logical counts padded positions too, so that truncation matches the GPU tier
  for (size_t c = 0; c < chosen.size(); ++c) {
    const size_t base = static_cast<size_t>(chosen[c]) * 16;
    for (size_t j = 0; j < 16 && logical < k; ++j, ++logical) {
      if (base + j >= n) continue;   // zero padding of the tail block carries nothing
      dst_idx[w] = static_cast<uint32_t>(base + j) + idx_offset;
      dst_val[w] = src[base + j];
      ++w;
    }
  }
  return w;
}

// ---------------------------------------------------------------- random-k
size_t RandomkCompressor::compress(const std::string& tensor, const float* src, size_t n, uint32_t k, uint32_t* dst_idx,
                                   float* dst_val, int32_t idx_offset) {
  if (k == 0 || n == 0) return 0;
  k = static_cast<uint32_t>(std::min<size_t>(k, n));
  uint64_t call;
  {
    std::lock_guard<std::mutex> lk(mu_);
    call = calls_[tensor]++;
  }
  const uint64_t seed = seed_ ^ (std::hash<std::string>{}(tensor) * 0x9E3779B97F4A7C15ull) ^ (call << 32 | call);
  sample_without_replacement(static_cast<uint32_t>(n), k, seed, dst_idx);
  for (uint32_t j = 0; j < k; ++j) {
    dst_val[j] = src[dst_idx[j]];
    dst_idx[j] += idx_offset;
  }
  return k;
}

std::unique_ptr<Compressor> make_compressor(const std::string& method, ThreadPool* pool) {
  if (method == "topk") return std::make_unique<TopkCompressor>(pool);
  if (method == "thresholdv") return std::make_unique<ThresholdvCompressor>(pool);
  if (method == "thresholdv16") return std::make_unique<Thresholdv16Compressor>(pool);
  if (method == "randomk") return std::make_unique<RandomkCompressor>(pool);
  throw std::runtime_error("unknown compression method: " + method);
}

// ---------------------------------------------------------------- error feedback
size_t compress_with_feedback(Compressor& c, const std::string& tensor, const float* grad, float* resid, size_t n,
                              uint32_t k, uint32_t* dst_idx, float* dst_val, ThreadPool* pool) {
  size_t parts = 1;
  run_ranges(pool, n, [&](size_t, size_t b, size_t e) {
    add_arrays_nan_to_zero(resid + b, resid + b, grad + b, e - b);     // a = g + r in one pass, NaN dropped
  }, parts);
  const size_t cnt = c.compress(tensor, resid, n, k, dst_idx, dst_val, 0);
  for (size_t j = 0; j < cnt; ++j) resid[dst_idx[j]] = 0.f;
  return cnt;
}

}  // namespace stc
