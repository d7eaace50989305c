#include "optimizers.h"

#include <immintrin.h>

#include <cmath>
#include <stdexcept>

#include "array_util.h"

namespace stc {

// Gather / compute / scatter over 16 unique indices at a time (the reference's vector path,
// backend/src/optim/sgd.cpp:56-215, is compiled out by its build flags).  Same operations in the
// same order as the scalar loop, so results are bit-identical.
__attribute__((target("avx512f"))) static uint32_t sgd_avx512(float* param, float* bbuf, const float* grad,
                                                              const uint32_t* idx, uint32_t len, float lr, float mu,
                                                              float damp, float wd, bool first) {
  const __m512 vlr = _mm512_set1_ps(lr), vmu = _mm512_set1_ps(mu), vd = _mm512_set1_ps(1.f - damp),
               vwd = _mm512_set1_ps(wd);
  uint32_t j = 0;
  for (; j + 16 <= len; j += 16) {
    const __m512i vi = _mm512_loadu_si512(idx + j);
    const __m512 x = _mm512_i32gather_ps(vi, param, 4);
    __m512 g = _mm512_loadu_ps(grad + j);
    if (wd != 0.f) g = _mm512_add_ps(g, _mm512_mul_ps(vwd, x));
    if (mu != 0.f) {
      __m512 b = g;
      if (!first) b = _mm512_add_ps(_mm512_mul_ps(_mm512_i32gather_ps(vi, bbuf, 4), vmu), _mm512_mul_ps(vd, g));
      _mm512_i32scatter_ps(bbuf, vi, b, 4);
      g = b;
    }
    _mm512_i32scatter_ps(param, vi, _mm512_sub_ps(x, _mm512_mul_ps(vlr, g)), 4);
  }
  return j;
}

// ---------------------------------------------------------------- SGD
// The state of a tensor is created at its first update.  The arrays are allocated and zeroed outside the lock: in
// the first iteration every tensor of the model gets here at once from the pool's threads, and touching a few hundred
// megabytes of fresh pages under one mutex would make them queue up behind one another (updates of one tensor never
// overlap, so nobody else can be creating the same entry meanwhile).
SGD::State& SGD::state_for(const std::string& name, uint32_t len) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = state_.find(name);
    if (it != state_.end() && it->second.b.size() == len) return it->second;
  }
  std::vector<float> b(len, 0.f);
  std::vector<uint32_t> last(len, 0u);
  std::lock_guard<std::mutex> lk(mu_);
  State& s = state_[name];
  if (s.b.size() != len) {
    s.b.swap(b);
    s.last.swap(last);
    s.first = true;
    s.iter = 0;
  }
  return s;
}

void SGD::optimize_raw(float* param, uint32_t param_len, const std::string& name, const float* grad,
                       const uint32_t* idx, uint32_t grad_len) {
  State& s = state_for(name, param_len);
  const float lr = maximize_ ? -lr_ : lr_;
  const bool first = s.first;
  for (uint32_t j = 0; j < grad_len; ++j)
    if (idx[j] >= param_len) throw std::out_of_range("sparse SGD: index beyond the parameter");
  const bool simd = best_isa() == Isa::Avx512 && !smart_momentum_ && !nesterov_ && param_len < (1u << 31);
  for_ranges(grad_len, [&](uint32_t jb, uint32_t je) {
    uint32_t j0 = jb;
    if (simd) j0 = jb + sgd_avx512(param, s.b.data(), grad + jb, idx + jb, je - jb, lr, momentum_, dampening_, weight_decay_, first);
    for (uint32_t j = j0; j < je; ++j) {
      const uint32_t i = idx[j];
      const float x = param[i];
      float g = grad[j];
      float mu = momentum_;
      if (smart_momentum_ && s.iter != 0) mu = std::pow(momentum_, static_cast<float>(s.iter - s.last[i]));
      if (weight_decay_ != 0.f) g += weight_decay_ * x;
      if (momentum_ != 0.f) {
        const float b = first ? g : s.b[i] * mu + (1.f - dampening_) * g;
        g = nesterov_ ? g + mu * b : b;
        s.b[i] = b;
      }
      param[i] = x - lr * g;
      if (smart_momentum_) s.last[i] = s.iter;
    }
  });
  s.first = false;
  ++s.iter;
}

void SGD::configure(const std::string& o, float v) {
  if (o == "lr") lr_ = v;
  else if (o == "momentum") momentum_ = v;
  else if (o == "weight_decay") weight_decay_ = v;
  else if (o == "dampening") dampening_ = v;
  else throw std::runtime_error("NO OPTION");
}

void SGD::configure(const std::string& o, bool v) {
  if (o == "nestrov" || o == "nesterov") nesterov_ = v;
  else if (o == "maximize") maximize_ = v;
  else if (o == "smart_momentum") smart_momentum_ = v;
  else throw std::runtime_error("NO OPTION");
}

std::map<std::string, SparseOptimizer::TensorState> SGD::export_state() {
  std::lock_guard<std::mutex> lk(mu_);
  std::map<std::string, TensorState> out;
  for (auto& kv : state_) {
    TensorState t;
    t.arrays["b"] = kv.second.b;
    t.arrays["last"] = std::vector<float>(kv.second.last.begin(), kv.second.last.end());
    t.counters["first"] = kv.second.first;
    t.counters["iter"] = kv.second.iter;
    out[kv.first] = std::move(t);
  }
  return out;
}

void SGD::import_state(const std::map<std::string, TensorState>& st) {
  std::lock_guard<std::mutex> lk(mu_);
  state_.clear();
  for (auto& kv : st) {
    State s;
    s.b = kv.second.arrays.at("b");
    const auto& l = kv.second.arrays.at("last");
    s.last.assign(l.begin(), l.end());
    s.first = kv.second.counters.at("first") != 0;
    s.iter = static_cast<uint32_t>(kv.second.counters.at("iter"));
    state_[kv.first] = std::move(s);
  }
}

// ---------------------------------------------------------------- Adam
Adam::State& Adam::state_for(const std::string& name, uint32_t len) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = state_.find(name);
    if (it != state_.end() && it->second.m.size() == len && (!amsgrad_ || it->second.vmax.size() == len)) return it->second;
  }
  std::vector<float> m(len, 0.f), v(len, 0.f), vmax(amsgrad_ ? len : 0, 0.f);   // outside the lock, see SGD::state_for
  std::lock_guard<std::mutex> lk(mu_);
  State& s = state_[name];
  if (s.m.size() != len) {
    s.m.swap(m);
    s.v.swap(v);
    s.vmax.swap(vmax);
    s.tick = 1;
  } else if (amsgrad_ && s.vmax.size() != len) {
    s.vmax.swap(vmax);
  }
  return s;
}

void Adam::optimize_raw(float* param, uint32_t param_len, const std::string& name, const float* grad,
                        const uint32_t* idx, uint32_t grad_len) {
  State& s = state_for(name, param_len);
  const double b1 = b1_, b2 = b2_, lr = lr_, eps = eps_;
  const double c1 = 1.0 - std::pow(b1, static_cast<double>(s.tick));
  const double c2 = 1.0 - std::pow(b2, static_cast<double>(s.tick));
  for (uint32_t j = 0; j < grad_len; ++j)
    if (idx[j] >= param_len) throw std::out_of_range("sparse Adam: index beyond the parameter");
  for_ranges(grad_len, [&](uint32_t jb, uint32_t je) {
    for (uint32_t j = jb; j < je; ++j) {
      const uint32_t i = idx[j];
      const float x = param[i];
      float g = grad[j];
      if (maximize_) g = -g;
      if (weight_decay_ != 0.f) g += weight_decay_ * x;
      const double mt = b1 * s.m[i] + (1.0 - b1) * g;
      const double vt = b2 * s.v[i] + (1.0 - b2) * static_cast<double>(g) * g;
      const double mh = mt / c1;
      double vh = vt / c2;
      if (amsgrad_) {
        vh = std::max(static_cast<double>(s.vmax[i]), vh);
        s.vmax[i] = static_cast<float>(vh);
      }
      param[i] = static_cast<float>(x - lr * mh / (std::sqrt(vh) + eps));
      s.m[i] = static_cast<float>(mt);
      s.v[i] = static_cast<float>(vt);
    }
  });
  ++s.tick;
}

void Adam::configure(const std::string& o, float v) {
  if (o == "lr") lr_ = v;
  else if (o == "b1") b1_ = v;
  else if (o == "b2") b2_ = v;
  else if (o == "weight_decay") weight_decay_ = v;
  else if (o == "eps") eps_ = v;
  else throw std::runtime_error("NO OPTION");
}

void Adam::configure(const std::string& o, bool v) {
  if (o == "amsgrad") amsgrad_ = v;
  else if (o == "maximize") maximize_ = v;
  else throw std::runtime_error("NO OPTION");
}

std::map<std::string, SparseOptimizer::TensorState> Adam::export_state() {
  std::lock_guard<std::mutex> lk(mu_);
  std::map<std::string, TensorState> out;
  for (auto& kv : state_) {
    TensorState t;
    t.arrays["m"] = kv.second.m;
    t.arrays["v"] = kv.second.v;
    t.arrays["vmax"] = kv.second.vmax;
    t.counters["tick"] = kv.second.tick;
    out[kv.first] = std::move(t);
  }
  return out;
}

void Adam::import_state(const std::map<std::string, TensorState>& st) {
  std::lock_guard<std::mutex> lk(mu_);
  state_.clear();
  for (auto& kv : st) {
    State s;
    s.m = kv.second.arrays.at("m");
    s.v = kv.second.arrays.at("v");
    s.vmax = kv.second.arrays.at("vmax");
    s.tick = static_cast<uint32_t>(kv.second.counters.at("tick"));
    state_[kv.first] = std::move(s);
  }
}

// ---------------------------------------------------------------- dense oracle
void SGDNaive::optimize_raw(float* param, uint32_t param_len, const std::string& name, const float* grad,
                            const uint32_t* idx, uint32_t grad_len) {
  std::vector<float> dense(param_len, 0.f);
  for (uint32_t j = 0; j < grad_len; ++j) dense.at(idx[j]) += grad[j];
  std::lock_guard<std::mutex> lk(mu_);
  auto& b = b_[name];
  bool& started = started_[name];
  if (b.size() != param_len) { b.assign(param_len, 0.f); started = false; }
  const float lr = maximize_ ? -lr_ : lr_;
  for (uint32_t i = 0; i < param_len; ++i) {
    float g = dense[i];
    if (weight_decay_ != 0.f) g += weight_decay_ * param[i];
    if (momentum_ != 0.f) {
      b[i] = started ? momentum_ * b[i] + (1.f - dampening_) * g : g;
      g = nesterov_ ? g + momentum_ * b[i] : b[i];
    }
    param[i] -= lr * g;
  }
  started = true;
}

void SGDNaive::configure(const std::string& o, float v) {
  if (o == "lr") lr_ = v;
  else if (o == "momentum") momentum_ = v;
  else if (o == "weight_decay") weight_decay_ = v;
  else if (o == "dampening") dampening_ = v;
  else throw std::runtime_error("NO OPTION");
}

void SGDNaive::configure(const std::string& o, bool v) {
  if (o == "nestrov" || o == "nesterov") nesterov_ = v;
  else if (o == "maximize") maximize_ = v;
  else throw std::runtime_error("NO OPTION");
}

std::unique_ptr<SparseOptimizer> make_optimizer(const std::string& name) {
  if (name == "sgd") return std::make_unique<SGD>();
  if (name == "adam") return std::make_unique<Adam>();
  if (name == "sgd_naive") return std::make_unique<SGDNaive>();
  throw std::runtime_error("unknown optimizer: " + name);
}

// ---------------------------------------------------------------- merge
size_t merge_streams(const uint32_t* const* idx, const float* const* val, const size_t* counts, const float* weights,
                     int sources, float* scratch, uint8_t* touched, size_t n, uint32_t* out_idx, float* out_val) {
  size_t out = 0;
  for (int s = 0; s < sources; ++s) {
    const float w = weights[s];
    for (size_t j = 0; j < counts[s]; ++j) {
      const uint32_t i = idx[s][j];
      if (i == 0xFFFFFFFFu) continue;
      if (i >= n) throw std::out_of_range("merge: index beyond the tensor");
      scratch[i] += val[s][j] * w;
      if (!touched[i]) {
        touched[i] = 1;
        out_idx[out++] = i;
      }
    }
  }
  for (size_t j = 0; j < out; ++j) {
    const uint32_t i = out_idx[j];
    out_val[j] = scratch[i];
    scratch[i] = 0.f;
    touched[i] = 0;
  }
  return out;
}

}  // namespace stc
