// Lazy ("touched indices only") optimisers of the CPU tier.
//
// Interface and rules after the reference's SparseOptimizer family
// (backend/src/optim/sparse_optimizer.h:10-46, sgd.cpp:221-262, adam.cpp:19-87, sgd_naive.cpp:3-58).
// State is kept per tensor name.  Differences, shared with the GPU tier and the oracle: AMSGrad keeps a
// per-element maximum (the reference one scalar per tensor), smart momentum counts optimiser steps per
// tensor, and Adam needs no global lock because state is per tensor.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../core/threadpool.h"

namespace stc {

class SparseOptimizer {
 public:
  virtual ~SparseOptimizer() = default;
  virtual const char* kind() const = 0;
  // param[idx[j]] is updated with grad[j] for j < grad_len; indices must be unique and < param_len.
  virtual void optimize_raw(float* param, uint32_t param_len, const std::string& name, const float* grad,
                            const uint32_t* idx, uint32_t grad_len) = 0;
  virtual void configure(const std::string& option, float value) = 0;   // unknown option: runtime_error("NO OPTION")
  virtual void configure(const std::string& option, bool value) = 0;
  // flat per-tensor state for checkpoints: named float arrays plus named counters
  struct TensorState {
    std::map<std::string, std::vector<float>> arrays;
    std::map<std::string, int64_t> counters;
  };
  virtual std::map<std::string, TensorState> export_state() = 0;
  virtual void import_state(const std::map<std::string, TensorState>& st) = 0;
  float lr() const { return lr_; }
  // Long index lists are split over this pool (indices of one call are unique, so the ranges touch disjoint
  // elements); without a pool, or for short lists, the calling thread does all the work.  The reference runs
  // its Adam loop under one global mutex (backend/src/optim/adam.cpp:47).
  void set_pool(ThreadPool* pool) { pool_ = pool; }

 protected:
  template <typename F>
  void for_ranges(uint32_t n, F&& fn) {
    if (pool_ != nullptr && n >= (1u << 15))
      pool_->parallel_for(n, 1u << 13, [&](size_t b, size_t e) { fn(static_cast<uint32_t>(b), static_cast<uint32_t>(e)); });
    else
      fn(0u, n);
  }
  ThreadPool* pool_ = nullptr;
  float lr_ = 1e-3f;   // backend/src/optim/sparse_optimizer.h:30
};

class SGD : public SparseOptimizer {
 public:
  const char* kind() const override { return "sgd"; }
  void optimize_raw(float* param, uint32_t param_len, const std::string& name, const float* grad, const uint32_t* idx,
                    uint32_t grad_len) override;
  void configure(const std::string& option, float value) override;
  void configure(const std::string& option, bool value) override;
  std::map<std::string, TensorState> export_state() override;
  void import_state(const std::map<std::string, TensorState>& st) override;

 private:
  struct State {
    std::vector<float> b;
    std::vector<uint32_t> last;
    bool first = true;
    uint32_t iter = 0;
  };
  State& state_for(const std::string& name, uint32_t len);
  float momentum_ = 0.f, dampening_ = 0.f, weight_decay_ = 0.f;
  bool nesterov_ = false, maximize_ = false, smart_momentum_ = false;
  std::mutex mu_;
  std::map<std::string, State> state_;
};

class Adam : public SparseOptimizer {
 public:
  const char* kind() const override { return "adam"; }
  void optimize_raw(float* param, uint32_t param_len, const std::string& name, const float* grad, const uint32_t* idx,
                    uint32_t grad_len) override;
  void configure(const std::string& option, float value) override;
  void configure(const std::string& option, bool value) override;
  std::map<std::string, TensorState> export_state() override;
  void import_state(const std::map<std::string, TensorState>& st) override;

 private:
  struct State {
    std::vector<float> m, v, vmax;
    uint32_t tick = 1;
  };
  State& state_for(const std::string& name, uint32_t len);
  float b1_ = 0.9f, b2_ = 0.999f, eps_ = 1e-8f, weight_decay_ = 0.f;
  bool amsgrad_ = false, maximize_ = false;
  std::mutex mu_;
  std::map<std::string, State> state_;
};

// Dense restatement of SGD used as a debugging oracle (backend/src/optim/sgd_naive.cpp:3-58): the
// sparse gradient is scattered into a dense one and EVERY element takes a momentum step.
class SGDNaive : public SparseOptimizer {
 public:
  const char* kind() const override { return "sgd_naive"; }
  void optimize_raw(float* param, uint32_t param_len, const std::string& name, const float* grad, const uint32_t* idx,
                    uint32_t grad_len) override;
  void configure(const std::string& option, float value) override;
  void configure(const std::string& option, bool value) override;
  std::map<std::string, TensorState> export_state() override { return {}; }
  void import_state(const std::map<std::string, TensorState>&) override {}

 private:
  float momentum_ = 0.f, dampening_ = 0.f, weight_decay_ = 0.f;
  bool nesterov_ = false, maximize_ = false;
  std::mutex mu_;
  std::map<std::string, std::vector<float>> b_;
  std::map<std::string, bool> started_;
};

std::unique_ptr<SparseOptimizer> make_optimizer(const std::string& name);

// Merge of W sparse streams (backend/src/engine/modules/cpu_optimize.cpp:40-72): weighted sum per
// index over the sources, each index reported once.  `scratch` must hold n zeros on entry and holds
// n zeros again on return.  Returns the number of merged entries written to out_idx/out_val
// (capacity: total number of input entries).
size_t merge_streams(const uint32_t* const* idx, const float* const* val, const size_t* counts, const float* weights,
                     int sources, float* scratch, uint8_t* touched, size_t n, uint32_t* out_idx, float* out_val);

}  // namespace stc
