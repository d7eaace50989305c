// Pipeline stages of the CPU tier, in execution order.  Stage-by-stage counterpart of the
// reference's modules (backend/src/engine/modules/: d2h_copy.cpp:20-94, cpu_gather.cpp:32-92,
// compress.cpp:19-216, grad_exchange.cpp:18-81, cpu_optimize.cpp:26-140, h2d_copy.cpp:15-72,
// barrier_checker.cpp:5-30, null.cpp:3-9), instantiated by load_modules like core_module_load.cpp:15-28.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>

#include "../cpu/array_util.h"
#include "config.h"
#include "cuda_api.h"
#include "engine.h"
#include "logger.h"

namespace stc {

namespace {

uint32_t entries_for(uint32_t numel, double ratio, int world) {
  // k = max(min(n, 1), n * (1 - ratio) / W)   (reference compress.cpp:44-52)
  const double k_frac = (1.0 - ratio) / std::max(1, world);
  const uint32_t k = static_cast<uint32_t>(static_cast<double>(numel) * k_frac + 1e-6);   // same rounding guard as buckets.py
  return std::min(numel, std::max<uint32_t>(std::min<uint32_t>(numel, 1u), k));
}

class ModuleNull : public Module {
 public:
  const char* name() const override { return "Null"; }
  void run(CpuEngine&, const std::shared_ptr<TrainTask>&) override {}
};

// Self-check of the task barriers: 60 rounds of "write own slot | barrier | read the neighbour's slot
// | barrier"; a lost wake-up or a miscounted barrier shows up as a wrong value or a timeout.
class ModuleBarrierChecker : public Module {
 public:
  const char* name() const override { return "BarrierChecker"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    auto& p = e.param(t->param_index);
    const int N = e.options().local_world, r = e.options().local_rank;
    std::lock_guard<std::mutex> lk(mu_);
    int& step = steps_[t->key];           // even: write phase, odd: read phase
    float* mine = p.slot[t->iter % 2][r];
    if (step == 0) parked_[t->key].assign(mine, mine + p.numel);   // the real gradient waits here
    const int round = step / 2 + 1;
    if (step == 120) {
      steps_.erase(t->key);
      std::memcpy(mine, parked_[t->key].data(), static_cast<size_t>(p.numel) * sizeof(float));
      parked_.erase(t->key);
      e.schedule(e.module("CopyIn"), t);
      return;
    }
    if (step % 2 == 0) {
      if (p.numel >= 1) mine[0] = static_cast<float>(-round);
    } else if (N > 1 && p.numel >= 1) {
      const float seen = p.slot[t->iter % 2][(r + 1) % N][0];
      if (seen != static_cast<float>(-round)) throw std::runtime_error("barrier self-check read a stale value");
    }
    ++step;
    e.schedule_after_barrier(this, t, kCheckerBase + step);
  }

 private:
  std::mutex mu_;
  std::map<std::string, int> steps_;
  std::map<std::string, std::vector<float>> parked_;
};

class ModuleCopyIn : public Module {
 public:
  const char* name() const override { return "CopyIn"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    t->advance(TaskState::CopyIn);
    if (e.options().debug_accuracy) {
      auto& p = e.param(t->param_index);
      if (has_nan(p.slot[t->iter % 2][e.options().local_rank], p.numel)) throw std::runtime_error("NaN in the gradient");
    }
    e.schedule_after_barrier(e.module("GatherGate"), t, kAfterCopyIn);
  }
};

// Iterations of one parameter pass gather..optimise one at a time (error-feedback residual, optimiser
// state and master copy are carried from one iteration to the next).
class ModuleGatherGate : public Module {
 public:
  const char* name() const override { return "GatherGate"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override { e.schedule_after_previous(e.module("Gather"), t); }
};

class ModuleGather : public Module {
 public:
  const char* name() const override { return "Gather"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    t->advance(TaskState::Gather);
    auto& p = e.param(t->param_index);
    const int N = e.options().local_world, r = e.options().local_rank;
    const size_t len = p.numel;
    const size_t b = len * static_cast<size_t>(r) / N, en = len * static_cast<size_t>(r + 1) / N;
    // The slice of the residual takes the sum: r <- r + g_0 + ... + g_{N-1}.  Accumulating into the residual instead of
    // into a gradient slot lets the compress stage work in place, so no copy back into the residual is needed afterwards
    // (the reference sums into slot 0 and copies the whole tensor back, cpu_gather.cpp:63-82, compress.cpp:172-188).
    float* dst = p.resid + b;
    if (e.options().skip_critical_paths) {
      e.schedule_after_barrier(e.module("Compress"), t, kAfterGather);
      return;
    }
    t->stat_start("CRIT_PATH_gather");
    // the last addition also applies the NaN policy shared with the GPU tier: a NaN is dropped (neither sent nor kept)
    for (int g = 0; g + 1 < N; ++g) add_arrays(dst, p.slot[t->iter % 2][g] + b, en - b);
    add_arrays_nan_to_zero(dst, dst, p.slot[t->iter % 2][N - 1] + b, en - b);
    t->stat_end("CRIT_PATH_gather");
    e.schedule_after_barrier(e.module("Compress"), t, kAfterGather);
  }
};

class ModuleCompress : public Module {
 public:
  const char* name() const override { return "Compress"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    t->advance(TaskState::Compress);
    if (!e.node_master()) {
      e.schedule_after_barrier(e.module("WaitModel"), t, kAfterOptimize);
      return;
    }
    auto& p = e.param(t->param_index);
    const int W = e.options().world;
    float* acc = p.resid;                                        // gradient sum plus residual, NaN dropped, left by the gather stage
    // a bundle keeps the per-tensor rule: every member has its own k and its own threshold
    uint32_t k = 0;
    if (p.members.empty()) k = entries_for(p.numel, t->ratio, W);
    else for (const auto& m : p.members) k += entries_for(m.numel, t->ratio, W);
    t->k = k;
    t->idx.assign(static_cast<size_t>(k) * W, 0xFFFFFFFFu);
    t->val.assign(static_cast<size_t>(k) * W, 0.f);
    t->counts.assign(W, 0);
    t->stat_start("CRIT_PATH_compress");
    size_t cnt = 0;
    if (e.options().skip_critical_paths) {
    } else if (p.members.empty()) {
      cnt = e.compressor().compress(t->persistent_key, acc, p.numel, k, t->idx.data(), t->val.data(), 0);
    } else {
      for (const auto& m : p.members)
        cnt += e.compressor().compress(m.key, acc + m.off, m.numel, entries_for(m.numel, t->ratio, W), t->idx.data() + cnt,
                                       t->val.data() + cnt, static_cast<int32_t>(m.off));
    }
    t->stat_end("CRIT_PATH_compress");
    t->counts[0] = cnt;
    if (e.options().debug_accuracy)
      for (size_t j = 0; j < cnt; ++j)
        if (t->idx[j] >= p.numel || t->val[j] != acc[t->idx[j]]) throw std::runtime_error("compressor output is inconsistent");
    t->stat_start("CRIT_PATH_save_residual");
    const int vf = W > 1 ? e.wire_value_format() : 0;
    if (vf == 0) {
      for (size_t j = 0; j < cnt; ++j) acc[t->idx[j]] = 0.f;
    } else {
      // narrow values on the wire: send what the receiver will decode and keep the rounding error here
      std::vector<uint16_t> half(cnt);
      std::vector<float> sent(cnt);
      if (vf == 1) { f32_to_f16(t->val.data(), half.data(), cnt); f16_to_f32(half.data(), sent.data(), cnt); }
      else { f32_to_bf16(t->val.data(), half.data(), cnt); bf16_to_f32(half.data(), sent.data(), cnt); }
      for (size_t j = 0; j < cnt; ++j) {
        const float s = std::isfinite(sent[j]) ? sent[j] : 0.f;   // fp16 overflow: keep the whole value for later
        acc[t->idx[j]] = t->val[j] - s;
        t->val[j] = s;
      }
    }
    t->stat_end("CRIT_PATH_save_residual");      // what was not sent already sits in the residual
    if (W == 1) e.schedule_after_master_free(e.module("Optimize"), t);
    else e.schedule(e.module("GradExchange"), t);
  }
};

class ModuleGradExchange : public Module {
 public:
  const char* name() const override { return "GradExchange"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    if (t->state() != TaskState::Exchange) t->advance(TaskState::Exchange);
    const int W = e.options().world;
    const int round = t->exchange_round;
    if (round >= W - 1) {
      e.schedule_after_master_free(e.module("Optimize"), t);
      return;
    }
    // ring all-gather: forward slot `round` to the successor, expect slot `round + 1` from the predecessor
    const std::string key = t->key + "!" + std::to_string(round);
    const size_t off = static_cast<size_t>(round) * t->k;
    e.comm()->queue_tx(t->priority(), key, t->idx.data() + off, t->val.data() + off, t->counts[round], t->numel,
                       true, e.wire_value_format(), e.wire_blocks());
    e.schedule_after_comm(this, t, key, round + 1);
  }
};

class ModuleOptimize : public Module {
 public:
  const char* name() const override { return "Optimize"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    t->advance(TaskState::Optimize);
    auto& p = e.param(t->param_index);
    const int W = e.options().world;
    if (p.merge_scratch.size() != p.numel) {
      p.merge_scratch.assign(p.numel, 0.f);
      p.merge_touched.assign(p.numel, 0);
    }
    std::vector<const uint32_t*> idx(W);
    std::vector<const float*> val(W);
    // mean over nodes (cpu_optimize.cpp:55) unless the nodes were given their shares of the global batch; slot 0 is this
    // node's own stream, slot s the stream that started s hops up the ring
    const std::vector<float> by_node = e.node_weights_at(t->iter);
    std::vector<float> weights(W);
    for (int s = 0; s < W; ++s) weights[s] = by_node[static_cast<size_t>(((e.options().rank - s) % W + W) % W)];
    size_t total = 0;
    for (int s = 0; s < W; ++s) {
      idx[s] = t->idx.data() + static_cast<size_t>(s) * t->k;
      val[s] = t->val.data() + static_cast<size_t>(s) * t->k;
      total += t->counts[s];
    }
    std::vector<uint32_t> midx(total);
    std::vector<float> mval(total);
    const size_t n = merge_streams(idx.data(), val.data(), t->counts.data(), weights.data(), W, p.merge_scratch.data(),
                                   p.merge_touched.data(), p.numel, midx.data(), mval.data());
    t->stat_start("CRIT_PATH_optimize_raw");
    e.sparse_optimizer()->optimize_raw(p.master, p.numel, t->persistent_key, mval.data(), midx.data(), static_cast<uint32_t>(n));
    t->stat_end("CRIT_PATH_optimize_raw");
    if (e.options().debug_accuracy && has_nan(p.master, p.numel)) throw std::runtime_error("NaN in the parameter");
    t->idx.clear(); t->idx.shrink_to_fit();
    t->val.clear(); t->val.shrink_to_fit();
    e.schedule_after_barrier(e.module("WaitModel"), t, kAfterOptimize);
  }
};

class ModuleWaitModel : public Module {
 public:
  const char* name() const override { return "WaitModel"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    t->advance(TaskState::WaitModel);
    e.mark_sequenced(t);
    e.schedule_after_model_complete(e.module("CopyOut"), t);
  }
};

class ModuleCopyOut : public Module {
 public:
  const char* name() const override { return "CopyOut"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    t->advance(TaskState::CopyOut);
    auto& p = e.param(t->param_index);
    // the slot is consumed: clear this process's part for the next use
    std::memset(p.slot[t->iter % 2][e.options().local_rank], 0, static_cast<size_t>(p.numel) * sizeof(float));
    const bool device_members = !p.members.empty() && p.members[0].device_param != nullptr;
    if (p.device_param != nullptr || device_members) {
      // host-to-device copy on the stream that carried this parameter's latest gradient copy: that copy waited for the
      // backward kernels that last read the parameter, so stream order keeps the write behind every reader
      const CudaApi* api = cuda_api();
      e.use_engine_device();
      void* stream = p.last_copy_stream ? p.last_copy_stream : e.copy_stream_for(t->param_index);
      int rc = api ? 0 : -1;
      if (rc == 0 && !device_members)
        rc = api->memcpy_h2d_async(p.device_param, p.master, static_cast<size_t>(p.numel) * sizeof(float), stream);
      for (size_t m = 0; rc == 0 && device_members && m < p.members.size(); ++m)
        rc = api->memcpy_h2d_async(p.members[m].device_param, p.master + p.members[m].off,
                                   static_cast<size_t>(p.members[m].numel) * sizeof(float), stream);
      if (rc != 0) {
        e.fail_task(t, "host-to-device copy of the parameter failed");
        return;
      }
      e.schedule_after_cuda(e.module("CopyOutPost"), t, stream);
      return;
    }
    bool host_members = false;
    for (const auto& m : p.members) {
      if (!m.user_param) continue;
      host_members = true;
      std::memcpy(m.user_param, p.master + m.off, static_cast<size_t>(m.numel) * sizeof(float));
    }
    if (p.user_param == nullptr && !host_members) {
      e.push_ready_update(t->param_index, t->iter);   // the caller copies and reports copy_out_done()
      return;
    }
    if (p.user_param) std::memcpy(p.user_param, p.master, static_cast<size_t>(p.numel) * sizeof(float));
    e.schedule_after_barrier(e.module("CopyOutDone"), t, kAfterCopyOut);
  }
};

// Behind the asynchronous host-to-device copy (reference H2D_Copy_Post, h2d_copy.cpp:59-72): wait for the other local
// processes, then finish.
class ModuleCopyOutPost : public Module {
 public:
  const char* name() const override { return "CopyOutPost"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    e.schedule_after_barrier(e.module("CopyOutDone"), t, kAfterCopyOut);
  }
};

// Every local process has copied the master parameter out: the optimise stage of the next iteration may
// write it again, the forward pass may use the copy, the gradient slot is free.
class ModuleCopyOutDone : public Module {
 public:
  const char* name() const override { return "CopyOutDone"; }
  void run(CpuEngine& e, const std::shared_ptr<TrainTask>& t) override {
    t->advance(TaskState::Finished);
    e.mark_master_read(t);
    e.update_model_version(t);
    e.return_after_use(t);
    e.schedule_terminate(t);
  }
};

}  // namespace

void CpuEngine::load_modules() {
  auto add = [this](std::unique_ptr<Module> m) {
    const std::string n = m->name();
    modules_[n] = std::move(m);
  };
  add(std::make_unique<ModuleNull>());
  add(std::make_unique<ModuleBarrierChecker>());
  add(std::make_unique<ModuleCopyIn>());
  add(std::make_unique<ModuleGatherGate>());
  add(std::make_unique<ModuleGather>());
  add(std::make_unique<ModuleCompress>());
  add(std::make_unique<ModuleGradExchange>());
  add(std::make_unique<ModuleOptimize>());
  add(std::make_unique<ModuleWaitModel>());
  add(std::make_unique<ModuleCopyOut>());
  add(std::make_unique<ModuleCopyOutPost>());
  add(std::make_unique<ModuleCopyOutDone>());
}

}  // namespace stc
