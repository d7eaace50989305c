#include "task.h"

#include <functional>
#include <stdexcept>

#include "config.h"

namespace stc {

const char* task_state_name(TaskState s) {
  static const char* names[] = {"Created", "CopyIn", "Gather", "Compress", "Exchange", "Optimize",
                                "WaitModel", "CopyOut", "Finished", "Failed"};
  return names[static_cast<int>(s)];
}

bool task_transition_allowed(TaskState from, TaskState to) {
  if (to == TaskState::Failed) return from != TaskState::Finished && from != TaskState::Failed;
  switch (from) {
    case TaskState::Created: return to == TaskState::CopyIn;
    case TaskState::CopyIn: return to == TaskState::Gather;
    case TaskState::Gather: return to == TaskState::Compress;
    // a single-node job skips the exchange; processes that are not node master skip to WaitModel
    case TaskState::Compress: return to == TaskState::Exchange || to == TaskState::Optimize || to == TaskState::WaitModel;
    case TaskState::Exchange: return to == TaskState::Exchange || to == TaskState::Optimize;
    case TaskState::Optimize: return to == TaskState::WaitModel;
    case TaskState::WaitModel: return to == TaskState::CopyOut;
    case TaskState::CopyOut: return to == TaskState::Finished;
    default: return false;
  }
}

static std::string make_key(int64_t iter, int layer, const std::string& name) {
  return std::to_string(iter) + "@" + std::to_string(layer) + "@" + name;
}

TrainTask::TrainTask(int64_t it, int ly, const std::string& nm)
    : iter(it), layer(ly), name(nm), key(make_key(it, ly, nm)), persistent_key(std::to_string(ly) + "@" + nm) {
  if (static_cast<int>(persistent_key.size()) > cfg::kMaxNameLen)
    throw std::runtime_error("parameter key longer than " + std::to_string(cfg::kMaxNameLen) + " characters: " + persistent_key);
}

uint64_t TrainTask::barrier_key(int stage) const {
  uint64_t h = std::hash<std::string>{}(key);
  h ^= (static_cast<uint64_t>(stage) + 0x9E3779B97F4A7C15ull) + (h << 6) + (h >> 2);
  return h ? h : 1;
}

void TrainTask::advance(TaskState to) {
  const TaskState from = state_.load(std::memory_order_acquire);
  if (!task_transition_allowed(from, to))
    throw std::logic_error(std::string("illegal task transition ") + task_state_name(from) + " -> " +
                           task_state_name(to) + " for " + key);
  state_.store(to, std::memory_order_release);
}

void TrainTask::fail(const std::string& why) {
  error_ = why;
  state_.store(TaskState::Failed, std::memory_order_release);
}

void TrainTask::stat_start(const std::string& event) {
  std::lock_guard<std::mutex> lk(stat_mu_);
  started_[event] = std::chrono::steady_clock::now();
}

void TrainTask::stat_end(const std::string& event) {
  std::lock_guard<std::mutex> lk(stat_mu_);
  auto it = started_.find(event);
  if (it == started_.end()) return;
  elapsed_[event] = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - it->second).count();
}

std::map<std::string, double> TrainTask::stats() const {
  std::lock_guard<std::mutex> lk(stat_mu_);
  std::map<std::string, double> out = elapsed_;
  for (auto& kv : started_)
    if (!out.count(kv.first)) out[kv.first] = -1.0;
  return out;
}

}  // namespace stc
