// Task model of the CPU tier: one task per parameter tensor per iteration.
//
// After the reference's TrainTaskV2 (backend/src/engine/task.h:16-184, task.cpp:34-125): keys
// "{iter}@{layer}@{name}" (per iteration) and "{layer}@{name}" (persistent), priority
// iter*1000+layer (smaller runs first), and a state machine whose transitions are checked.  A
// transition that is not in the table is a programming error and throws; a stage that fails moves
// the task to Failed, which is terminal and reported to the waiter instead of hanging it.
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace stc {

enum class TaskState : int {
  Created = 0,
  CopyIn,        // gradient of this process copied into its shared slot          (reference: D2H_Copy)
  Gather,        // slice-parallel sum over local slots + residual                (CPU_Gather)
  Compress,      // node master: sparsify with error feedback                     (Compress)
  Exchange,      // node master: ring all-gather of the sparse streams            (GradientExchange)
  Optimize,      // node master: merge + sparse optimiser on the shared parameter (CPU_Optimize)
  WaitModel,     // wait until the previous version of this layer is no longer in use (H2D_Copy_Pre)
  CopyOut,       // updated parameter handed back to the framework                (H2D_Copy)
  Finished,
  Failed,
};
const char* task_state_name(TaskState s);
bool task_transition_allowed(TaskState from, TaskState to);

struct TrainTask {
  TrainTask(int64_t iter, int layer, const std::string& name);

  const int64_t iter;
  const int layer;
  const std::string name;
  const std::string key;              // "{iter}@{layer}@{name}"
  const std::string persistent_key;   // "{layer}@{name}"
  int64_t priority() const { return iter * 1000 + layer; }
  uint64_t barrier_key(int stage) const;   // identifies (task, stage) in the shared barrier table

  TaskState state() const { return state_.load(std::memory_order_acquire); }
  void advance(TaskState to);          // throws std::logic_error on an illegal transition
  void fail(const std::string& why);
  const std::string& error() const { return error_; }

  // working set
  uint32_t numel = 0;
  int param_index = -1;                // row in the shared parameter table
  std::vector<uint32_t> idx;           // [world * k] sparse streams, slot s at [s*k, (s+1)*k)
  std::vector<float> val;
  std::vector<size_t> counts;          // valid entries per slot
  uint32_t k = 0;
  double ratio = 0.99;                 // compression ratio of this iteration, fixed when the task is created
  int exchange_round = 0;

  // stage timers in milliseconds, -1 when a stage did not run (reference core.cpp:1151-1207).
  // Thread-safe: a stage hands the task to the next one before its own timer is closed, so two
  // workers can be inside these calls for one task at the same time.
  void stat_start(const std::string& event);
  void stat_end(const std::string& event);
  std::map<std::string, double> stats() const;

 private:
  std::atomic<TaskState> state_{TaskState::Created};
  std::string error_;
  mutable std::mutex stat_mu_;
  std::map<std::string, std::chrono::steady_clock::time_point> started_;
  std::map<std::string, double> elapsed_;
};

}  // namespace stc
