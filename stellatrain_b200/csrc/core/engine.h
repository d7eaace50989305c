// Engine of the CPU-offload tier: per-parameter task pipeline over shared memory and TCP.
//
// Structure after the reference's FasterDpEngine and its module API
// (backend/src/engine/core.h:47-310, core.cpp:64-183 configure, 712-758 pre_forward_process, 761-834
// pre_train_init, 1025-1095 post_backward_process, 1097-1140 synchronize_backend; core_module_api.cpp:
// schedule 7-24, schedule_terminate 27-40, schedule_after_use 43-109, schedule_after_barrier 113-199,
// schedule_after_model_complete 279-310, schedule_after_comm 313-375, update_model_version 462-472).
// One process per local device; the processes of a node share gradients and master parameters through
// ShmManager, the node master compresses, exchanges and optimises; nodes form a TCP ring.
//
// Device copies stay in the framework: the engine works on host pointers.  For CUDA training the
// Python side copies gradients into the pinned shared slots and parameters back (see
// stellatrain_b200/cpu_tier.py); for host tensors the engine copies by itself.
//
// Every wait is bounded: a timeout marks the task Failed and surfaces as an exception from
// synchronize()/pre_forward(), it never blocks forever.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <future>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../comm/comm_manager.h"
#include "../cpu/compressors.h"
#include "../cpu/optimizers.h"
#include "shm_manager.h"
#include "task.h"
#include "threadpool.h"

namespace stc {

struct EngineOptions {
  std::string master_addr = "127.0.0.1";
  uint16_t master_port = 5555;
  int world = 1;              // nodes
  int rank = 0;               // node rank
  int64_t session = 0;        // names the node's shared-memory segments
  int local_world = 1;
  int local_rank = 0;
  std::string method = "thresholdv16";
  int grad_accumulation = 1;
  int staleness = 1;
  double ratio = 0.99;        // fraction dropped
  size_t data_bytes = 0;      // 0: default from config.h
  size_t meta_bytes = 0;
  int timeout_ms = 30000;
  int workers = 0;            // 0: 32 on the node master, 16 otherwise
  bool pin_cuda = false;      // cudaHostRegister the data segment
  bool debug_accuracy = false;
  bool debug_barrier = false; // run the barrier self-check before the first task of every parameter
  // Leave out the arithmetic of the critical path (gradient accumulation, selection, optimiser step) so that what
  // remains is the cost of the pipeline itself: copies, barriers, scheduling, exchange of empty streams.  The
  // reference has this as the compile-time switch SKIP_SOME_CRITICAL_PATHS (backend/src/engine/config.h:35-67).
  // Also set by STELLATRAIN_SKIP_CRITICAL_PATHS=1.  Parameters do not change in this mode.
  bool skip_critical_paths = false;
};

struct SharedParamEntry;       // row of the parameter table in shared memory

// Stage ids of the node-wide task barriers.
enum BarrierStage : int { kAfterCopyIn = 0, kAfterGather = 1, kAfterOptimize = 2, kAfterCopyOut = 3, kCheckerBase = 16 };

class CpuEngine;

// A pipeline stage ("module" in the reference, backend/src/engine/modules/module.h:18-34).
class Module {
 public:
  virtual ~Module() = default;
  virtual const char* name() const = 0;
  virtual void run(CpuEngine& engine, const std::shared_ptr<TrainTask>& task) = 0;
};

class CpuEngine {
 public:
  CpuEngine();
  ~CpuEngine();

  // ---- lifecycle and configuration
  void configure(const EngineOptions& opt);
  bool ready() const { return ready_; }
  const EngineOptions& options() const { return opt_; }
  bool node_master() const { return opt_.local_rank == 0; }
  void set_optimizer(const std::string& name);
  SparseOptimizer* sparse_optimizer() { return optimizer_.get(); }
  void configure_compression(const std::string& method);
  void configure_compression_ratio(double ratio);
  double compression_ratio() const;
  // The ratio that tasks of iteration `iter` and later will use (iterations count per parameter from 0 and agree
  // between nodes, so every node switches at the same task: the instruction protocol of the controller, effective a
  // few iterations after issue, backend/src/engine/batch_rate_alloc_optim.py:454-479).  A task's ratio is fixed when
  // the task is created; configure_compression_ratio() changes it for every task created afterwards.
  void configure_compression_ratio_from(int64_t iter, double ratio);
  double compression_ratio_at(int64_t iter) const;
  // Wire format of the gradient messages between nodes.  `blocks`: whole aligned runs of 16 indices travel as one
  // block id (what threshold-v16 selects).  `value_format`: 0 fp32, 1 fp16, 2 bf16; with 1 or 2 the compress stage
  // keeps the rounding error of every sent value in the residual, so narrow values delay mass instead of losing it.
  // Every node must use the same value format (the block form is self-describing).
  // Weight of every node's stream in the merge, indexed by node rank (default: 1 / nodes each, the reference's mean,
  // backend/src/engine/modules/cpu_optimize.cpp:55).  With unequal batch sizes per node the share of the global batch
  // keeps the merged gradient unbiased.  Counts from iteration `from_iter` on (same rule as the ratio switch); every
  // node must be given the same weights for the same iteration.
  void set_node_weights(const std::vector<float>& weights, int64_t from_iter = 0);
  std::vector<float> node_weights_at(int64_t iter) const;
  void configure_wire(bool blocks, int value_format);
  bool wire_blocks() const { return wire_blocks_; }
  int wire_value_format() const { return wire_values_; }
  int gradient_accumulation() const { return opt_.grad_accumulation; }
  void barrier();               // all processes of all nodes
  void synchronize();           // flush the pipeline (throws on failed tasks)
  std::string stats_json(bool clear);

  // ---- per-parameter protocol
  // Registers a parameter (same order in every process).  `user_param` may be null when the caller
  // moves data itself; the master copy then starts from `init_values` (numel floats, read during the call; zeros
  // when null too).  With more than one node every node's master copy takes rank 0's values.  Returns the
  // parameter index.
  int pre_train_init(int layer, const std::string& name, uint32_t numel, float* user_param,
                     const float* init_values = nullptr);
  void pre_forward_process(int param_index);
  // `grad` is a host pointer with numel floats; it is accumulated into this process's slot of the
  // current iteration.  The last micro-iteration starts the pipeline.
  void post_backward_process(int param_index, const float* grad);
  // Callers that copy by themselves:
  float* grad_slot(int param_index);              // where to put this iteration's gradient (zeroed by the engine)
  // Same, for a caller whose copy into the slot completes later (an asynchronous device copy): hands out the slots
  // of successive iterations in turn, so a second backward pass that is issued before the first copy has been
  // reported cannot be given the same slot.  One claim per iteration, followed by post_backward_in_slot().
  float* claim_grad_slot(int param_index);
  void post_backward_in_slot(int param_index);    // gradient already is in grad_slot()
  const float* master_param(int param_index) const;
  // Error-feedback residual of a parameter in shared memory (reference get_grad_residual, core_module_api.cpp:516-526);
  // written by the node master's compress stage, readable by every local process.
  float* grad_residual(int param_index) { return params_.at(param_index).resid; }
  // Stage timers of a task, as the stages themselves use them (reference record_stat_start/end, core_module_api.cpp:504-514)
  void record_stat_start(const std::shared_ptr<TrainTask>& t, const std::string& event) { t->stat_start(event); }
  void record_stat_end(const std::shared_ptr<TrainTask>& t, const std::string& event) { t->stat_end(event); }
  // Updates whose parameters are ready to be copied out by the caller: (param_index, iteration)
  std::vector<std::pair<int, int64_t>> pop_ready_updates(int max_wait_ms);
  void copy_out_done(int param_index, int64_t iter);
  // ---- device copies done by the engine itself (the reference's D2H_Copy and H2D_Copy stages)
  // True when a CUDA runtime (or a replacement table, see cuda_api.h) is available.
  bool device_copies_available() const;
  // The parameter's copy on the device: CopyOut then writes the master copy there on one of the engine's copy streams
  // and the task goes on when the stream has reached that point (schedule_after_cuda).
  void attach_device_param(int param_index, void* device_param);
  // The accumulated gradient of the last micro-iteration, on the device.  An event on `producer_stream` orders
  // the copy after the kernels that wrote the gradient; the copy runs on the parameter's copy stream into the pinned
  // slot and the pipeline starts from a host callback behind it.  The caller keeps `device_grad` alive until that
  // stream has passed the copy.  `copy_stream` may be null: the engine then uses a stream of its own.
  void post_backward_device(int param_index, const void* device_grad, void* producer_stream, void* copy_stream);
  // ---- bundles: several small tensors registered as ONE parameter, so that they share one task per iteration
  // A model like ResNet-152 has hundreds of tensors of a few hundred elements; each task costs the same handful of
  // barriers, wake-ups and callbacks whatever its size.  A bundle is a parameter whose elements are the members laid
  // end to end at `offsets` (multiples of 16, so that aligned blocks of a member stay aligned in the bundle; the
  // gaps stay zero).  Selection keeps the per-tensor rule: every member is compressed by itself, with its own k and
  // its own threshold under its own key, and the streams are joined.  Everything else (slots, gather, exchange,
  // merge, optimiser state, master copy) treats the bundle as one flat parameter.
  // `user_params[m]` (host tensors; may be null) is where the engine writes member m's updated values.
  void set_param_members(int param_index, const std::vector<std::string>& keys, const std::vector<uint32_t>& offsets,
                         const std::vector<uint32_t>& numels, const std::vector<float*>& user_params);
  // Host gradient of one member; the bundle's micro-iteration counts once every member has reported.
  void post_backward_member(int param_index, int member, const float* grad);
  void attach_device_members(int param_index, const std::vector<void*>& device_params);
  // Accumulated device gradients of all members (same order as the members): one event, one stream wait, one copy
  // per member into the pinned slot, one host callback that starts the task.
  void post_backward_device_members(int param_index, const std::vector<const void*>& device_grads, void* producer_stream,
                                    void* copy_stream);
  double force_model_sync(int param_index, bool dry_run);
  int64_t model_version(int param_index) const;
  int num_params() const { return static_cast<int>(params_.size()); }

  // ---- module API used by the stages
  void schedule(Module* m, const std::shared_ptr<TrainTask>& t);
  void schedule_after_barrier(Module* m, const std::shared_ptr<TrainTask>& t, int stage_id);
  void schedule_after_comm(Module* m, const std::shared_ptr<TrainTask>& t, const std::string& key, int slot);
  void schedule_after_model_complete(Module* m, const std::shared_ptr<TrainTask>& t);
  // Runs `m` once `stream` has finished the work enqueued so far (a host callback in the stream; reference
  // core_module_api.cpp:201-277).  Without a CUDA runtime the stage runs at once.
  void schedule_after_cuda(Module* m, const std::shared_ptr<TrainTask>& t, void* stream);
  void* copy_stream_for(int param_index);
  // Makes the engine's CUDA device current in the calling thread (pool workers start on device 0).
  void use_engine_device();
  // Runs `m` once the previous iteration of the same parameter has left its optimise stage:
  // residual, optimiser state and master parameter are per-parameter state that iteration i+1 must
  // see as iteration i left it.
  void schedule_after_previous(Module* m, const std::shared_ptr<TrainTask>& t);
  void mark_sequenced(const std::shared_ptr<TrainTask>& t);
  // Runs `m` (the optimise stage, the only writer of the master parameter) once the copy-out of the previous
  // iteration has finished reading the master: otherwise the copy handed to the framework could mix two updates,
  // differently in every local process.  mark_master_read is called when that copy is complete.
  void schedule_after_master_free(Module* m, const std::shared_ptr<TrainTask>& t);
  void mark_master_read(const std::shared_ptr<TrainTask>& t);
  void schedule_after_use(Module* m, const std::shared_ptr<TrainTask>& t);
  void return_after_use(const std::shared_ptr<TrainTask>& t);
  void schedule_terminate(const std::shared_ptr<TrainTask>& t);
  void update_model_version(const std::shared_ptr<TrainTask>& t);
  void fail_task(const std::shared_ptr<TrainTask>& t, const std::string& why);

  // accessors for stages
  ShmManager& shm() { return *shm_; }
  CommManager* comm() { return comm_.get(); }
  ThreadPool& pool() { return *pool_; }
  Compressor& compressor() { return *compressor_; }
  struct Member {
    std::string key;                         // "{layer}@{name}" of the tensor: names its threshold state
    uint32_t off = 0, numel = 0;
    float* user_param = nullptr;
    void* device_param = nullptr;
  };
  struct ParamLocal {
    int layer = 0;
    std::string name;
    uint32_t numel = 0;
    float* user_param = nullptr;
    float* master = nullptr;                 // shared master copy
    float* resid = nullptr;                  // shared residual (node master writes)
    std::vector<float*> slot[2];             // [iter % 2][local rank]
    int64_t iteration_cnt = 0;               // forwards seen
    int64_t model_version = 0;               // updates applied
    int64_t alloc_cnt = 0;                   // backwards (tasks) created
    int64_t completed_version = -1;
    int64_t sequenced_iter = -1;             // last iteration that left the optimise stage
    int64_t master_read_iter = -1;           // last iteration whose copy-out has finished reading the master
    int micro = 0;
    int64_t claim_cnt = 0;                   // gradient slots handed out by claim_grad_slot
    void* device_param = nullptr;            // set by attach_device_param
    void* grad_event = nullptr;              // orders the device-to-host copy after the backward kernels
    void* last_copy_stream = nullptr;        // stream of the latest device-to-host copy of this parameter
    bool checked_barrier = false;
    std::vector<Member> members;             // empty: a plain parameter
    int members_seen = 0;                    // members that reported their gradient in this micro-iteration
    std::vector<float> merge_scratch;        // node master: dense accumulator of the merge
    std::vector<uint8_t> merge_touched;
  };
  ParamLocal& param(int index) { return params_[index]; }
  Module* module(const std::string& name) { return modules_.at(name).get(); }
  void push_ready_update(int param_index, int64_t iter);

 private:
  struct GradPart { const void* src; uint32_t off, numel; };
  void copy_device_grads(int param_index, const std::vector<GradPart>& parts, void* producer_stream, void* copy_stream);
  void load_modules();
  void barrier_manager_main();
  void start_task(int param_index);
  void notify_layer_usage_finished(ParamLocal& p, int64_t iter);
  std::string describe_task(const std::string& key);

  EngineOptions opt_;
  std::atomic<bool> ready_{false};
  std::atomic<bool> stop_{false};
  mutable std::mutex ratio_mu_;
  double ratio_ = 0.99;
  std::map<int64_t, double> ratio_from_;     // first iteration -> ratio, for switches that lie ahead
  std::map<int64_t, std::vector<float>> weights_from_;   // first iteration -> per-node merge weights
  std::atomic<bool> wire_blocks_{true};
  std::atomic<int> wire_values_{0};
  std::unique_ptr<ThreadPool> pool_;
  std::unique_ptr<ShmManager> shm_;
  std::unique_ptr<CommManager> comm_;
  std::unique_ptr<Compressor> compressor_;
  std::unique_ptr<SparseOptimizer> optimizer_;
  std::map<std::string, std::unique_ptr<Module>> modules_;
  SharedParamEntry* table_ = nullptr;
  uint32_t* table_count_ = nullptr;
  std::vector<ParamLocal> params_;

  // barrier manager
  struct PendingBarrier {
    uint64_t key;
    Module* next;
    std::shared_ptr<TrainTask> task;
    std::chrono::steady_clock::time_point deadline;
  };
  std::thread barrier_thread_;
  std::mutex barrier_mu_;
  std::list<PendingBarrier> pending_barriers_;

  // model-version gates
  std::mutex version_mu_;
  std::condition_variable version_cv_;
  // by parameter: a new backward pass of a parameter can only release tasks of that parameter, so start_task looks at
  // one short list instead of at every waiting task of the model
  std::map<int, std::list<std::pair<Module*, std::shared_ptr<TrainTask>>>> waiting_model_;
  std::list<std::pair<Module*, std::shared_ptr<TrainTask>>> waiting_prev_;
  std::list<std::pair<Module*, std::shared_ptr<TrainTask>>> waiting_master_;

  // exclusive use of (parameter, slot)
  std::mutex use_mu_;
  std::map<std::string, bool> in_use_;
  std::map<std::string, std::list<std::pair<Module*, std::shared_ptr<TrainTask>>>> use_waiters_;

  // bookkeeping
  std::mutex tasks_mu_;
  std::map<std::string, std::shared_ptr<TrainTask>> tasks_;
  std::list<std::pair<std::string, std::shared_future<void>>> futures_;
  std::map<std::string, std::shared_ptr<std::promise<void>>> promises_;
  std::string first_error_;
  std::mutex stats_mu_;
  std::list<std::pair<std::string, std::map<std::string, double>>> stat_ring_;   // bounded history

  // device copies
  std::mutex copy_mu_;
  std::vector<void*> copy_streams_;
  int device_ = -1;                          // CUDA device of the thread that attached the first device parameter
  std::atomic<int> callbacks_in_flight_{0};
  std::atomic<int> grad_copies_pending_{0};    // gradient copies whose task has not been created yet
  // Continuations behind device copies run here, in the order in which their host callbacks fired: the callback itself
  // (a thread of the CUDA runtime, which holds back the stream while it runs) only appends to this queue.
  std::thread after_cuda_thread_;
  std::mutex after_cuda_mu_;
  std::condition_variable after_cuda_cv_;
  std::deque<std::function<void()>> after_cuda_q_;
  bool after_cuda_stop_ = false;
 public:
  void run_after_cuda(std::function<void()> fn);      // called by the host callback
 private:
  void after_cuda_main();

  std::mutex ready_mu_;
  std::condition_variable ready_cv_;
  std::list<std::pair<int, int64_t>> ready_updates_;
};

}  // namespace stc
