#include "engine.h"

#include <pthread.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <sstream>
#include <stdexcept>

#include "../cpu/array_util.h"
#include "config.h"
#include "cuda_api.h"
#include "logger.h"

namespace stc {

struct SharedParamEntry {
  char name[cfg::kMaxNameLen + 1];
  uint32_t numel;
  uint32_t ready;      // 0 absent, 1 allocated and initialised locally, 2 synchronised across nodes
  uint64_t master_off, resid_off;
  uint64_t slot_off[2][cfg::kMaxLocalRanks];
};

using Clock = std::chrono::steady_clock;

CpuEngine::CpuEngine() = default;

CpuEngine::~CpuEngine() {
  stop_ = true;
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    version_cv_.notify_all();
  }
  if (barrier_thread_.joinable()) barrier_thread_.join();
  if (const CudaApi* api = cuda_api()) {
    // host callbacks still queued in a copy stream refer to this object
    for (void* s : copy_streams_) api->stream_synchronize(s);
    for (int i = 0; i < 2000 && callbacks_in_flight_.load() > 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    for (void* s : copy_streams_) api->stream_destroy(s);
    for (auto& p : params_) if (p.grad_event) api->event_destroy(p.grad_event);
  }
  {
    std::lock_guard<std::mutex> lk(after_cuda_mu_);
    after_cuda_stop_ = true;
  }
  after_cuda_cv_.notify_all();
  if (after_cuda_thread_.joinable()) after_cuda_thread_.join();
  pool_.reset();      // joins the workers before the memory they use goes away
  comm_.reset();
  shm_.reset();
}

// ---------------------------------------------------------------- configuration
void CpuEngine::configure(const EngineOptions& o) {
  if (ready_) throw std::runtime_error("engine is already configured");
  if (o.local_world < 1 || o.local_world > cfg::kMaxLocalRanks) throw std::invalid_argument("local_world out of range");
  if (o.staleness < 0 || o.staleness > 1) throw std::invalid_argument("staleness must be 0 or 1");
  opt_ = o;
  if (cfg::env_long("STELLATRAIN_SKIP_CRITICAL_PATHS", 0) != 0) opt_.skip_critical_paths = true;
  {
    std::lock_guard<std::mutex> lk(ratio_mu_);
    ratio_ = o.ratio;
  }
  const int workers = o.workers > 0 ? o.workers : (node_master() ? cfg::kWorkersNodeMaster : cfg::kWorkersOther);
  pool_ = std::make_unique<ThreadPool>(static_cast<size_t>(workers));
  const size_t data_bytes = o.data_bytes ? o.data_bytes : static_cast<size_t>(cfg::env_long("STELLATRAIN_SHM_BYTES", static_cast<long>(cfg::kShmDataBytes)));
  const size_t meta_bytes = o.meta_bytes ? o.meta_bytes : cfg::kShmMetaBytes;
  shm_ = std::make_unique<ShmManager>(node_master(), o.session, o.local_rank, o.local_world, data_bytes, meta_bytes, o.timeout_ms);
  const size_t table_bytes = 64 + sizeof(SharedParamEntry) * cfg::kMaxParams;
  unsigned char* base;
  if (node_master()) {
    base = static_cast<unsigned char*>(shm_->alloc_meta(table_bytes));
    std::memset(base, 0, table_bytes);
    if (base != shm_->meta_first()) throw std::logic_error("parameter table is not the first metadata allocation");
  } else {
    base = static_cast<unsigned char*>(shm_->meta_first());
  }
  table_count_ = reinterpret_cast<uint32_t*>(base);
  table_ = reinterpret_cast<SharedParamEntry*>(base + 64);
  if (o.pin_cuda) shm_->pin_for_cuda();
  compressor_ = make_compressor(o.method, pool_.get());
  optimizer_ = make_optimizer("sgd");
  optimizer_->set_pool(pool_.get());
  load_modules();
  if (o.world > 1 && node_master()) {
    comm_ = std::make_unique<CommManager>(o.master_addr, o.master_port, o.timeout_ms);
    if (o.rank == 0) comm_->start_server(o.world);
    if (!comm_->start_client(o.rank, o.world, o.local_world)) throw std::runtime_error("comm start failed: " + comm_->failure());
  }
  if (!shm_->barrier(o.timeout_ms)) throw std::runtime_error("local processes did not all reach configure()");
  barrier_thread_ = std::thread([this] { barrier_manager_main(); });
  ready_ = true;
}

void CpuEngine::set_optimizer(const std::string& name) {
  optimizer_ = make_optimizer(name);
  optimizer_->set_pool(pool_.get());
}

void CpuEngine::configure_compression(const std::string& method) { compressor_ = make_compressor(method, pool_.get()); }

void CpuEngine::configure_compression_ratio(double ratio) {
  if (!(ratio > 0.0 && ratio <= 1.0)) throw std::invalid_argument("compression ratio must be in (0, 1]");
  std::lock_guard<std::mutex> lk(ratio_mu_);
  ratio_ = ratio;
  ratio_from_.clear();
}

double CpuEngine::compression_ratio() const {
  std::lock_guard<std::mutex> lk(ratio_mu_);
  return ratio_;
}

void CpuEngine::configure_compression_ratio_from(int64_t iter, double ratio) {
  if (!(ratio > 0.0 && ratio <= 1.0)) throw std::invalid_argument("compression ratio must be in (0, 1]");
  std::lock_guard<std::mutex> lk(ratio_mu_);
  ratio_from_[iter] = ratio;
}

double CpuEngine::compression_ratio_at(int64_t iter) const {
  std::lock_guard<std::mutex> lk(ratio_mu_);
  double r = ratio_;
  for (auto& kv : ratio_from_) {       // ordered by iteration: the last switch at or before `iter` wins
    if (kv.first > iter) break;
    r = kv.second;
  }
  return r;
}

void CpuEngine::set_node_weights(const std::vector<float>& weights, int64_t from_iter) {
  if (static_cast<int>(weights.size()) != opt_.world) throw std::invalid_argument("one weight per node is needed");
  for (float w : weights)
    if (!(w >= 0.f) || !std::isfinite(w)) throw std::invalid_argument("weights must be finite and not negative");
  std::lock_guard<std::mutex> lk(ratio_mu_);
  weights_from_[from_iter] = weights;
}

std::vector<float> CpuEngine::node_weights_at(int64_t iter) const {
  std::lock_guard<std::mutex> lk(ratio_mu_);
  std::vector<float> w(static_cast<size_t>(std::max(1, opt_.world)), 1.0f / static_cast<float>(std::max(1, opt_.world)));
  for (auto& kv : weights_from_) {
    if (kv.first > iter) break;
    w = kv.second;
  }
  return w;
}

void CpuEngine::configure_wire(bool blocks, int value_format) {
  if (value_format < 0 || value_format > 2) throw std::invalid_argument("value format must be 0 (fp32), 1 (fp16) or 2 (bf16)");
  wire_blocks_ = blocks;
  wire_values_ = value_format;
}

void CpuEngine::barrier() {
  if (!shm_->barrier(opt_.timeout_ms)) throw std::runtime_error("node barrier timed out");
  if (comm_ && !comm_->global_barrier()) throw std::runtime_error("global barrier timed out");
  if (!shm_->barrier(opt_.timeout_ms)) throw std::runtime_error("node barrier timed out");
}

// ---------------------------------------------------------------- registration
int CpuEngine::pre_train_init(int layer, const std::string& name, uint32_t numel, float* user_param, const float* init_values) {
  if (!ready_) throw std::runtime_error("configure() first");
  const int index = static_cast<int>(params_.size());
  if (index >= cfg::kMaxParams) throw std::runtime_error("too many parameters");
  const std::string pkey = std::to_string(layer) + "@" + name;
  if (static_cast<int>(pkey.size()) > cfg::kMaxNameLen) throw std::runtime_error("parameter key too long: " + pkey);
  SharedParamEntry* e = &table_[index];
  const int N = opt_.local_world;
  if (node_master()) {
    std::strncpy(e->name, pkey.c_str(), cfg::kMaxNameLen);
    e->numel = numel;
    const size_t bytes = static_cast<size_t>(numel) * sizeof(float);
    float* master = static_cast<float*>(shm_->alloc(bytes));
    float* resid = static_cast<float*>(shm_->alloc(bytes));
    std::memset(resid, 0, bytes);
    const float* init = init_values ? init_values : user_param;
    if (init) std::memcpy(master, init, bytes); else std::memset(master, 0, bytes);
    e->master_off = shm_->offset_of(master);
    e->resid_off = shm_->offset_of(resid);
    for (int s = 0; s < 2; ++s)
      for (int r = 0; r < N; ++r) {
        float* g = static_cast<float*>(shm_->alloc(bytes));
        std::memset(g, 0, bytes);
        e->slot_off[s][r] = shm_->offset_of(g);
      }
    __atomic_store_n(&e->ready, 1u, __ATOMIC_RELEASE);
    // every node starts from rank 0's values (reference core.cpp:841-885)
    if (comm_) {
      const std::string key = "init@" + pkey;
      const bool ok = opt_.rank == 0 ? comm_->send_init_model(key, master, numel) : comm_->recv_init_model(key, master, numel);
      if (!ok) throw std::runtime_error("initial model exchange failed for " + pkey);
    }
    __atomic_store_n(&e->ready, 2u, __ATOMIC_RELEASE);
    __atomic_store_n(table_count_, static_cast<uint32_t>(index + 1), __ATOMIC_RELEASE);
  } else {
    const auto t0 = Clock::now();
    while (__atomic_load_n(&e->ready, __ATOMIC_ACQUIRE) != 2u) {
      if (Clock::now() - t0 > std::chrono::milliseconds(opt_.timeout_ms))
        throw std::runtime_error("node master never registered parameter " + pkey);
      std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    if (pkey != e->name || e->numel != numel)
      throw std::runtime_error("parameter registration order differs between local processes at " + pkey);
  }
  ParamLocal p;
  p.layer = layer;
  p.name = name;
  p.numel = numel;
  p.user_param = user_param;
  p.master = static_cast<float*>(shm_->from_offset(e->master_off));
  p.resid = static_cast<float*>(shm_->from_offset(e->resid_off));
  for (int s = 0; s < 2; ++s)
    for (int r = 0; r < N; ++r) p.slot[s].push_back(static_cast<float*>(shm_->from_offset(e->slot_off[s][r])));
  if (user_param) std::memcpy(user_param, p.master, static_cast<size_t>(numel) * sizeof(float));
  params_.push_back(std::move(p));
  return index;
}

const float* CpuEngine::master_param(int index) const { return params_.at(index).master; }

int64_t CpuEngine::model_version(int index) const { return params_.at(index).model_version; }

// ---------------------------------------------------------------- forward gate
void CpuEngine::pre_forward_process(int index) {
  ParamLocal& p = params_.at(index);
  std::unique_lock<std::mutex> lk(version_mu_);
  const int64_t j = p.iteration_cnt++;
  const int64_t need = j - opt_.staleness;
  const bool ok = version_cv_.wait_for(lk, std::chrono::milliseconds(opt_.timeout_ms), [&] {
    return stop_ || !first_error_.empty() || p.model_version >= need;
  });
  if (!first_error_.empty()) throw std::runtime_error("pipeline failed: " + first_error_);
  if (!ok) throw std::runtime_error("timed out waiting for update " + std::to_string(need) + " of " + p.name);
}

// ---------------------------------------------------------------- backward
float* CpuEngine::grad_slot(int index) {
  ParamLocal& p = params_.at(index);
  return p.slot[p.alloc_cnt % 2][opt_.local_rank];
}

float* CpuEngine::claim_grad_slot(int index) {
  ParamLocal& p = params_.at(index);
  return p.slot[p.claim_cnt++ % 2][opt_.local_rank];
}

// ---------------------------------------------------------------- device copies
namespace {
constexpr int kCopyStreams = 4;

struct AfterCuda {
  CpuEngine* engine;
  std::function<void()> fn;
  std::atomic<int>* in_flight;
};

// Runs on a thread of the CUDA runtime, in stream order, and the stream does not go on until it returns: it must not
// call the runtime and has to be short.  It only hands the continuation to the engine's own thread, which runs the
// continuations in the order in which they were handed over (two callbacks of one parameter keep the order of their
// copies).
void after_cuda_trampoline(void* user) {
  std::unique_ptr<AfterCuda> a(static_cast<AfterCuda*>(user));
  std::atomic<int>* in_flight = a->in_flight;
  std::function<void()> fn = std::move(a->fn);
  a->engine->run_after_cuda([fn = std::move(fn), in_flight] {
    try {
      fn();
    } catch (const std::exception& e) {
      LOG_ERROR("CpuEngine", "continuation behind a device copy failed: " << e.what());
    }
    in_flight->fetch_sub(1);
  });
}
}  // namespace

void CpuEngine::run_after_cuda(std::function<void()> fn) {
  {
    std::lock_guard<std::mutex> lk(after_cuda_mu_);
    if (!after_cuda_thread_.joinable()) after_cuda_thread_ = std::thread([this] { after_cuda_main(); });
    after_cuda_q_.push_back(std::move(fn));
  }
  after_cuda_cv_.notify_one();
}

void CpuEngine::after_cuda_main() {
  pthread_setname_np(pthread_self(), "AfterCuda");
  for (;;) {
    std::function<void()> fn;
    {
      std::unique_lock<std::mutex> lk(after_cuda_mu_);
      after_cuda_cv_.wait(lk, [this] { return after_cuda_stop_ || !after_cuda_q_.empty(); });
      if (after_cuda_q_.empty()) return;       // stop requested and nothing left
      fn = std::move(after_cuda_q_.front());
      after_cuda_q_.pop_front();
    }
    fn();
  }
}

bool CpuEngine::device_copies_available() const { return cuda_api() != nullptr; }

void* CpuEngine::copy_stream_for(int index) {
  const CudaApi* api = cuda_api();
  if (!api) return nullptr;
  use_engine_device();
  std::lock_guard<std::mutex> lk(copy_mu_);
  if (copy_streams_.empty()) {
    for (int i = 0; i < kCopyStreams; ++i) {
      void* s = nullptr;
      if (api->stream_create(&s) != 0) throw std::runtime_error("could not create a copy stream");
      copy_streams_.push_back(s);
    }
  }
  return copy_streams_[static_cast<size_t>(index) % copy_streams_.size()];
}

void CpuEngine::attach_device_param(int index, void* device_param) {
  const CudaApi* api = cuda_api();
  if (!api) throw std::runtime_error("attach_device_param: no CUDA runtime in this process");
  if (device_ < 0 && api->get_device(&device_) != 0) throw std::runtime_error("cudaGetDevice failed");
  params_.at(index).device_param = device_param;
}

void CpuEngine::use_engine_device() {
  thread_local int current = -1;
  if (device_ < 0 || current == device_) return;
  if (const CudaApi* api = cuda_api())
    if (api->set_device(device_) == 0) current = device_;
}

void CpuEngine::post_backward_device(int index, const void* device_grad, void* producer_stream, void* copy_stream) {
  ParamLocal& p = params_.at(index);
  if (!p.members.empty()) throw std::runtime_error("post_backward_device: parameter is a bundle, hand in every member");
  copy_device_grads(index, {{device_grad, 0u, p.numel}}, producer_stream, copy_stream);
}

void CpuEngine::post_backward_device_members(int index, const std::vector<const void*>& device_grads, void* producer_stream,
                                             void* copy_stream) {
  ParamLocal& p = params_.at(index);
  if (device_grads.size() != p.members.size() || p.members.empty())
    throw std::runtime_error("post_backward_device_members: one gradient per member");
  std::vector<GradPart> parts;
  parts.reserve(p.members.size());
  for (size_t m = 0; m < p.members.size(); ++m) parts.push_back({device_grads[m], p.members[m].off, p.members[m].numel});
  copy_device_grads(index, parts, producer_stream, copy_stream);
}

void CpuEngine::copy_device_grads(int index, const std::vector<GradPart>& parts, void* producer_stream, void* copy_stream) {
  const CudaApi* api = cuda_api();
  if (!api) throw std::runtime_error("post_backward_device: no CUDA runtime in this process");
  ParamLocal& p = params_.at(index);
  if (!copy_stream) copy_stream = copy_stream_for(index);
  if (!p.grad_event && api->event_create(&p.grad_event) != 0) throw std::runtime_error("could not create an event");
  float* slot = claim_grad_slot(index);
  p.last_copy_stream = copy_stream;
  const int reps = opt_.grad_accumulation;   // the device accumulated the micro-iterations: one copy stands for all
  auto* after = new AfterCuda{this, [this, index, reps] {
    try {
      for (int i = 0; i < reps; ++i) post_backward_in_slot(index);
    } catch (const std::exception& e) {
      LOG_ERROR("CpuEngine", "starting the task of parameter " << index << " failed: " << e.what());
    }
    grad_copies_pending_.fetch_sub(1);
  }, &callbacks_in_flight_};
  // in order, stopping at the first failure: a callback that was never enqueued must not be waited for
  int rc = api->event_record(p.grad_event, producer_stream);
  if (rc == 0) rc = api->stream_wait_event(copy_stream, p.grad_event);
  for (size_t i = 0; i < parts.size() && rc == 0; ++i)
    rc = api->memcpy_d2h_async(slot + parts[i].off, parts[i].src, static_cast<size_t>(parts[i].numel) * sizeof(float), copy_stream);
  if (rc == 0) {
    callbacks_in_flight_.fetch_add(1);
    grad_copies_pending_.fetch_add(1);
    rc = api->launch_host_func(copy_stream, after_cuda_trampoline, after);
    if (rc != 0) {
      callbacks_in_flight_.fetch_sub(1);
      grad_copies_pending_.fetch_sub(1);
    }
  }
  if (rc != 0) {
    delete after;
    --p.claim_cnt;      // the slot was not used
    throw std::runtime_error("a CUDA runtime call of the gradient copy failed with code " + std::to_string(rc));
  }
}

void CpuEngine::set_param_members(int index, const std::vector<std::string>& keys, const std::vector<uint32_t>& offsets,
                                  const std::vector<uint32_t>& numels, const std::vector<float*>& user_params) {
  ParamLocal& p = params_.at(index);
  if (p.alloc_cnt != 0 || p.iteration_cnt != 0) throw std::runtime_error("set_param_members: the parameter is already in use");
  if (keys.empty() || keys.size() != offsets.size() || keys.size() != numels.size() ||
      (!user_params.empty() && user_params.size() != keys.size()))
    throw std::runtime_error("set_param_members: lists of different lengths");
  uint64_t end = 0;
  std::vector<Member> members(keys.size());
  for (size_t m = 0; m < keys.size(); ++m) {
    if (offsets[m] % 16 != 0 || offsets[m] < end) throw std::runtime_error("set_param_members: offsets must ascend in steps of 16");
    end = static_cast<uint64_t>(offsets[m]) + numels[m];
    if (end > p.numel) throw std::runtime_error("set_param_members: members exceed the parameter");
    members[m].key = keys[m];
    members[m].off = offsets[m];
    members[m].numel = numels[m];
    members[m].user_param = user_params.empty() ? nullptr : user_params[m];
    if (members[m].user_param)
      std::memcpy(members[m].user_param, p.master + offsets[m], static_cast<size_t>(numels[m]) * sizeof(float));
  }
  p.members = std::move(members);
}

void CpuEngine::attach_device_members(int index, const std::vector<void*>& device_params) {
  const CudaApi* api = cuda_api();
  if (!api) throw std::runtime_error("attach_device_members: no CUDA runtime in this process");
  if (device_ < 0 && api->get_device(&device_) != 0) throw std::runtime_error("cudaGetDevice failed");
  ParamLocal& p = params_.at(index);
  if (device_params.size() != p.members.size() || p.members.empty())
    throw std::runtime_error("attach_device_members: one pointer per member");
  for (size_t m = 0; m < p.members.size(); ++m) p.members[m].device_param = device_params[m];
}

void CpuEngine::post_backward_member(int index, int member, const float* grad) {
  ParamLocal& p = params_.at(index);
  const Member& m = p.members.at(static_cast<size_t>(member));
  float* dst = grad_slot(index) + m.off;
  if (p.micro == 0) std::memcpy(dst, grad, static_cast<size_t>(m.numel) * sizeof(float));
  else add_arrays(dst, grad, m.numel);
  if (++p.members_seen < static_cast<int>(p.members.size())) return;
  p.members_seen = 0;
  post_backward_in_slot(index);
}

void CpuEngine::schedule_after_cuda(Module* next, const std::shared_ptr<TrainTask>& t, void* stream) {
  const CudaApi* api = cuda_api();
  if (!api) {
    schedule(next, t);
    return;
  }
  auto* after = new AfterCuda{this, [this, next, t] { schedule(next, t); }, &callbacks_in_flight_};
  callbacks_in_flight_.fetch_add(1);
  if (api->launch_host_func(stream, after_cuda_trampoline, after) != 0) {
    callbacks_in_flight_.fetch_sub(1);
    delete after;
    fail_task(t, "cudaLaunchHostFunc failed before " + std::string(next->name()));
  }
}

void CpuEngine::post_backward_process(int index, const float* grad) {
  ParamLocal& p = params_.at(index);
  float* slot = grad_slot(index);
  if (p.micro == 0) std::memcpy(slot, grad, static_cast<size_t>(p.numel) * sizeof(float));
  else add_arrays(slot, grad, p.numel);
  if (++p.micro < opt_.grad_accumulation) return;
  p.micro = 0;
  start_task(index);
}

void CpuEngine::post_backward_in_slot(int index) {
  ParamLocal& p = params_.at(index);
  if (++p.micro < opt_.grad_accumulation) return;
  p.micro = 0;
  start_task(index);
}

void CpuEngine::notify_layer_usage_finished(ParamLocal& p, int64_t iter) {
  std::lock_guard<std::mutex> lk(version_mu_);
  p.completed_version = std::max<int64_t>(-1, iter - opt_.staleness);
}

void CpuEngine::start_task(int index) {
  ParamLocal& p = params_.at(index);
  const int64_t iter = p.alloc_cnt++;
  notify_layer_usage_finished(p, iter);
  auto task = std::make_shared<TrainTask>(iter, p.layer, p.name);
  task->numel = p.numel;
  task->param_index = index;
  task->ratio = compression_ratio_at(iter);
  task->stat_start("Total");
  auto prom = std::make_shared<std::promise<void>>();
  {
    std::lock_guard<std::mutex> lk(tasks_mu_);
    tasks_[task->key] = task;
    promises_[task->key] = prom;
    futures_.emplace_back(task->key, prom->get_future().share());
  }
  // tasks blocked on "previous version no longer in use" may be able to run now
  std::list<std::pair<Module*, std::shared_ptr<TrainTask>>> runnable;
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    auto mine = waiting_model_.find(index);
    if (mine != waiting_model_.end()) {
      for (auto it = mine->second.begin(); it != mine->second.end();) {
        if (p.completed_version >= it->second->iter) {
          runnable.push_back(*it);
          it = mine->second.erase(it);
        } else {
          ++it;
        }
      }
    }
  }
  for (auto& r : runnable) schedule(r.first, r.second);
  Module* first = opt_.debug_barrier && !p.checked_barrier ? module("BarrierChecker") : module("CopyIn");
  p.checked_barrier = true;
  schedule_after_use(first, task);
}

// ---------------------------------------------------------------- module API
void CpuEngine::schedule(Module* m, const std::shared_ptr<TrainTask>& t) {
  pool_->enqueue(t->priority(), [this, m, t] {
    if (t->state() == TaskState::Failed) return;
    try {
      t->stat_start(m->name());
      m->run(*this, t);
      t->stat_end(m->name());
    } catch (const std::exception& e) {
      fail_task(t, std::string(m->name()) + ": " + e.what());
    }
  });
}

void CpuEngine::fail_task(const std::shared_ptr<TrainTask>& t, const std::string& why) {
  LOG_ERROR("CpuEngine", "task " << t->key << " failed: " << why);
  t->fail(why);
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    if (first_error_.empty()) first_error_ = t->key + ": " + why;
    version_cv_.notify_all();
  }
  std::shared_ptr<std::promise<void>> prom;
  {
    std::lock_guard<std::mutex> lk(tasks_mu_);
    auto it = promises_.find(t->key);
    if (it != promises_.end()) { prom = it->second; promises_.erase(it); }
    tasks_.erase(t->key);
  }
  if (prom) prom->set_exception(std::make_exception_ptr(std::runtime_error(t->key + ": " + why)));
}

void CpuEngine::schedule_after_barrier(Module* next, const std::shared_ptr<TrainTask>& t, int stage_id) {
  const int N = opt_.local_world;
  if (N == 1) { schedule(next, t); return; }
  const uint64_t key = t->barrier_key(stage_id);
  if (shm_->arrive(key, N)) {
    shm_->depart(key, N);
    schedule(next, t);
    return;
  }
  std::lock_guard<std::mutex> lk(barrier_mu_);
  pending_barriers_.push_back({key, next, t, Clock::now() + std::chrono::milliseconds(opt_.timeout_ms)});
}

void CpuEngine::barrier_manager_main() {
  pthread_setname_np(pthread_self(), "BarrierManager");
  while (!stop_) {
    shm_->wait_change(5);
    std::list<PendingBarrier> done, late;
    {
      std::lock_guard<std::mutex> lk(barrier_mu_);
      const auto now = Clock::now();
      for (auto it = pending_barriers_.begin(); it != pending_barriers_.end();) {
        if (shm_->complete(it->key)) { done.push_back(*it); it = pending_barriers_.erase(it); }
        else if (now > it->deadline) { late.push_back(*it); it = pending_barriers_.erase(it); }
        else ++it;
      }
    }
    for (auto& b : done) {
      shm_->depart(b.key, opt_.local_world);
      schedule(b.next, b.task);
    }
    for (auto& b : late) fail_task(b.task, "a local process did not reach the barrier before " + std::string(b.next->name()));
  }
}

void CpuEngine::schedule_after_comm(Module* next, const std::shared_ptr<TrainTask>& t, const std::string& key, int slot) {
  if (!comm_) throw std::logic_error("schedule_after_comm without a comm manager");
  comm_->post_recv(key, [this, next, t, slot](SparseMessage&& m) {
    const size_t k = t->k;
    const size_t n = std::min(m.idx.size(), k);
    std::copy(m.idx.begin(), m.idx.begin() + static_cast<long>(n), t->idx.begin() + static_cast<long>(slot * k));
    std::copy(m.val.begin(), m.val.begin() + static_cast<long>(n), t->val.begin() + static_cast<long>(slot * k));
    t->counts[slot] = n;
    ++t->exchange_round;
    schedule(next, t);
  });
}

void CpuEngine::schedule_after_model_complete(Module* next, const std::shared_ptr<TrainTask>& t) {
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    if (params_[t->param_index].completed_version < t->iter) {
      waiting_model_[t->param_index].emplace_back(next, t);
      return;
    }
  }
  schedule(next, t);
}

void CpuEngine::schedule_after_previous(Module* next, const std::shared_ptr<TrainTask>& t) {
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    if (params_[t->param_index].sequenced_iter < t->iter - 1) {
      waiting_prev_.emplace_back(next, t);
      return;
    }
  }
  schedule(next, t);
}

void CpuEngine::mark_sequenced(const std::shared_ptr<TrainTask>& t) {
  std::pair<Module*, std::shared_ptr<TrainTask>> next{nullptr, nullptr};
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    params_[t->param_index].sequenced_iter = t->iter;
    for (auto it = waiting_prev_.begin(); it != waiting_prev_.end(); ++it)
      if (it->second->param_index == t->param_index && it->second->iter == t->iter + 1) {
        next = *it;
        waiting_prev_.erase(it);
        break;
      }
  }
  if (next.first) schedule(next.first, next.second);
}

void CpuEngine::schedule_after_master_free(Module* next, const std::shared_ptr<TrainTask>& t) {
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    if (params_[t->param_index].master_read_iter < t->iter - 1) {
      waiting_master_.emplace_back(next, t);
      return;
    }
  }
  schedule(next, t);
}

void CpuEngine::mark_master_read(const std::shared_ptr<TrainTask>& t) {
  std::pair<Module*, std::shared_ptr<TrainTask>> next{nullptr, nullptr};
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    auto& p = params_[t->param_index];
    p.master_read_iter = std::max(p.master_read_iter, t->iter);
    for (auto it = waiting_master_.begin(); it != waiting_master_.end(); ++it)
      if (it->second->param_index == t->param_index && it->second->iter <= p.master_read_iter + 1) {
        next = *it;
        waiting_master_.erase(it);
        break;
      }
  }
  if (next.first) schedule(next.first, next.second);
}

void CpuEngine::schedule_after_use(Module* next, const std::shared_ptr<TrainTask>& t) {
  const std::string slot_key = t->persistent_key + "#" + std::to_string(t->iter % 2);
  {
    std::lock_guard<std::mutex> lk(use_mu_);
    if (in_use_[slot_key]) {
      use_waiters_[slot_key].emplace_back(next, t);
      return;
    }
    in_use_[slot_key] = true;
  }
  schedule(next, t);
}

void CpuEngine::return_after_use(const std::shared_ptr<TrainTask>& t) {
  const std::string slot_key = t->persistent_key + "#" + std::to_string(t->iter % 2);
  std::pair<Module*, std::shared_ptr<TrainTask>> next{nullptr, nullptr};
  {
    std::lock_guard<std::mutex> lk(use_mu_);
    auto& q = use_waiters_[slot_key];
    if (q.empty()) in_use_[slot_key] = false;
    else { next = q.front(); q.pop_front(); }
  }
  if (next.first) schedule(next.first, next.second);
}

void CpuEngine::update_model_version(const std::shared_ptr<TrainTask>& t) {
  std::lock_guard<std::mutex> lk(version_mu_);
  ++params_[t->param_index].model_version;
  version_cv_.notify_all();
}

void CpuEngine::schedule_terminate(const std::shared_ptr<TrainTask>& t) {
  t->stat_end("Total");
  {
    std::lock_guard<std::mutex> lk(stats_mu_);
    stat_ring_.emplace_back(t->key, t->stats());
    if (stat_ring_.size() > 8192) stat_ring_.pop_front();   // bounded, unlike the reference's map
  }
  std::shared_ptr<std::promise<void>> prom;
  {
    std::lock_guard<std::mutex> lk(tasks_mu_);
    auto it = promises_.find(t->key);
    if (it != promises_.end()) { prom = it->second; promises_.erase(it); }
    tasks_.erase(t->key);
  }
  if (prom) prom->set_value();
}

void CpuEngine::push_ready_update(int index, int64_t iter) {
  std::lock_guard<std::mutex> lk(ready_mu_);
  ready_updates_.emplace_back(index, iter);
  ready_cv_.notify_all();
}

std::vector<std::pair<int, int64_t>> CpuEngine::pop_ready_updates(int max_wait_ms) {
  std::unique_lock<std::mutex> lk(ready_mu_);
  if (ready_updates_.empty() && max_wait_ms > 0)
    ready_cv_.wait_for(lk, std::chrono::milliseconds(max_wait_ms), [this] { return !ready_updates_.empty() || stop_; });
  std::vector<std::pair<int, int64_t>> out(ready_updates_.begin(), ready_updates_.end());
  ready_updates_.clear();
  return out;
}

void CpuEngine::copy_out_done(int index, int64_t iter) {
  ParamLocal& p = params_.at(index);
  std::shared_ptr<TrainTask> t;
  {
    std::lock_guard<std::mutex> lk(tasks_mu_);
    auto it = tasks_.find(std::to_string(iter) + "@" + std::to_string(p.layer) + "@" + p.name);
    if (it == tasks_.end()) throw std::runtime_error("copy_out_done for an unknown task");
    t = it->second;
  }
  // the caller has copied the master parameter out; the rest happens once every local process has
  schedule_after_barrier(module("CopyOutDone"), t, kAfterCopyOut);
}

// Where a task currently is: its state and the gate it waits at, for timeout messages.
std::string CpuEngine::describe_task(const std::string& key) {
  std::shared_ptr<TrainTask> t;
  {
    std::lock_guard<std::mutex> lk(tasks_mu_);
    auto it = tasks_.find(key);
    if (it == tasks_.end()) return "no longer tracked";
    t = it->second;
  }
  std::string where = std::string("state ") + task_state_name(t->state());
  auto holds = [&](const std::list<std::pair<Module*, std::shared_ptr<TrainTask>>>& l) {
    for (auto& e : l) if (e.second.get() == t.get()) return true;
    return false;
  };
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    for (auto& kv : waiting_model_)
      if (holds(kv.second)) where += ", waits for the previous version to be released";
    if (holds(waiting_prev_)) where += ", waits for the previous iteration of the parameter";
    if (holds(waiting_master_)) where += ", waits for the previous copy-out of the parameter";
  }
  {
    std::lock_guard<std::mutex> lk(use_mu_);
    for (auto& kv : use_waiters_) if (holds(kv.second)) where += ", waits for its gradient slot";
  }
  {
    std::lock_guard<std::mutex> lk(barrier_mu_);
    for (auto& b : pending_barriers_) if (b.task.get() == t.get()) where += ", waits at a node barrier";
  }
  where += ", " + std::to_string(pool_->pending()) + " jobs queued";
  return where;
}

// ---------------------------------------------------------------- synchronize
void CpuEngine::synchronize() {
  // gradient copies still in a stream have not started their tasks yet: wait for them first
  if (const CudaApi* api = cuda_api()) {
    std::vector<void*> streams;
    for (auto& p : params_)
      if (p.last_copy_stream && std::find(streams.begin(), streams.end(), p.last_copy_stream) == streams.end())
        streams.push_back(p.last_copy_stream);
    for (void* st : streams)
      if (api->stream_synchronize(st) != 0) throw std::runtime_error("a copy stream did not finish");
    // the host callbacks have fired; the tasks are created by the engine's own thread just behind them
    const auto limit = Clock::now() + std::chrono::milliseconds(opt_.timeout_ms);
    while (grad_copies_pending_.load() > 0) {
      if (Clock::now() > limit) throw std::runtime_error("tasks behind finished gradient copies were not created in time");
      std::this_thread::sleep_for(std::chrono::microseconds(100));
    }
  }
  // release every "previous version still in use" gate (reference core.cpp:910-922)
  std::list<std::pair<Module*, std::shared_ptr<TrainTask>>> runnable;
  {
    std::lock_guard<std::mutex> lk(version_mu_);
    for (auto& p : params_) p.completed_version = p.alloc_cnt - 1;
    for (auto& kv : waiting_model_) runnable.splice(runnable.end(), kv.second);
  }
  for (auto& r : runnable) schedule(r.first, r.second);
  std::list<std::pair<std::string, std::shared_future<void>>> futs;
  {
    std::lock_guard<std::mutex> lk(tasks_mu_);
    futs.swap(futures_);
  }
  std::string err;
  const auto deadline = Clock::now() + std::chrono::milliseconds(opt_.timeout_ms);
  for (auto& f : futs) {
    for (;;) {
      const auto st = f.second.wait_for(std::chrono::milliseconds(std::min(5000, std::max(100, opt_.timeout_ms / 4))));
      if (st == std::future_status::ready) break;
      LOG_WARN("CpuEngine", "waiting for " << f.first << " for more than 5 s (" << futs.size() << " tasks in flight)");
      if (comm_ && comm_->failed()) {
        err = "communication failed: " + comm_->failure();
        break;
      }
      if (Clock::now() > deadline) {
        err = "synchronize timed out on " + f.first + " (" + describe_task(f.first) + ")";
        break;
      }
    }
    if (!err.empty()) break;
    try {
      f.second.get();
    } catch (const std::exception& e) {
      if (err.empty()) err = e.what();
    }
  }
  if (!err.empty()) throw std::runtime_error(err);
}

// ---------------------------------------------------------------- model sync
double CpuEngine::force_model_sync(int index, bool dry_run) {
  ParamLocal& p = params_.at(index);
  double drift = 0.0;
  static std::atomic<uint64_t> serial{0};
  if (comm_ && node_master()) {
    const std::string key = "sync" + std::to_string(serial++) + "@" + std::to_string(p.layer) + "@" + p.name;
    if (opt_.rank == 0) {
      if (!comm_->send_init_model(key, p.master, p.numel)) throw std::runtime_error("model sync send failed");
    } else {
      std::vector<float> ref(p.numel);
      if (!comm_->recv_init_model(key, ref.data(), p.numel)) throw std::runtime_error("model sync receive failed");
      for (uint32_t i = 0; i < p.numel; ++i) drift = std::max(drift, static_cast<double>(std::fabs(ref[i] - p.master[i])));
      if (!dry_run) std::memcpy(p.master, ref.data(), static_cast<size_t>(p.numel) * sizeof(float));
    }
  }
  bool host_members = false;
  for (const Member& m : p.members) host_members = host_members || m.user_param != nullptr;
  if (!dry_run && (p.user_param || host_members)) {
    if (!shm_->barrier(opt_.timeout_ms)) throw std::runtime_error("node barrier timed out in model sync");
    if (p.user_param) std::memcpy(p.user_param, p.master, static_cast<size_t>(p.numel) * sizeof(float));
    for (const Member& m : p.members)
      if (m.user_param) std::memcpy(m.user_param, p.master + m.off, static_cast<size_t>(m.numel) * sizeof(float));
  }
  return drift;
}

// ---------------------------------------------------------------- stats
std::string CpuEngine::stats_json(bool clear) {
  std::lock_guard<std::mutex> lk(stats_mu_);
  std::ostringstream os;
  os << "{";
  bool first = true;
  for (auto& kv : stat_ring_) {
    os << (first ? "" : ",") << "\"" << kv.first << "\":{";
    bool f2 = true;
    for (auto& ev : kv.second) {
      os << (f2 ? "" : ",") << "\"" << ev.first << "\":" << ev.second;
      f2 = false;
    }
    os << "}";
    first = false;
  }
  os << "}";
  if (clear) stat_ring_.clear();
  return os.str();
}

}  // namespace stc
