// See native_engine.h.  This is the only translation unit of the extension that includes torch headers.
#include "native_engine.h"

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/autograd/function_hook.h>
#include <torch/csrc/autograd/python_variable.h>
#include <torch/csrc/autograd/variable.h>

#include <atomic>
#include <cstring>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>

namespace st {

namespace {

struct ParamRec {
  at::Tensor tensor;
  int bucket = 0;
  int seg = 0;
};

struct BucketRec {
  NativeBucketSpec spec;
  at::Tensor flat_grad;
  std::vector<int> params;
  int full = 0, pending = 0;
  int tab_slot = 0;
  std::vector<cudaEvent_t> tab_events;     // copy of ring row i has been enqueued behind this event
  std::vector<char> tab_event_set;
  std::vector<at::Tensor> held;            // gradients the coming select reads
  at::Tensor capture_row;                  // pinned row of gradient addresses of the running capture
  cudaEvent_t grad_ready = nullptr;
  cudaEvent_t apply_done = nullptr;
  bool apply_done_set = false;
  cudaEvent_t select_done = nullptr;       // the latest select of this bucket has read its gradients
  bool select_done_set = false;
  bool has_pending_apply = false;
  int64_t select_count = 0, apply_count = 0;
};

// Shared between the engine and its hooks: a hook that outlives the engine (a parameter that is still referenced
// somewhere) finds `alive` false and does nothing.
struct Shared {
  std::atomic<bool> alive{true};
  NativeEngine::Impl* impl = nullptr;
};

}  // namespace

struct NativeEngine::Impl {
  int device = 0;
  cudaStream_t sparse = nullptr;
  int staleness = 1, ga = 1;
  std::vector<BucketRec> buckets;
  std::vector<ParamRec> params;
  std::shared_ptr<Shared> shared;
  std::mutex mu;                 // hooks run on autograd's thread, control calls on the interpreter's
  bool capturing = false;
  std::vector<at::Tensor> capture_keep;
  struct Saved { int64_t sel, app; bool pending; };
  std::vector<Saved> capture_saved;
  int64_t kernels = 0, kernels_saved = 0;
  uint64_t shaped = 0, shaped_saved = 0;
  void* shaper = nullptr;
  uint64_t shaper_cap_ns = 0;
  std::atomic<int> error{0};

  void check(cudaError_t e) {
    if (e != cudaSuccess) {
      int expected = 0;
      error.compare_exchange_strong(expected, (int)e);
    }
  }

  uint64_t* row_of(BucketRec& b) {
    if (!capturing) return b.spec.table_host + (size_t)b.tab_slot * b.spec.seg_off.size();
    if (!b.capture_row.defined()) {
      // a row of the capture's own: the captured copy reads it on every replay, long after eager steps have moved
      // on through the ring
      b.capture_row = at::empty({(int64_t)b.spec.seg_off.size()}, at::TensorOptions().dtype(at::kLong).pinned_memory(true));
      std::memcpy(b.capture_row.data_ptr(), b.spec.table_host, b.spec.seg_off.size() * sizeof(uint64_t));
      capture_keep.push_back(b.capture_row);
    }
    return reinterpret_cast<uint64_t*>(b.capture_row.data_ptr());
  }

  void apply(BucketRec& b) {
    check(b.spec.handle->apply(sparse, 0));
    check(cudaEventRecord(b.apply_done, sparse));
    b.apply_done_set = true;
    b.has_pending_apply = false;
    b.apply_count += 1;
    kernels += b.spec.handle->apply_kernels();
  }

  void select(BucketRec& b) {
    BucketHandle* h = b.spec.select_handle ? b.spec.select_handle : b.spec.handle;
    if (b.spec.handle->has_group) {
      check(b.spec.handle->group_reduce(sparse));
      kernels += 3;
    }
    if (shaper != nullptr && b.spec.shaped_bytes) {
      check(launch_shape(static_cast<ShaperState*>(shaper), b.spec.shaped_bytes, shaper_cap_ns, sparse));
      shaped += b.spec.shaped_bytes;
      kernels += 1;
    }
    check(h->select(sparse));
    if (!capturing) {
      check(cudaEventRecord(b.select_done, sparse));
      b.select_done_set = true;
    }
    b.select_count += 1;
    kernels += h->select_kernels();
  }

  // The hook of parameter `pi`: called by autograd once the gradient has been accumulated into `.grad`.
  void on_grad(int pi, const at::Tensor& param) {
    std::lock_guard<std::mutex> lock(mu);
    ParamRec& pr = params[pi];
    BucketRec& b = buckets[pr.bucket];
    b.pending -= 1;
    if (b.spec.steal && b.pending < b.spec.n_params) {      // last micro-iteration: the gradient is final
      at::Tensor g = param.grad();
      const uint32_t off = b.spec.seg_off[pr.seg], numel = b.spec.seg_numel[pr.seg];
      if (!g.defined() || g.scalar_type() != at::kFloat || g.strides() != param.strides() ||
          (reinterpret_cast<uintptr_t>(g.data_ptr()) & 15u)) {
        // not the parameter's layout, or not aligned for 16-byte loads: through the flat buffer, which the previous
        // iteration's select may still have to read (see bucket_ready)
        if (!capturing && b.select_done_set) {
          c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
          check(cudaStreamWaitEvent(c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)device).stream(), b.select_done, 0));
        }
        at::Tensor flat = b.flat_grad.narrow(0, off, numel).as_strided(param.sizes(), param.strides());
        if (g.defined()) flat.copy_(g); else flat.zero_();
        g = flat;
      }
      row_of(b)[pr.seg] = reinterpret_cast<uint64_t>(g.data_ptr());
      b.held.push_back(std::move(g));
    }
    if (b.pending == 0) {
      b.pending = b.full;
      bucket_ready(b);
    }
  }

  void bucket_ready(BucketRec& b) {
    c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
    const c10::cuda::CUDAStream cur_s = c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)device);
    cudaStream_t cur = cur_s.stream();
    // Gradients of this bucket that autograd handed over: they are released at the end of this function, once the
    // select that reads them is in the sparse stream.  The allocator defers the reuse of a block that was recorded
    // on a stream only past the work that stream had been given when the block was freed, so a release in front of
    // the launch would leave the select reading memory that the next allocation may already have taken.
    std::vector<at::Tensor> release;
    if (b.spec.steal) {
      const size_t n = b.spec.seg_off.size();
      // The bucket has one table of gradient addresses on the device.  The select of the previous iteration reads it
      // in the sparse stream and may still be waiting there (for acknowledgements of a slow peer, for the link shaper)
      // when this iteration's backward pass gets here: the new addresses go in behind it.  Replays of a captured
      // iteration follow one another on their stream and need no such wait.
      if (!capturing && b.select_done_set) check(cudaStreamWaitEvent(cur, b.select_done, 0));
      check(cudaMemcpyAsync(b.spec.table_dev, row_of(b), n * sizeof(uint64_t), cudaMemcpyHostToDevice, cur));
      if (!capturing) {
        check(cudaEventRecord(b.tab_events[b.tab_slot], cur));
        b.tab_event_set[b.tab_slot] = 1;
        b.tab_slot = (b.tab_slot + 1) % b.spec.table_ring;
        // the copy that last used the next row must be done before the hooks rewrite it
        if (b.tab_event_set[b.tab_slot]) check(cudaEventSynchronize(b.tab_events[b.tab_slot]));
        const c10::cuda::CUDAStream sparse_s = c10::cuda::getStreamFromExternal(sparse, (c10::DeviceIndex)device);
        for (auto& g : b.held)   // the allocator must not reuse them before the select has read them
          c10::cuda::CUDACachingAllocator::recordStream(g.storage().data_ptr(), sparse_s);
        release.swap(b.held);
      } else {
        for (auto& g : b.held) capture_keep.push_back(std::move(g));   // a replay reads these addresses again
        b.held.clear();
      }
      for (int pi : b.params) params[pi].tensor.mutable_grad().reset();
    }
    check(cudaEventRecord(b.grad_ready, cur));
    check(cudaStreamWaitEvent(sparse, b.grad_ready, 0));
    if (staleness == 1 && b.has_pending_apply) apply(b);
    select(b);
    if (staleness == 0) apply(b);
    else b.has_pending_apply = true;
    release.clear();   // after the launches, see above
  }
};

namespace {

struct GradHook : public torch::autograd::PostAccumulateGradHook {
  std::shared_ptr<Shared> shared;
  int param = 0;
  std::unique_ptr<torch::autograd::PostAccumulateGradHook> before;   // hooks Python code had registered

  void operator()(const torch::autograd::Variable& tensor) override {
    if (before) (*before)(tensor);
    if (shared->alive.load(std::memory_order_acquire)) shared->impl->on_grad(param, tensor);
  }
};

at::Tensor tensor_of(PyObject* obj, const char* what) {
  if (obj == nullptr || !THPVariable_Check(obj)) throw std::runtime_error(std::string(what) + " must be a torch tensor");
  return THPVariable_Unpack(obj);
}

}  // namespace

NativeEngine::NativeEngine(int device, uint64_t sparse_stream, int staleness, int grad_accumulation) : impl_(new Impl) {
  impl_->device = device;
  impl_->sparse = reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(sparse_stream));
  impl_->staleness = staleness;
  impl_->ga = grad_accumulation < 1 ? 1 : grad_accumulation;
  impl_->shared = std::make_shared<Shared>();
  impl_->shared->impl = impl_;
}

NativeEngine::~NativeEngine() {
  remove_hooks();
  for (auto& b : impl_->buckets) {
    for (auto ev : b.tab_events) cudaEventDestroy(ev);
    if (b.grad_ready) cudaEventDestroy(b.grad_ready);
    if (b.apply_done) cudaEventDestroy(b.apply_done);
    if (b.select_done) cudaEventDestroy(b.select_done);
  }
  delete impl_;
}

int NativeEngine::add_bucket(const NativeBucketSpec& spec) {
  if (spec.handle == nullptr || spec.n_params <= 0) throw std::runtime_error("a bucket needs its handle and its parameters");
  if (spec.seg_off.size() != spec.seg_numel.size() || (int)spec.seg_off.size() != spec.n_params)
    throw std::runtime_error("one offset and one length per parameter");
  if (spec.steal && (spec.table_host == nullptr || spec.table_dev == nullptr || spec.table_ring < 2))
    throw std::runtime_error("a pointer-table bucket needs its pinned ring and its device table");
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)impl_->device);
  BucketRec b;
  b.spec = spec;
  if (spec.flat_grad != nullptr) b.flat_grad = tensor_of(spec.flat_grad, "flat_grad");
  b.spec.flat_grad = nullptr;
  b.full = b.pending = spec.n_params * impl_->ga;
  b.tab_events.resize(spec.steal ? spec.table_ring : 0);
  b.tab_event_set.assign(b.tab_events.size(), 0);
  for (auto& ev : b.tab_events)
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) throw std::runtime_error("cudaEventCreate failed");
  if (cudaEventCreateWithFlags(&b.grad_ready, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&b.apply_done, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&b.select_done, cudaEventDisableTiming) != cudaSuccess)
    throw std::runtime_error("cudaEventCreate failed");
  impl_->buckets.push_back(std::move(b));
  return (int)impl_->buckets.size() - 1;
}

void NativeEngine::add_param(int bucket, int seg, PyObject* parameter) {
  if (bucket < 0 || bucket >= (int)impl_->buckets.size()) throw std::runtime_error("no such bucket");
  BucketRec& b = impl_->buckets[bucket];
  if (seg < 0 || seg >= b.spec.n_params) throw std::runtime_error("no such tensor in the bucket");
  ParamRec pr;
  pr.tensor = tensor_of(parameter, "parameter");
  pr.bucket = bucket;
  pr.seg = seg;
  if (!pr.tensor.requires_grad() || !pr.tensor.is_leaf()) throw std::runtime_error("hooks go on leaf tensors that require gradients");
  const int pi = (int)impl_->params.size();
  impl_->params.push_back(pr);
  b.params.push_back(pi);
  auto hook = std::make_unique<GradHook>();
  hook->shared = impl_->shared;
  hook->param = pi;
  auto& slot = torch::autograd::impl::post_acc_grad_hooks(pr.tensor);
  hook->before = std::move(slot);
  torch::autograd::impl::set_post_acc_grad_hooks(pr.tensor, std::move(hook));
}

void NativeEngine::remove_hooks() {
  impl_->shared->alive.store(false, std::memory_order_release);
  std::lock_guard<std::mutex> lock(impl_->mu);
  for (auto& pr : impl_->params) {
    if (!pr.tensor.defined()) continue;
    auto& slot = torch::autograd::impl::post_acc_grad_hooks(pr.tensor);
    auto* mine = dynamic_cast<GradHook*>(slot.get());
    if (mine != nullptr && mine->shared == impl_->shared) {
      std::unique_ptr<torch::autograd::PostAccumulateGradHook> before = std::move(mine->before);
      torch::autograd::impl::set_post_acc_grad_hooks(pr.tensor, std::move(before));
    }
    pr.tensor = at::Tensor();
  }
}

void NativeEngine::set_shaper(void* shaper_state, uint64_t cap_ns) {
  std::lock_guard<std::mutex> lock(impl_->mu);
  impl_->shaper = shaper_state;
  impl_->shaper_cap_ns = cap_ns;
}

void NativeEngine::set_shaped_bytes(int bucket, uint64_t bytes) {
  std::lock_guard<std::mutex> lock(impl_->mu);
  impl_->buckets.at(bucket).spec.shaped_bytes = bytes;
}

void NativeEngine::wait_applies(uint64_t stream, int bucket) {
  std::lock_guard<std::mutex> lock(impl_->mu);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream));
  for (int i = 0; i < (int)impl_->buckets.size(); ++i) {
    if (bucket >= 0 && i != bucket) continue;
    BucketRec& b = impl_->buckets[i];
    if (b.apply_done_set) impl_->check(cudaStreamWaitEvent(s, b.apply_done, 0));
    // With a flat gradient buffer the coming backward pass accumulates into the memory that the latest select reads
    // and clears: the two must not overlap (with stolen gradients the select has its own tensors, see bucket_ready).
    if (!b.spec.steal && b.select_done_set) impl_->check(cudaStreamWaitEvent(s, b.select_done, 0));
  }
}

void NativeEngine::flush(uint64_t stream) {
  std::lock_guard<std::mutex> lock(impl_->mu);
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)impl_->device);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream));
  cudaEvent_t ev = nullptr;
  impl_->check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  if (ev == nullptr) return;
  impl_->check(cudaEventRecord(ev, s));
  impl_->check(cudaStreamWaitEvent(impl_->sparse, ev, 0));
  for (auto& b : impl_->buckets)
    if (b.has_pending_apply) impl_->apply(b);
  impl_->check(cudaEventRecord(ev, impl_->sparse));
  impl_->check(cudaStreamWaitEvent(s, ev, 0));
  cudaEventDestroy(ev);     // released once the waits that refer to it have been enqueued
}

void NativeEngine::begin_capture() {
  std::lock_guard<std::mutex> lock(impl_->mu);
  impl_->capturing = true;
  impl_->capture_keep.clear();
  impl_->capture_saved.clear();
  for (auto& b : impl_->buckets) {
    impl_->capture_saved.push_back({b.select_count, b.apply_count, b.has_pending_apply});
    b.capture_row = at::Tensor();
  }
  impl_->kernels_saved = impl_->kernels;
  impl_->shaped_saved = impl_->shaped;
}

PyObject* NativeEngine::end_capture() {
  std::lock_guard<std::mutex> lock(impl_->mu);
  impl_->capturing = false;
  for (size_t i = 0; i < impl_->buckets.size() && i < impl_->capture_saved.size(); ++i) {
    BucketRec& b = impl_->buckets[i];
    b.capture_row = at::Tensor();
    b.apply_done_set = false;      // events recorded under capture are not waitable outside
    b.select_done_set = false;     // and the selects of a replay are joined before the replay ends
  }
  PyObject* list = PyList_New((Py_ssize_t)impl_->capture_keep.size());
  for (size_t i = 0; i < impl_->capture_keep.size(); ++i)
    PyList_SET_ITEM(list, (Py_ssize_t)i, THPVariable_Wrap(impl_->capture_keep[i]));
  impl_->capture_keep.clear();
  return list;
}

int64_t NativeEngine::select_count(int bucket) const { return impl_->buckets.at(bucket).select_count; }
int64_t NativeEngine::apply_count(int bucket) const { return impl_->buckets.at(bucket).apply_count; }
bool NativeEngine::pending_apply(int bucket) const { return impl_->buckets.at(bucket).has_pending_apply; }
int NativeEngine::pending_hooks(int bucket) const { return impl_->buckets.at(bucket).pending; }
void NativeEngine::set_counts(int bucket, int64_t selects, int64_t applies, bool pending_apply) {
  std::lock_guard<std::mutex> lock(impl_->mu);
  BucketRec& b = impl_->buckets.at(bucket);
  b.select_count = selects;
  b.apply_count = applies;
  b.has_pending_apply = pending_apply;
  b.pending = b.full;
}
int64_t NativeEngine::kernels_launched() const { return impl_->kernels; }
uint64_t NativeEngine::shaped_bytes() const { return impl_->shaped; }
int NativeEngine::last_error() const { return impl_->error.load(); }

}  // namespace st
