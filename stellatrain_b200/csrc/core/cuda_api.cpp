#include "cuda_api.h"

#include <dlfcn.h>

#include <atomic>
#include <mutex>

namespace stc {

namespace {

// entry points of libcudart with their real signatures
using StreamCreateFn = int (*)(void**, unsigned);
using StreamFn = int (*)(void*);
using EventCreateFn = int (*)(void**, unsigned);
using EventRecordFn = int (*)(void*, void*);
using StreamWaitFn = int (*)(void*, void*, unsigned);
using MemcpyAsyncFn = int (*)(void*, const void*, size_t, int, void*);
using HostFuncFn = int (*)(void*, void (*)(void*), void*);
using GetDeviceFn = int (*)(int*);
using SetDeviceFn = int (*)(int);

struct Runtime {
  StreamCreateFn stream_create = nullptr;
  StreamFn stream_destroy = nullptr, stream_sync = nullptr, event_destroy = nullptr;
  EventCreateFn event_create = nullptr;
  EventRecordFn event_record = nullptr;
  StreamWaitFn stream_wait = nullptr;
  MemcpyAsyncFn memcpy_async = nullptr;
  HostFuncFn host_func = nullptr;
  GetDeviceFn get_device = nullptr;
  SetDeviceFn set_device = nullptr;
} rt;

int w_stream_create(void** s) { return rt.stream_create(s, 0x01 /* cudaStreamNonBlocking */); }
int w_stream_destroy(void* s) { return rt.stream_destroy(s); }
int w_stream_sync(void* s) { return rt.stream_sync(s); }
int w_event_create(void** e) { return rt.event_create(e, 0x02 /* cudaEventDisableTiming */); }
int w_event_destroy(void* e) { return rt.event_destroy(e); }
int w_event_record(void* e, void* s) { return rt.event_record(e, s); }
int w_stream_wait(void* s, void* e) { return rt.stream_wait(s, e, 0); }
int w_d2h(void* d, const void* s, size_t n, void* st) { return rt.memcpy_async(d, s, n, 2 /* cudaMemcpyDeviceToHost */, st); }
int w_h2d(void* d, const void* s, size_t n, void* st) { return rt.memcpy_async(d, s, n, 1 /* cudaMemcpyHostToDevice */, st); }
int w_host_func(void* s, void (*fn)(void*), void* u) { return rt.host_func(s, fn, u); }
int w_get_device(int* d) { return rt.get_device(d); }
int w_set_device(int d) { return rt.set_device(d); }

const CudaApi kRuntimeTable = {w_stream_create, w_stream_destroy, w_stream_sync, w_event_create, w_event_destroy,
                               w_event_record,  w_stream_wait,    w_d2h,         w_h2d,          w_host_func,
                               w_get_device,    w_set_device};

std::atomic<const CudaApi*> installed{nullptr};
std::once_flag load_once;
bool runtime_ok = false;

void load_runtime() {
  // The framework that owns the GPU has loaded a runtime already: use that copy (streams and events are shared with
  // it), and only load one when there is none.
  void* lib = dlopen("libcudart.so.12", RTLD_NOW | RTLD_NOLOAD);
  if (!lib) lib = dlopen("libcudart.so.12", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libcudart.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return;
  auto sym = [lib](const char* name) { return dlsym(lib, name); };
  rt.stream_create = reinterpret_cast<StreamCreateFn>(sym("cudaStreamCreateWithFlags"));
  rt.stream_destroy = reinterpret_cast<StreamFn>(sym("cudaStreamDestroy"));
  rt.stream_sync = reinterpret_cast<StreamFn>(sym("cudaStreamSynchronize"));
  rt.event_create = reinterpret_cast<EventCreateFn>(sym("cudaEventCreateWithFlags"));
  rt.event_destroy = reinterpret_cast<StreamFn>(sym("cudaEventDestroy"));
  rt.event_record = reinterpret_cast<EventRecordFn>(sym("cudaEventRecord"));
  rt.stream_wait = reinterpret_cast<StreamWaitFn>(sym("cudaStreamWaitEvent"));
  rt.memcpy_async = reinterpret_cast<MemcpyAsyncFn>(sym("cudaMemcpyAsync"));
  rt.host_func = reinterpret_cast<HostFuncFn>(sym("cudaLaunchHostFunc"));
  rt.get_device = reinterpret_cast<GetDeviceFn>(sym("cudaGetDevice"));
  rt.set_device = reinterpret_cast<SetDeviceFn>(sym("cudaSetDevice"));
  runtime_ok = rt.stream_create && rt.stream_destroy && rt.stream_sync && rt.event_create && rt.event_destroy &&
               rt.event_record && rt.stream_wait && rt.memcpy_async && rt.host_func && rt.get_device && rt.set_device;
}

}  // namespace

const CudaApi* cuda_api() {
  if (const CudaApi* a = installed.load(std::memory_order_acquire)) return a;
  std::call_once(load_once, load_runtime);
  return runtime_ok ? &kRuntimeTable : nullptr;
}

void set_cuda_api(const CudaApi* api) { installed.store(api, std::memory_order_release); }

}  // namespace stc
