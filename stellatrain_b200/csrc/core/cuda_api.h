// The handful of CUDA runtime calls the CPU tier needs for its device copies, behind a table of function
// pointers.
//
// The reference's copy stages call the runtime directly (backend/src/engine/modules/d2h_copy.cpp:44-60:
// event, stream wait, asynchronous copy, cudaLaunchHostFunc; h2d_copy.cpp:45-53).  This tier is also built
// and tested on machines without a GPU, so the runtime is looked up with dlopen when it is first needed, and a
// test can install a table of its own whose "streams" are ordinary worker threads and whose "device memory"
// is host memory.
#pragma once
#include <cstddef>

namespace stc {

struct CudaApi {
  // all return 0 on success, like the runtime
  int (*stream_create)(void** stream);                                  // non-blocking stream
  int (*stream_destroy)(void* stream);
  int (*stream_synchronize)(void* stream);
  int (*event_create)(void** event);                                    // timing disabled
  int (*event_destroy)(void* event);
  int (*event_record)(void* event, void* stream);
  int (*stream_wait_event)(void* stream, void* event);
  int (*memcpy_d2h_async)(void* dst, const void* src, size_t bytes, void* stream);
  int (*memcpy_h2d_async)(void* dst, const void* src, size_t bytes, void* stream);
  int (*launch_host_func)(void* stream, void (*fn)(void*), void* user);
  int (*get_device)(int* device);                                       // device of the calling thread
  int (*set_device)(int device);
};

// The table in use: an installed one, else the dlopen'ed runtime, else nullptr (no CUDA runtime in this process).
const CudaApi* cuda_api();
// Installs (or, with nullptr, removes) a replacement table.  For tests on machines without a GPU.
void set_cuda_api(const CudaApi* api);

// The replacement table of fake_cuda.cpp: streams are worker threads, device memory is host memory, every copy
// takes `delay_ms` longer.  Counters: copies in each direction and host callbacks run since it was installed.
void install_fake_cuda(int delay_ms);
void remove_fake_cuda();
void fake_cuda_counters(long* d2h, long* h2d, long* host_funcs);

}  // namespace stc
