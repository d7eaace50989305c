// Native step engine of the GPU-resident tier: what happens between "autograd produced a gradient" and "the
// bucket's kernels are in the stream", without the interpreter.
//
// Role of the reference's C++ scheduler for one iteration (backend/src/engine/core.cpp:775-797: the hook that the
// engine registers on every parameter; 1025-1095: post_backward_process, which turns a finished gradient into a
// task; backend/src/engine/core_module_api.cpp:7-109: scheduling of the stages).  Here the "stages" are the kernel
// chains of a bucket, ordered against autograd's stream by events: the hooks are C++ objects on the autograd
// graph's accumulation nodes, they run on autograd's own thread without the interpreter lock, note where the
// gradient lives, and the hook of a bucket's last parameter enqueues the bucket's select + push and the apply of
// the previous iteration (bounded staleness 1) on the sparse stream.
//
// The header names no torch type: parameters come in as the interpreter's tensor objects, so that the binding
// (bindings.cpp) needs no torch header.
#pragma once
#include <stdint.h>

#include <vector>

#include "bucket_handle.h"

typedef struct _object PyObject;

namespace st {

struct NativeBucketSpec {
  BucketHandle* handle = nullptr;          // launches apply (and select, unless select_handle is set)
  BucketHandle* select_handle = nullptr;
  int n_params = 0;
  bool steal = false;                      // kernels read autograd's own gradient tensors through a pointer table
  uint64_t* table_host = nullptr;          // pinned [ring][n_segs] rows of gradient addresses
  int table_ring = 0;
  uint64_t* table_dev = nullptr;           // device copy the kernels read
  PyObject* flat_grad = nullptr;           // the bucket's flat gradient buffer (a gradient that does not have its
                                           // parameter's layout is copied there)
  std::vector<uint32_t> seg_off, seg_numel;
  uint64_t shaped_bytes = 0;               // bytes a select of this bucket stores into other groups
};

class NativeEngine {
 public:
  NativeEngine(int device, uint64_t sparse_stream, int staleness, int grad_accumulation);
  ~NativeEngine();
  NativeEngine(const NativeEngine&) = delete;
  NativeEngine& operator=(const NativeEngine&) = delete;

  int add_bucket(const NativeBucketSpec& spec);
  // Registers the C++ post-accumulate hook on the parameter.  A parameter carries one such hook object: hooks that
  // Python code registered on it before are kept and run first; none can be added from Python afterwards.
  void add_param(int bucket, int seg, PyObject* parameter);
  void remove_hooks();

  void set_shaper(void* shaper_state, uint64_t cap_ns);     // device token bucket taken before every select, or null
  void set_shaped_bytes(int bucket, uint64_t bytes);        // after a change of the compression ratio
  // Forward gate (backend/src/engine/core.cpp:730-739 on a stream): `stream` waits for the updates the coming
  // forward must see; bucket < 0 = all of them.
  void wait_applies(uint64_t stream, int bucket);
  // Flush (backend/src/engine/core.cpp:1097-1140): pending applies are enqueued; `stream` waits for the sparse stream.
  void flush(uint64_t stream);

  // Stream capture of a whole iteration: gradients stay referenced instead of being handed to the allocator, the
  // gradient addresses go to rows of the capture's own.  end_capture returns what the capture must keep alive
  // (a list of tensors) and undoes the bookkeeping of the captured, not executed, iteration.
  void begin_capture();
  PyObject* end_capture();

  int64_t select_count(int bucket) const;
  int64_t apply_count(int bucket) const;
  void set_counts(int bucket, int64_t selects, int64_t applies, bool pending_apply);
  bool pending_apply(int bucket) const;
  int pending_hooks(int bucket) const;          // gradient hooks still to come before the bucket is ready
                                                // (parameters x accumulation steps between iterations)
  int64_t kernels_launched() const;
  uint64_t shaped_bytes() const;
  // First CUDA error a hook met (hooks cannot raise through autograd's thread), or 0.
  int last_error() const;

  struct Impl;     // defined in native_engine.cpp

 private:
  Impl* impl_;
};

}  // namespace st
