// One bucket's pre-filled kernel arguments and the launches that use them.  Filled once at set-up by the Python
// side (bindings.cpp); `select` and `apply` are then a handful of kernel launches without any per-call
// marshalling, from Python or from the native step engine (native_engine.cpp).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "launchers.h"

namespace st {

struct BucketHandle {
  SelectArgs sel;
  ApplyArgs app;
  GroupArgs grp;
  bool has_group = false;
  uint32_t randomk_seed = 0x5DEECE66u;
  int max_ctas_per_source = 148 * 16;
  uint32_t max_chunk_len = 0;      // longest chunk of the chunk table (decides whether the one-pass select may run)
  // One-pass select of the threshold compressors: allowed by configuration, and possible once every tensor of
  // the bucket has its threshold (one select through the four-kernel chain, or a restored checkpoint).
  bool fused_enabled = true;
  bool thresholds_ready = false;
  bool last_select_fused = false;

  bool can_fuse() const { return fused_select_possible(sel, max_chunk_len); }

  cudaError_t select(cudaStream_t stream) {
    const bool fused = fused_enabled && thresholds_ready && can_fuse();
    const cudaError_t e = fused ? launch_select_fused(sel, stream) : launch_select(sel, randomk_seed, stream);
    thresholds_ready = true;       // the four-kernel chain leaves every tensor with a threshold
    last_select_fused = fused;
    return e;
  }

  // kernels of the last select (telemetry's launch count)
  int select_kernels() const { return (sel.compressor == kRandomk || last_select_fused) ? 2 : 4; }

  cudaError_t apply(cudaStream_t stream, int phase) { return launch_apply(app, max_ctas_per_source, phase, stream); }

  int apply_kernels() const {
    return (app.owner_mode ? 3 : 2) + (app.deterministic ? app.world - 1 : 0) + (app.use_flags ? 1 : 0);
  }

  cudaError_t group_reduce(cudaStream_t stream) {
    if (!has_group) return cudaSuccess;
    grp.segs = sel.segs;
    grp.chunks = sel.chunks;
    grp.n_chunks = sel.n_chunks;
    grp.epoch = sel.epoch;
    grp.status = sel.status;
    grp.timeout_ns = sel.timeout_ns;
    return launch_group_reduce(grp, stream);
  }
};

}  // namespace st
