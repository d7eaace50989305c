// Host-side entry points of the sm_100a kernels (definitions in the .cu files of this folder).
#pragma once
#include <cuda_runtime.h>
#include "sparse_types.h"

namespace st {

// Error-feedback select + push of one bucket: four kernels on `stream` (two for random-k).
cudaError_t launch_select(const SelectArgs& args, uint32_t randomk_seed, cudaStream_t stream);

// One-pass variant for threshold-v and threshold-v16 once every tensor has its threshold: two kernels.  Usable
// when fused_select_possible() says so (max_chunk_len: the longest chunk of the bucket's chunk table).
bool fused_select_possible(const SelectArgs& args, uint32_t max_chunk_len);
cudaError_t launch_select_fused(const SelectArgs& args, cudaStream_t stream);

// Bounded wait + scatter-add + sparse optimiser of one bucket: two kernels on `stream`, plus the copy of
// the owners' new parameter values when the optimiser state is partitioned.  phase 0 = all, 1 = scatter and
// apply only, 2 = parameter copy only.
cudaError_t launch_apply(const ApplyArgs& args, int max_ctas_per_source, int phase, cudaStream_t stream);

// max |a - b| as float bits, atomically folded into *out_bits (caller zeroes it).
cudaError_t launch_max_abs_diff(const float* a, const float* b, uint64_t n, uint32_t* out_bits,
                                cudaStream_t stream);

// dst[0..n) = src[0..n); either side may be peer memory. n % 4 == 0, both 16-byte aligned.
cudaError_t launch_peer_copy(float* dst, const float* src, uint64_t n, cudaStream_t stream);

// Grouped mode: signal, reduce the owned tensors over the group-mates' buffers, wait until the mates
// have finished reading this rank's gradients.  Three kernels on `stream`.
cudaError_t launch_group_reduce(const GroupArgs& args, cudaStream_t stream);

// Holds `stream` for *ns_ptr nanoseconds (at most cap_ns).
cudaError_t launch_delay(const uint64_t* ns_ptr, uint64_t cap_ns, cudaStream_t stream);

// Takes nbytes from the device-resident token bucket; holds `stream` while the bucket is in debt (at most cap_ns).
cudaError_t launch_shape(ShaperState* state, uint64_t nbytes, uint64_t cap_ns, cudaStream_t stream);

// *slot = device clock (ns) when `stream` reaches this point.
cudaError_t launch_stamp(uint64_t* slot, cudaStream_t stream);

// Device-clock time of a copy of n floats; out3 = {elapsed, min start, max end}; the caller sets
// out3[1] = UINT64_MAX, out3[2] = 0 and *ctr = 0 beforehand.
cudaError_t launch_link_probe(float* dst, const float* src, uint64_t n, uint64_t* out3, uint32_t* ctr, cudaStream_t stream);

}  // namespace st
