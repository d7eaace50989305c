// Host-side entry points of the sm_100a kernels (definitions in the .cu files of this folder).
#pragma once
#include <cuda_runtime.h>
#include "sparse_types.h"

namespace st {

// Error-feedback select + push of one bucket: four kernels on `stream` (two for random-k).
cudaError_t launch_select(const SelectArgs& args, uint32_t randomk_seed, cudaStream_t stream);

// Bounded wait + scatter-add + sparse optimiser of one bucket: two kernels on `stream`.
cudaError_t launch_apply(const ApplyArgs& args, int max_ctas_per_source, cudaStream_t stream);

// max |a - b| as float bits, atomically folded into *out_bits (caller zeroes it).
cudaError_t launch_max_abs_diff(const float* a, const float* b, uint64_t n, uint32_t* out_bits,
                                cudaStream_t stream);

// dst[0..n) = src[0..n); either side may be peer memory. n % 4 == 0, both 16-byte aligned.
cudaError_t launch_peer_copy(float* dst, const float* src, uint64_t n, cudaStream_t stream);

}  // namespace st
