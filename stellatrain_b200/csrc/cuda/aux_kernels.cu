// Kernels around the sparse path for grouped topologies and link measurement.
//
//   group reduce   dense sum of a bucket's gradients inside a group of GPUs, each rank reducing the
//                  tensors it owns by reading its group-mates' buffers over NVLink.  GPU form of the
//                  reference's slice-parallel CPU gather (backend/src/engine/modules/cpu_gather.cpp:58-82),
//                  partitioned by tensor instead of by slice so that per-tensor selection stays whole.
//   delay          holds a stream for a number of nanoseconds read from device memory: the serialisation
//                  time of a payload on an emulated slow link (token bucket on the host decides the value).
//   link probe     times a peer-to-peer copy with the device clock (the reference's bandwidth monitor
//                  counts bytes on a socket, backend/src/misc/bandwidth_monitor.h:8-84).
// Handshake of the group reduce, all flags are epochs in symmetric memory and every wait is bounded:
//   1. signal_ready : "my gradients of epoch e are complete"      -> every mate
//   2. reduce       : wait for the mates' ready flags, g_mine[owned] += sum g_mate[owned];
//                     the last CTA tells every mate "I have finished reading epoch e"
//   3. wait_done    : wait until every mate has finished reading, only then may later kernels
//                     overwrite (zero) this rank's gradients.
#include "device_utils.cuh"
#include "launchers.h"

namespace st {

namespace {
constexpr int kThreads = 256;
}

__global__ void k_group_signal_ready(GroupArgs A) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint32_t epoch = *A.epoch;
  __threadfence_system();
  for (int m = 0; m < A.n_mates; ++m) st_release_sys_u64(A.ready_peer[m], (uint64_t)epoch);
}

__global__ void __launch_bounds__(kThreads) k_group_reduce(GroupArgs A) {
  __shared__ int s_ok;
  const Chunk ch = A.chunks[blockIdx.x];
  const SegDesc sd = A.segs[ch.seg];
  const uint32_t epoch = *A.epoch;
  const bool owned = (sd.reserved & kSegSkip) == 0u;
  if (owned) {
    if (threadIdx.x == 0) {
      int ok = ld_volatile_u32(A.status) == kOk;
      for (int m = 0; ok && m < A.n_mates; ++m) {
        if (!wait_ge_bounded(A.ready_local + A.mate_slot[m], (uint64_t)epoch, A.timeout_ns)) {
          set_status(A.status, kTimeoutFlag);
          ok = 0;
        }
      }
      s_ok = ok;
    }
    __syncthreads();
    if (s_ok) {
      float* mine = A.grad_local + ch.start;
      for (uint32_t i = threadIdx.x * 4; i < ch.len; i += kThreads * 4) {
        float4 a = *reinterpret_cast<const float4*>(mine + i);
        for (int m = 0; m < A.n_mates; ++m) {
          // plain loads from the mate's memory; bypass L1, the data was just written remotely
          const float4 b = __ldcg(reinterpret_cast<const float4*>(A.grad_peer[m] + ch.start + i));
          a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        *reinterpret_cast<float4*>(mine + i) = a;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(A.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *A.done_ctr = 0;
      __threadfence_system();
      for (int m = 0; m < A.n_mates; ++m) st_release_sys_u64(A.done_peer[m], (uint64_t)epoch);
    }
  }
}

__global__ void k_group_wait_done(GroupArgs A) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint32_t epoch = *A.epoch;
  if (ld_volatile_u32(A.status) != kOk) return;
  for (int m = 0; m < A.n_mates; ++m) {
    if (!wait_ge_bounded(A.done_local + A.mate_slot[m], (uint64_t)epoch, A.timeout_ns)) {
      set_status(A.status, kTimeoutAck);
      return;
    }
  }
}

cudaError_t launch_group_reduce(const GroupArgs& A, cudaStream_t stream) {
  if (A.n_mates <= 0 || A.n_chunks == 0) return cudaSuccess;
  if (A.n_mates > kMaxWorld) return cudaErrorInvalidValue;
  k_group_signal_ready<<<1, 32, 0, stream>>>(A);
  k_group_reduce<<<A.n_chunks, kThreads, 0, stream>>>(A);
  k_group_wait_done<<<1, 32, 0, stream>>>(A);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
__global__ void k_delay(const uint64_t* ns_ptr, uint64_t cap_ns) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  uint64_t ns = *ns_ptr;
  if (ns > cap_ns) ns = cap_ns;       // never hold a stream longer than the stated bound
  const uint64_t t0 = global_timer_ns();
  while (global_timer_ns() - t0 < ns) __nanosleep(1000);
}

cudaError_t launch_delay(const uint64_t* ns_ptr, uint64_t cap_ns, cudaStream_t stream) {
  k_delay<<<1, 32, 0, stream>>>(ns_ptr, cap_ns);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// out[0] = nanoseconds (device clock) the grid spent copying n4 float4 from src to dst.
__global__ void __launch_bounds__(kThreads) k_link_probe(float4* dst, const float4* src, uint64_t n4, uint64_t* out,
                                                        uint32_t* ctr) {
  __shared__ uint64_t s_t0;
  if (threadIdx.x == 0) {
    s_t0 = global_timer_ns();
    atomicMin(reinterpret_cast<unsigned long long*>(out + 1), (unsigned long long)s_t0);
  }
  __syncthreads();
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += (uint64_t)gridDim.x * kThreads)
    dst[i] = __ldcg(src + i);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint64_t t1 = global_timer_ns();
    atomicMax(reinterpret_cast<unsigned long long*>(out + 2), (unsigned long long)t1);
    if (atomicAdd(ctr, 1u) == gridDim.x - 1) {
      *ctr = 0;
      out[0] = out[2] - out[1];
    }
  }
}

cudaError_t launch_link_probe(float* dst, const float* src, uint64_t n, uint64_t* out3, uint32_t* ctr, cudaStream_t stream) {
  if (n == 0 || (n & 3u)) return cudaErrorInvalidValue;
  const uint64_t n4 = n / 4;
  int grid = (int)((n4 + kThreads * 8 - 1) / (kThreads * 8));
  if (grid > 148 * 4) grid = 148 * 4;
  k_link_probe<<<grid, kThreads, 0, stream>>>(reinterpret_cast<float4*>(dst), reinterpret_cast<const float4*>(src), n4, out3, ctr);
  return cudaGetLastError();
}

}  // namespace st
