// Kernels around the sparse path for grouped topologies and link measurement.
//
//   group reduce   dense sum of a bucket's gradients inside a group of GPUs, each rank reducing the
//                  tensors it owns by reading its group-mates' buffers over NVLink.  GPU form of the
//                  reference's slice-parallel CPU gather (backend/src/engine/modules/cpu_gather.cpp:58-82),
//                  partitioned by tensor instead of by slice so that per-tensor selection stays whole.
//   delay          holds a stream for a number of nanoseconds read from device memory.
//   shape          token bucket of an emulated slow link, kept on the device: a payload that the bucket cannot
//                  cover holds the stream for its serialisation time at the scheduled rate.  Because the state
//                  and the clock are the GPU's own, the shaper also works inside a captured step.
//   stamp          writes the device clock into a slot (step timing that survives CUDA-graph replay).
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

// Token bucket whose fill rate follows a piecewise-constant schedule (ShaperState::rate, one level per period,
// origin at the first use).  Takes `nbytes`; when the bucket goes negative the stream is held for the time the
// debt needs at the current rate, at most cap_ns (a bound, so that a mis-set schedule cannot hold a GPU).
__global__ void k_shape(ShaperState* s, uint64_t nbytes, uint64_t cap_ns) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint64_t now = global_timer_ns();
  if (s->last_ns == 0) {
    s->t0_ns = now;
    s->last_ns = now;
    s->tokens = (double)s->burst_bytes;
  }
  const uint32_t levels = s->levels ? s->levels : 1u;
  const double period_ns = (double)s->period_s * 1e9;
  auto rate_at = [&](uint64_t t) -> double {
    const uint64_t lvl = period_ns > 0.0 ? (uint64_t)((double)(t - s->t0_ns) / period_ns) : 0ull;
    const double r = (double)s->rate[lvl % levels];
    return r > 1.0 ? r : 1.0;
  };
  const double dt = (double)(now - s->last_ns) * 1e-9;
  double tokens = s->tokens + dt * rate_at(s->last_ns);
  if (tokens > (double)s->burst_bytes) tokens = (double)s->burst_bytes;
  tokens -= (double)nbytes;
  s->tokens = tokens;
  s->last_ns = now;
  s->sent_bytes += nbytes;
  if (tokens >= 0.0) return;
  double wait = -tokens / rate_at(now) * 1e9;
  if (wait > (double)cap_ns) wait = (double)cap_ns;
  const uint64_t ns = (uint64_t)wait;
  s->waited_ns += ns;
  while (global_timer_ns() - now < ns) __nanosleep(1000);
}

cudaError_t launch_shape(ShaperState* state, uint64_t nbytes, uint64_t cap_ns, cudaStream_t stream) {
  if (state == nullptr) return cudaErrorInvalidValue;
  k_shape<<<1, 32, 0, stream>>>(state, nbytes, cap_ns);
  return cudaGetLastError();
}

__global__ void k_stamp(uint64_t* slot) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *slot = global_timer_ns();
}

cudaError_t launch_stamp(uint64_t* slot, cudaStream_t stream) {
  if (slot == nullptr) return cudaErrorInvalidValue;
  k_stamp<<<1, 32, 0, stream>>>(slot);
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
