// Receive side of the sparse exchange fused with the merge and the lazy sparse optimisers.
//
// Replaces the reference's CPU stages
//   wait for W-1 ring messages      backend/src/engine/modules/grad_exchange.cpp:18-81
//   merge (sum over sources, / W, union of indices)
//                                   backend/src/engine/modules/cpu_optimize.cpp:40-72
//   sparse SGD / sparse Adam        backend/src/optim/sgd.cpp:221-262, backend/src/optim/adam.cpp:19-87
//   H2D copy of updated parameters  backend/src/engine/modules/h2d_copy.cpp:31-56  (no longer needed)
// by two kernels per bucket:
//   scatter  each CTA waits (bounded) for the arrival flag of the source it serves, then adds the
//            source's weighted values into a dense accumulator with red.global.add.f32
//   apply    walks the same streams again; the first thread to stamp an index with the current epoch
//            owns it, reads and clears the accumulator and applies the optimiser rule once, which
//            is the "apply once at the union of indices" contract without building the union; the
//            last CTA acknowledges the slot to every source and advances the counters.
#include "device_utils.cuh"

namespace st {

namespace {
constexpr int kThreads = 256;
}

__global__ void __launch_bounds__(kThreads) k_scatter(ApplyArgs A) {
  __shared__ int s_ok;
  const int src = blockIdx.y;
  const uint32_t epoch = *A.epoch;
  const uint32_t slot = epoch & 1u;
  // Nothing was selected for this epoch yet (e.g. a captured step replayed right after a flush):
  // the pair of kernels is a no-op and leaves every counter untouched.
  if (epoch >= ld_volatile_u32(A.sel_epoch)) return;
  if (threadIdx.x == 0) {
    int ok = ld_volatile_u32(A.status) == kOk;
    if (ok && A.use_flags) {
      ok = wait_ge_bounded(A.flag_local + (size_t)slot * A.world + src, (uint64_t)epoch, A.timeout_ns);
      if (!ok) set_status(A.status, kTimeoutFlag);
    }
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const uint2* in = A.recv + (size_t)slot * A.slot_stride + (size_t)src * A.cap;
  const float w = A.weight[src];
  for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < A.cap; i += gridDim.x * kThreads) {
    const uint2 e = __ldcg(in + i);   // written by a peer: bypass L1
    if (e.x == kSentinelIdx) continue;
    if (e.x >= A.n_total) { set_status(A.status, kBadIndex); continue; }
    atomicAdd(A.acc + e.x, __uint_as_float(e.y) * w);
  }
}

__global__ void __launch_bounds__(kThreads) k_apply(ApplyArgs A) {
  __shared__ float s_bc[2];
  const int src = blockIdx.y;
  const uint32_t epoch = *A.epoch;
  const uint32_t slot = epoch & 1u;
  if (epoch >= ld_volatile_u32(A.sel_epoch)) return;
  const bool ok = ld_volatile_u32(A.status) == kOk;
  const OptState o = *A.opt;

  if (ok) {
    if (threadIdx.x == 0) {
      // bias corrections in double, as the reference computes them (adam.cpp:41-42)
      s_bc[0] = (float)(1.0 - pow((double)o.beta1, (double)o.tick));
      s_bc[1] = (float)(1.0 - pow((double)o.beta2, (double)o.tick));
    }
    __syncthreads();
    const float bc1 = s_bc[0], bc2 = s_bc[1];
    const uint32_t m_iter = o.tick - 1u;
    const float lr = (o.kind == 0 && o.maximize) ? -o.lr : o.lr;
    const uint2* in = A.recv + (size_t)slot * A.slot_stride + (size_t)src * A.cap;
    for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < A.cap; i += gridDim.x * kThreads) {
      const uint2 e = __ldcg(in + i);
      const uint32_t idx = e.x;
      if (idx >= A.n_total) continue;               // sentinel or invalid (already reported)
      if (atomicExch(A.stamp + idx, epoch) == epoch) continue;   // another entry owns this index
      float g = A.acc[idx];
      A.acc[idx] = 0.f;
      const float x = A.param[idx];
      if (o.kind == 0) {
        float mu = o.momentum;
        if (o.smart_momentum && A.last != nullptr && m_iter != 0u)
          mu = powf(o.momentum, (float)(m_iter - A.last[idx]));
        if (o.weight_decay != 0.f) g += o.weight_decay * x;
        if (o.momentum != 0.f) {
          const float b = o.first ? g : A.m[idx] * mu + (1.f - o.dampening) * g;
          g = o.nesterov ? g + mu * b : b;
          A.m[idx] = b;
        }
        A.param[idx] = x - lr * g;
        if (o.smart_momentum && A.last != nullptr) A.last[idx] = m_iter;
      } else {
        if (o.maximize) g = -g;
        if (o.weight_decay != 0.f) g += o.weight_decay * x;
        const float mt = o.beta1 * A.m[idx] + (1.f - o.beta1) * g;
        const float vt = o.beta2 * A.v[idx] + (1.f - o.beta2) * g * g;
        const float mh = mt / bc1;
        float vh = vt / bc2;
        if (o.amsgrad && A.vmax != nullptr) {
          vh = fmaxf(A.vmax[idx], vh);
          A.vmax[idx] = vh;
        }
        A.param[idx] = x - o.lr * mh / (sqrtf(vh) + o.eps);
        A.m[idx] = mt;
        A.v[idx] = vt;
      }
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(A.done_ctr, 1u);
    if (prev == gridDim.x * gridDim.y - 1) {
      *A.done_ctr = 0;
      if (A.use_acks && ld_volatile_u32(A.status) == kOk) {
        __threadfence_system();
        for (int p = 0; p < A.world; ++p)
          st_release_sys_u64(A.ack[p] + (size_t)slot * A.ack_slot_stride, (uint64_t)epoch);
      }
      A.opt->tick = o.tick + 1u;
      A.opt->first = 0u;
      *A.epoch = epoch + 1u;
    }
  }
}

cudaError_t launch_apply(const ApplyArgs& A, int max_ctas_per_source, cudaStream_t stream) {
  if (A.cap == 0 || A.world <= 0) return cudaSuccess;
  if (A.world > kMaxWorld) return cudaErrorInvalidValue;
  // one entry per thread: the update of an entry is a chain of dependent random accesses, so the
  // only way to hide its latency is to have every entry in flight at once
  int parts = (int)((A.cap + kThreads - 1) / kThreads);
  if (parts < 1) parts = 1;
  if (parts > max_ctas_per_source) parts = max_ctas_per_source;
  dim3 grid(parts, A.world);
  k_scatter<<<grid, kThreads, 0, stream>>>(A);
  k_apply<<<grid, kThreads, 0, stream>>>(A);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Replica parity: max |mine - peer| over a flat range, read through a peer pointer.  The
// reference checks cross-node divergence by shipping whole tensors to the broker
// (backend/src/engine/core.cpp:843-847, 874-878); here one kernel reads the peer over NVLink.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) k_max_abs_diff(const float* a, const float* b, uint64_t n,
                                                          uint32_t* out_bits) {
  __shared__ uint32_t s_tmp[kThreads / 32 + 1];
  float mx = 0.f;
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (uint64_t)gridDim.x * kThreads) {
    const float d = fabsf(a[i] - b[i]);
    mx = (d == d) ? fmaxf(mx, d) : __uint_as_float(0x7f800000u);   // NaN counts as infinite drift
  }
  const uint32_t r = block_max_u32(__float_as_uint(mx), s_tmp);
  if (threadIdx.x == 0 && r) atomicMax(out_bits, r);
}

cudaError_t launch_max_abs_diff(const float* a, const float* b, uint64_t n, uint32_t* out_bits,
                                cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  int grid = (int)((n + kThreads * 8 - 1) / (kThreads * 8));
  if (grid > 148 * 8) grid = 148 * 8;
  k_max_abs_diff<<<grid, kThreads, 0, stream>>>(a, b, n, out_bits);
  return cudaGetLastError();
}

// Copy a flat range from a peer (initial parameter broadcast from rank 0; the reference relays
// every tensor through its broker: backend/src/engine/comm_manager.cpp:1022-1077).
__global__ void __launch_bounds__(kThreads) k_copy_f4(float4* dst, const float4* src, uint64_t n4) {
  for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += (uint64_t)gridDim.x * kThreads)
    dst[i] = src[i];
}

cudaError_t launch_peer_copy(float* dst, const float* src, uint64_t n, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  if ((n & 3u) || ((uintptr_t)dst & 15u) || ((uintptr_t)src & 15u)) return cudaErrorInvalidValue;
  const uint64_t n4 = n / 4;
  int grid = (int)((n4 + kThreads * 4 - 1) / (kThreads * 4));
  if (grid > 148 * 8) grid = 148 * 8;
  k_copy_f4<<<grid, kThreads, 0, stream>>>(reinterpret_cast<float4*>(dst), reinterpret_cast<const float4*>(src), n4);
  return cudaGetLastError();
}

}  // namespace st
