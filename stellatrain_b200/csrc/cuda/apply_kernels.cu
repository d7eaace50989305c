// Receive side of the sparse exchange fused with the merge and the lazy sparse optimisers.
//
// Replaces the reference's CPU stages
//   wait for W-1 ring messages      backend/src/engine/modules/grad_exchange.cpp:18-81
//   merge (sum over sources, / W, union of indices)
//                                   backend/src/engine/modules/cpu_optimize.cpp:40-72
//   sparse SGD / sparse Adam        backend/src/optim/sgd.cpp:221-262, backend/src/optim/adam.cpp:19-87
//   H2D copy of updated parameters  backend/src/engine/modules/h2d_copy.cpp:31-56  (no longer needed)
// by two kernels per bucket (three when the optimiser state is partitioned over the ranks):
//   wait     one warp waits (bounded) for the arrival flags of all sources (only when flags are in use)
//   scatter  adds every source's weighted values into a dense accumulator with red.global.add.f32
//   apply    walks the same streams again; the first thread to stamp an index with the current epoch
//            owns it, reads and clears the accumulator and applies the optimiser rule once, which
//            is the "apply once at the union of indices" contract without building the union; the
//            last CTA acknowledges the slot to every source and advances the counters.
//   param    partitioned state only.  A tensor's entries go to one rank, its owner, which keeps the
//   scatter  accumulator and the optimiser state for it (1/W of the memory), applies the update and
//            stores the new values into every rank's write-back area; this kernel waits (bounded) for
//            the owners' flags and copies the values into the local replica, so replicas agree bit for
//            bit.  The reference keeps full optimiser state in every process.
#include "device_utils.cuh"

namespace st {

namespace {
constexpr int kThreads = 256;
}

// One warp waits (bounded) for the arrival flags of all sources, one lane per source, and leaves the outcome
// in the status word.  The wide scatter grid that follows in the stream therefore never sits on the SMs
// spinning while a peer is late, which would keep the backward pass of the lower-priority compute stream out.
__global__ void k_wait_streams(ApplyArgs A) {
  const uint32_t epoch = *A.epoch;
  const uint32_t slot = epoch & 1u;
  // Nothing was selected for this epoch yet (e.g. a captured step replayed right after a flush):
  // the chain of kernels is a no-op and leaves every counter untouched.
  if (epoch >= ld_volatile_u32(A.sel_epoch)) return;
  if (ld_volatile_u32(A.status) == kOk) {
    for (int src = threadIdx.x; src < A.world; src += 32) {
      if (!wait_ge_bounded(A.flag_local + (size_t)slot * A.world + src, (uint64_t)epoch, A.timeout_ns))
        set_status(A.status, kTimeoutFlag);
    }
  }
  __syncwarp();
  if (threadIdx.x == 0 && A.stamps != nullptr) A.stamps[2] = global_timer_ns();
}

__global__ void __launch_bounds__(kThreads) k_scatter(ApplyArgs A) {
  const int src = blockIdx.y + A.src_first;
  const uint32_t epoch = *A.epoch;
  const uint32_t slot = epoch & 1u;
  if (epoch >= ld_volatile_u32(A.sel_epoch)) return;
  if (ld_volatile_u32(A.status) != kOk) return;   // includes "a stream did not arrive in time"
  if (!A.use_flags && A.stamps != nullptr && blockIdx.x == 0 && src == 0 && threadIdx.x == 0) A.stamps[2] = global_timer_ns();
  const uint2* in = A.recv + (size_t)slot * A.slot_stride + (size_t)src * A.cap;
  const float w = A.weight[(size_t)slot * A.world + src];
  uint32_t sum = 0;
  for (uint32_t i = A.ent_lo + blockIdx.x * kThreads + threadIdx.x; i < A.ent_hi; i += gridDim.x * kThreads) {
    const uint2 e = load_entry(A, in, i);
    if (e.x == kSentinelIdx) continue;
    sum += entry_hash(e.x, e.y);
    const uint32_t s = e.x - A.state_base;   // wraps to a large value below the base
    if (s >= A.state_len) { set_status(A.status, kBadIndex); continue; }
    atomicAdd(&A.rec[s].x, __uint_as_float(e.y) * w);
  }
  if (A.cksum_local != nullptr && sum != 0u) atomicAdd(A.rsum + src, sum);
}

// Store one write-back entry into the same stream position of every rank's write-back area.
__device__ __forceinline__ void emit_writeback(const ApplyArgs& A, uint64_t pos, uint32_t idx, float val) {
  const uint2 e = make_uint2(idx, __float_as_uint(val));
  if (A.wb_mc != nullptr) {
    multimem_st_pair(A.wb_mc + pos, e);
  } else {
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p) {
      if (p < A.world) A.wb[p][pos] = e;
    }
  }
}

// Last step of a chain: acknowledge the consumed receive slot to every source, advance the counters.
__device__ __forceinline__ void finish_apply(const ApplyArgs& A, uint32_t epoch, uint32_t tick) {
  const uint32_t slot = epoch & 1u;
  if (A.use_acks && ld_volatile_u32(A.status) == kOk) {
    __threadfence_system();
    for (int p = 0; p < A.world; ++p)
      st_release_sys_u64(A.ack[p] + (size_t)slot * A.ack_slot_stride, (uint64_t)epoch);
  }
  A.opt->tick = tick + 1u;
  A.opt->first = 0u;
  *A.epoch = epoch + 1u;
  if (A.stamps != nullptr) {
    A.stamps[3] = global_timer_ns();
    A.stamps[5] = epoch;
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
    const uint64_t src_off = (size_t)slot * A.slot_stride + (size_t)src * A.cap;
    uint2* in = A.recv + src_off;
    if (A.cksum_local != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
      // the scatter kernel has read the whole stream of this source: does it add up to what was sent?
      const uint32_t got = atomicExch(A.rsum + src, 0u);
      const uint32_t want = __ldcg(A.cksum_local + (size_t)slot * A.world + src);
      if (got != want) set_status(A.status, kBadChecksum);
    }
    for (uint32_t i = A.ent_lo + blockIdx.x * kThreads + threadIdx.x; i < A.ent_hi; i += gridDim.x * kThreads) {
      const uint2 e = load_entry(A, in, i);
      const uint32_t idx = e.x;
      const uint32_t s = idx - A.state_base;        // sentinel or invalid indices (already reported) fall outside
      // the first thread to stamp an index with this epoch owns it
      const bool won = s < A.state_len &&
                       atomicExch(reinterpret_cast<uint32_t*>(&A.rec[s].y), epoch) != epoch;
      float xn = 0.f;
      if (won) {
        const float4 rc = __ldcg(A.rec + s);     // accumulator, stamp, m, v in one 16-byte load
        float g = rc.x;
        float m_new = rc.z, v_new = rc.w;
        const float x = A.param[idx];
        if (o.kind == 0) {
          float mu = o.momentum;
          if (o.smart_momentum && A.last != nullptr && m_iter != 0u)
            mu = powf(o.momentum, (float)(m_iter - A.last[s]));
          if (o.weight_decay != 0.f) g += o.weight_decay * x;
          if (o.momentum != 0.f) {
            const float b = o.first ? g : rc.z * mu + (1.f - o.dampening) * g;
            g = o.nesterov ? g + mu * b : b;
            m_new = b;
          }
          xn = x - lr * g;
          if (o.smart_momentum && A.last != nullptr) A.last[s] = m_iter;
        } else {
          if (o.maximize) g = -g;
          if (o.weight_decay != 0.f) g += o.weight_decay * x;
          const float mt = o.beta1 * rc.z + (1.f - o.beta1) * g;
          const float vt = o.beta2 * rc.w + (1.f - o.beta2) * g * g;
          const float mh = mt / bc1;
          float vh = vt / bc2;
          if (o.amsgrad && A.vmax != nullptr) {
            vh = fmaxf(A.vmax[s], vh);
            A.vmax[s] = vh;
          }
          xn = x - o.lr * mh / (sqrtf(vh) + o.eps);
          m_new = mt;
          v_new = vt;
        }
        // accumulator cleared, stamp kept (a late loser's exchange writes the same epoch again)
        A.rec[s] = make_float4(0.f, __uint_as_float(epoch), m_new, v_new);
        A.param[idx] = xn;
      }
      // every consumed position is rewritten each epoch, so a stale value can never be read back
      if (A.owner_mode) emit_writeback(A, src_off + i, won ? idx : kSentinelIdx, xn);
      if (A.poison && !A.narrow) in[i] = make_uint2(kSentinelIdx, 0u);
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) {
    if (A.owner_mode) __threadfence_system();   // this CTA's stores into the peers before the count below
    else __threadfence();
    const uint32_t prev = atomicAdd(A.done_ctr, 1u);
    if (prev == gridDim.x * gridDim.y - 1) {
      *A.done_ctr = 0;
      if (!A.owner_mode) {
        finish_apply(A, epoch, o.tick);
      } else if (ld_volatile_u32(A.status) == kOk) {
        // the new values are on their way to every replica: tell them; the copy kernel finishes the chain
        __threadfence_system();
        for (int p = 0; p < A.world; ++p)
          st_release_sys_u64(A.pflag[p] + (size_t)slot * A.pflag_slot_stride, (uint64_t)epoch);
      }
    }
  }
}

// Partitioned state, every rank: wait (bounded) for each owner's values, copy them into the replica.
// CTAs with blockIdx.y == o serve the positions owner o consumed.
__global__ void __launch_bounds__(kThreads) k_param_scatter(ApplyArgs A) {
  __shared__ int s_ok;
  const int owner = blockIdx.y;
  const uint32_t epoch = *A.epoch;
  const uint32_t slot = epoch & 1u;
  if (epoch >= ld_volatile_u32(A.sel_epoch)) return;
  if (threadIdx.x == 0) {
    int ok = ld_volatile_u32(A.status) == kOk;
    if (ok) {
      ok = wait_ge_bounded(A.pflag_local + (size_t)slot * A.world + owner, (uint64_t)epoch, A.timeout_ns);
      if (!ok) set_status(A.status, kTimeoutFlag);
    }
    s_ok = ok;
  }
  __syncthreads();
  const uint32_t lo = A.own_lo[owner], len = A.own_lo[owner + 1] - lo;
  if (s_ok && owner != A.rank && len != 0u) {   // the owner has already written its own replica
    const uint64_t total = (uint64_t)len * (uint64_t)A.world;
    const uint2* in = A.wb_local + (size_t)slot * A.slot_stride;
    for (uint64_t t = (uint64_t)blockIdx.x * kThreads + threadIdx.x; t < total; t += (uint64_t)gridDim.x * kThreads) {
      const uint32_t src = (uint32_t)(t / len), i = lo + (uint32_t)(t % len);
      const uint2 e = __ldcg(in + (size_t)src * A.cap + i);
      if (e.x < A.n_total) A.param[e.x] = __uint_as_float(e.y);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(A.done_ctr, 1u);
    if (prev == gridDim.x * gridDim.y - 1) {
      *A.done_ctr = 0;
      finish_apply(A, epoch, A.opt->tick);
    }
  }
}

// phase 0: the whole chain; 1: scatter + apply only; 2: the parameter copy of partitioned state only
// (split launches let a test run several emulated ranks on one GPU without a kernel waiting for a later one).
cudaError_t launch_apply(const ApplyArgs& A, int max_ctas_per_source, int phase, cudaStream_t stream) {
  if (A.cap == 0 || A.world <= 0) return cudaSuccess;
  if (A.world > kMaxWorld) return cudaErrorInvalidValue;
  if (A.ent_hi < A.ent_lo || A.ent_hi > A.cap) return cudaErrorInvalidValue;
  // one entry per thread: the update of an entry is a chain of dependent random accesses, so the
  // only way to hide its latency is to have every entry in flight at once
  if (phase == 0 || phase == 1) {
    int parts = (int)((A.ent_hi - A.ent_lo + kThreads - 1) / kThreads);
    if (parts < 1) parts = 1;
    if (parts > max_ctas_per_source) parts = max_ctas_per_source;
    dim3 grid(parts, A.world);
    if (A.use_flags) k_wait_streams<<<1, 32, 0, stream>>>(A);
    if (A.deterministic) {
      ApplyArgs one = A;
      for (int src = 0; src < A.world; ++src) {   // one launch per source: a fixed order of additions
        one.src_first = (uint32_t)src;
        k_scatter<<<dim3(parts, 1), kThreads, 0, stream>>>(one);
      }
    } else {
      k_scatter<<<grid, kThreads, 0, stream>>>(A);
    }
    k_apply<<<grid, kThreads, 0, stream>>>(A);
  }
  if (A.owner_mode && (phase == 0 || phase == 2)) {
    uint32_t longest = 0;
    for (int o = 0; o < A.world; ++o) {
      if (A.own_lo[o + 1] < A.own_lo[o] || A.own_lo[o + 1] > A.cap) return cudaErrorInvalidValue;
      longest = A.own_lo[o + 1] - A.own_lo[o] > longest ? A.own_lo[o + 1] - A.own_lo[o] : longest;
    }
    uint64_t parts = ((uint64_t)longest * (uint64_t)A.world + kThreads - 1) / kThreads;
    if (parts < 1) parts = 1;
    if (parts > (uint64_t)max_ctas_per_source) parts = (uint64_t)max_ctas_per_source;
    dim3 grid((unsigned)parts, A.world);
    k_param_scatter<<<grid, kThreads, 0, stream>>>(A);
  }
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
