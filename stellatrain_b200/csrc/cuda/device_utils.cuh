// Device-side primitives shared by the select and apply kernels: system-scope flag accesses,
// bounded waits, block scans and the stores that push stream entries into peer memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "sparse_types.h"

namespace st {

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Spin until *p >= want.  Gives up after timeout_ns or a fixed number of polls, whichever comes
// first, so that a missing peer can never hang the GPU; the caller records the failure.
__device__ __forceinline__ bool wait_ge_bounded(const uint64_t* p, uint64_t want, uint64_t timeout_ns) {
  if (ld_acquire_sys_u64(p) >= want) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    if (ld_acquire_sys_u64(p) >= want) return true;
    if ((it & 15u) == 15u) {
      if (global_timer_ns() - t0 > timeout_ns) return false;
      __nanosleep(256);
    }
  }
  return false;
}

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t code) {
  atomicCAS(status, (uint32_t)kOk, code);
}

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  return *reinterpret_cast<const volatile uint32_t*>(p);
}

// One 8-byte store that NVSwitch replicates into every GPU bound to the multicast object.
__device__ __forceinline__ void multimem_st_pair(uint2* mc_addr, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y))
               : "memory");
}

__device__ __forceinline__ void multimem_st_u32(uint32_t* mc_addr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}

// Narrow wire format -----------------------------------------------------------------------------
// First element of the tensor when its entries travel as 4-byte words, else kNotNarrow.
__device__ __forceinline__ uint32_t narrow_base_of(const SegDesc& sd) {
  return (sd.reserved & kSegNarrow) ? sd.off : kNotNarrow;
}

// The value as it will arrive: unchanged, or rounded to bf16 (nearest even).  The sender keeps
// x - wire_value(x) in its residual, so the rounding error is fed back like every unsent entry.
__device__ __forceinline__ float wire_value(uint32_t narrow_base, float x) {
  if (narrow_base == kNotNarrow) return x;
  const uint32_t b = __float_as_uint(x);
  return __uint_as_float((b + 0x7FFFu + ((b >> 16) & 1u)) & 0xFFFF0000u);
}

// Order-independent stream checksum: the sum over entries of this hash (debug checks).
__device__ __forceinline__ uint32_t entry_hash(uint32_t idx, uint32_t val_bits) {
  return idx * 0x9E3779B1u + (val_bits ^ (val_bits >> 15));
}

// Destination of a segment's entries: one rank when the optimiser state is partitioned, else all (-1).
__device__ __forceinline__ int dest_of(const SelectArgs& A, const SegDesc& sd) {
  return A.owner_mode ? (int)((sd.reserved >> kSegOwnerShift) & kSegOwnerMask) : -1;
}

// Store one stream entry into the receive area of every destination (dest < 0) or of one rank.
// slot_off: start of the tensor's region in the stream; pos: entry inside the region; val must already
// be wire_value(narrow_base, .).
__device__ __forceinline__ void emit_entry(const SelectArgs& A, int dest, uint32_t narrow_base, uint64_t slot_off,
                                           uint32_t pos, uint32_t idx, float val) {
  if (A.cksum_acc != nullptr && idx != kSentinelIdx) {
    // narrow entries arrive with the low 16 value bits cleared: hash what the receiver will decode
    const uint32_t vb = narrow_base != kNotNarrow ? (__float_as_uint(val) & 0xFFFF0000u) : __float_as_uint(val);
    atomicAdd(A.cksum_acc + (dest >= 0 ? dest : 0), entry_hash(idx, vb));
  }
  if (narrow_base != kNotNarrow) {
    const uint32_t w = idx == kSentinelIdx ? 0xFFFFFFFFu : ((idx - narrow_base) | (__float_as_uint(val) & 0xFFFF0000u));
    if (dest >= 0) {
      reinterpret_cast<uint32_t*>(A.out[dest] + slot_off)[pos] = w;
    } else if (A.out_mc != nullptr) {
      multimem_st_u32(reinterpret_cast<uint32_t*>(A.out_mc + slot_off) + pos, w);
    } else {
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p) {
        if (p < A.world) reinterpret_cast<uint32_t*>(A.out[p] + slot_off)[pos] = w;
      }
    }
    return;
  }
  const uint2 e = make_uint2(idx, __float_as_uint(val));
  if (dest >= 0) {
    A.out[dest][slot_off + pos] = e;
  } else if (A.out_mc != nullptr) {
    multimem_st_pair(A.out_mc + slot_off + pos, e);
  } else {
#pragma unroll
    for (int p = 0; p < kMaxWorld; ++p) {
      if (p < A.world) A.out[p][slot_off + pos] = e;
    }
  }
}

// Entry at position i of one source's stream (`in` points at position 0), decoded to (bucket index, value).
__device__ __forceinline__ uint2 load_entry(const ApplyArgs& A, const uint2* in, uint32_t i) {
  if (!A.narrow) return __ldcg(in + i);   // written by a peer: bypass L1
  // last tensor whose region starts at or before i
  uint32_t lo = 0, hi = A.n_segs;
  while (hi - lo > 1u) {
    const uint32_t mid = (lo + hi) >> 1;
    if (A.segs[mid].out_off <= i) lo = mid; else hi = mid;
  }
  const SegDesc sd = A.segs[lo];
  if (!(sd.reserved & kSegNarrow)) return __ldcg(in + i);
  const uint32_t w = __ldcg(reinterpret_cast<const uint32_t*>(in + sd.out_off) + (i - sd.out_off));
  if (w == 0xFFFFFFFFu) return make_uint2(kSentinelIdx, 0u);
  return make_uint2(sd.off + (w & 0xFFFFu), w & 0xFFFF0000u);
}

// ---- TMA bulk copies (cp.async.bulk) with mbarrier completion --------------------------------
// One thread asks the copy engine for a contiguous global->shared transfer and every thread of the
// CTA waits on the transaction barrier; loads of the next tile are in flight while the current one
// is processed, independent of occupancy.  Addresses and sizes must be multiples of 16 bytes.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// Bounded wait for the phase with the given parity; false when the copy did not land in time.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

__device__ __forceinline__ uint32_t warp_incl_scan(uint32_t v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint32_t o = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += o;
  }
  return v;
}

// Exclusive scan over the CTA in thread order.  `total` receives the CTA sum.  `s` must hold
// blockDim.x/32 + 1 words.  Contains two barriers; all threads of the CTA must call it.
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t* s, uint32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const uint32_t incl = warp_incl_scan(v);
  __syncthreads();  // protects s against a previous call
  if (lane == 31) s[warp] = incl;
  __syncthreads();
  uint32_t warp_off = 0, sum = 0;
  for (int w = 0; w < nwarp; ++w) {
    const uint32_t x = s[w];
    if (w < warp) warp_off += x;
    sum += x;
  }
  total = sum;
  return warp_off + incl - v;
}

__device__ __forceinline__ uint32_t block_max_u32(uint32_t v, uint32_t* s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, d));
  __syncthreads();
  if (lane == 0) s[warp] = v;
  __syncthreads();
  uint32_t r = 0;
  for (int w = 0; w < nwarp; ++w) r = max(r, s[w]);
  return r;
}

}  // namespace st
