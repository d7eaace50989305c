// Error-feedback sparsification fused with the push of the (idx,val) stream into peer GPUs.
//
// Replaces, for one bucket of parameter tensors, the reference's CPU stages
//   gather + residual add      backend/src/engine/modules/cpu_gather.cpp:63-82
//   top-k / threshold-v / threshold-v16 selection
//                              backend/src/compress/topk.cpp:28-46 (intent; the shipped code is defective),
//                              backend/src/compress/thresholdv.cpp:40-83,
//                              backend/src/compress/thresholdv16.cpp:78-295
//   residual save              backend/src/engine/modules/compress.cpp:172-188
//   ring all-gather            backend/src/engine/modules/grad_exchange.cpp:45-62
// by a chain of four kernels per bucket on one stream:
//   pass1  a = g + r, r <- a, g <- 0; per-segment histogram of the top 11 key bits and/or per-chunk
//          count of items over the persistent threshold
//   plan   per segment: pick the histogram bin that holds the k-th largest key, or prefix-sum the
//          chunk counts; adapt the threshold (AIMD); wait (bounded) for the destinations'
//          acknowledgement of the receive slot about to be overwritten
//   pass2  re-read r (L2-resident for buckets below the L2 size), store every selected entry
//          straight into all destinations' receive areas (peer stores or one multimem store), zero it
//          in r, and append the undecided items of the threshold bin to a candidate list
//   cand   per segment: exact radix select over the remaining 20 key bits of the candidates (ties
//          broken by lowest index), emit them, initialise persistent thresholds; the last CTA
//          publishes the arrival flag to every destination with release semantics.
// An "item" is one element (top-k, threshold-v) or one aligned block of 16 elements whose key is
// its L1 norm (threshold-v16).  Keys are non-negative floats compared through their bit patterns.
#include "device_utils.cuh"

namespace st {

namespace {

constexpr int kThreads = 256;
constexpr int kPerIter = kThreads * 4;  // elements one CTA covers per loop iteration

__device__ __forceinline__ uint32_t key_bits(float a) { return __float_as_uint(a) & 0x7fffffffu; }

__device__ __forceinline__ float4 load4_guarded(const float* p, uint32_t i, uint32_t valid) {
  if (i + 4 <= valid) return *reinterpret_cast<const float4*>(p + i);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i + 0 < valid) v.x = p[i + 0];
  if (i + 1 < valid) v.y = p[i + 1];
  if (i + 2 < valid) v.z = p[i + 2];
  return v;
}

__device__ __forceinline__ void store4_guarded(float* p, uint32_t i, uint32_t valid, float4 v) {
  if (i + 4 <= valid) {
    *reinterpret_cast<float4*>(p + i) = v;
    return;
  }
  if (i + 0 < valid) p[i + 0] = v.x;
  if (i + 1 < valid) p[i + 1] = v.y;
  if (i + 2 < valid) p[i + 2] = v.z;
}

// L1 norm of the 16-element block held by four consecutive lanes (one float4 each).  The
// reduction tree is fixed, so the value is identical in all four lanes and reproducible.
__device__ __forceinline__ float quad_l1(const float4& a) {
  float s = (fabsf(a.x) + fabsf(a.y)) + (fabsf(a.z) + fabsf(a.w));
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  return s;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// pass 1
// ------------------------------------------------------------------------------------------------
template <bool B16>
__global__ void __launch_bounds__(kThreads) k_pass1(SelectArgs A) {
  __shared__ uint32_t s_hist[kHistBins];
  __shared__ uint32_t s_tmp[kThreads / 32 + 1];

  const Chunk ch = A.chunks[blockIdx.x];
  const SegDesc sd = A.segs[ch.seg];
  const SegState ss = A.state[ch.seg];
  const bool need_hist = (A.compressor == kTopk) || (A.compressor == kThresholdv16) || !ss.inited;
  const bool need_count = (A.compressor != kTopk) && ss.inited;
  const uint32_t tau_bits = __float_as_uint(ss.tau);

  if (blockIdx.x == 0 && threadIdx.x == 0) *A.cand_cursor = 0;
  if (need_hist) {
    for (int b = threadIdx.x; b < kHistBins; b += kThreads) s_hist[b] = 0;
  }
  __syncthreads();

  const uint32_t seg_rel = ch.start - sd.off;
  // Gradients handed over per tensor are not padded: guard the tail.  Flat buckets are.
  const bool tab = A.grad_tab != nullptr;
  float* g = tab ? A.grad_tab[ch.seg] + seg_rel : A.grad + ch.start;
  const uint32_t g_valid = tab ? (sd.n > seg_rel ? min(ch.len, sd.n - seg_rel) : 0u) : ch.len;
  float* r = A.resid + ch.start;

  uint32_t cnt = 0, mx = 0;
  const uint32_t len_up = (ch.len + kPerIter - 1) / kPerIter * kPerIter;
  for (uint32_t i = threadIdx.x * 4; i < len_up; i += kPerIter) {
    const bool act = i < ch.len;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (act) {
      a = *reinterpret_cast<const float4*>(r + i);
      if (!A.skip_ef) {
        const float4 gv = load4_guarded(g, i, g_valid);
        a.x += gv.x; a.y += gv.y; a.z += gv.z; a.w += gv.w;
        // NaN policy: a NaN is dropped (neither sent nor kept), so it cannot poison the residual.
        if (!(a.x == a.x)) a.x = 0.f;
        if (!(a.y == a.y)) a.y = 0.f;
        if (!(a.z == a.z)) a.z = 0.f;
        if (!(a.w == a.w)) a.w = 0.f;
        *reinterpret_cast<float4*>(r + i) = a;
        if (A.zero_grad) store4_guarded(g, i, g_valid, make_float4(0.f, 0.f, 0.f, 0.f));
      }
    }
    if (!B16) {
      if (act) {
        const uint32_t k0 = key_bits(a.x), k1 = key_bits(a.y), k2 = key_bits(a.z), k3 = key_bits(a.w);
        if (need_hist) {
          atomicAdd(&s_hist[k0 >> kHistShift], 1u);
          atomicAdd(&s_hist[k1 >> kHistShift], 1u);
          atomicAdd(&s_hist[k2 >> kHistShift], 1u);
          atomicAdd(&s_hist[k3 >> kHistShift], 1u);
        }
        if (need_count) cnt += (k0 >= tau_bits) + (k1 >= tau_bits) + (k2 >= tau_bits) + (k3 >= tau_bits);
        mx = max(max(mx, k0), max(max(k1, k2), k3));
      }
    } else {
      const uint32_t key = __float_as_uint(quad_l1(a));
      if (act && (threadIdx.x & 3) == 0) {
        if (need_hist) atomicAdd(&s_hist[key >> kHistShift], 1u);
        if (need_count) cnt += (key >= tau_bits);
      }
    }
  }
  __syncthreads();
  if (need_hist) {
    uint32_t* gh = A.hist + (size_t)ch.seg * kHistBins;
    for (int b = threadIdx.x; b < kHistBins; b += kThreads) {
      const uint32_t h = s_hist[b];
      if (h) atomicAdd(&gh[b], h);
    }
  }
  uint32_t total;
  block_excl_scan(cnt, s_tmp, total);
  if (!B16) mx = block_max_u32(mx, s_tmp);
  if (threadIdx.x == 0) {
    A.chunk_cnt[blockIdx.x] = total;
    if (!B16 && mx) atomicMax(&A.work[ch.seg].max_bits, mx);
  }
}

// ------------------------------------------------------------------------------------------------
// plan
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) k_plan(SelectArgs A) {
  __shared__ uint32_t s_tmp[kThreads / 32 + 1];
  __shared__ uint32_t s_res[4];

  const uint32_t seg = blockIdx.x;
  const SegDesc sd = A.segs[seg];
  SegState ss = A.state[seg];
  SegWork* w = &A.work[seg];
  const uint32_t epoch = *A.epoch;
  const bool b16 = A.compressor == kThresholdv16;
  const uint32_t kk = b16 ? (sd.k + 15u) / 16u : sd.k;   // items to take

  // The receive slot about to be overwritten was last used two epochs ago; every destination
  // must have consumed it.  One thread of one CTA waits; the kernels that store come later in
  // the stream and read the status it leaves behind.
  if (seg == 0 && threadIdx.x == 0 && A.use_acks && epoch > 2) {
    const uint64_t want = (uint64_t)epoch - 2u;
    for (int p = 0; p < A.world; ++p) {
      if (!wait_ge_bounded(A.ack_local + (size_t)(epoch & 1u) * A.world + p, want, A.timeout_ns)) {
        set_status(A.status, kTimeoutAck);
        break;
      }
    }
  }

  uint32_t mode = kModeTop;
  uint32_t found = 0;
  if (A.compressor != kTopk && ss.inited) {
    // prefix sum of the per-chunk counts of this segment
    uint32_t carry = 0;
    for (uint32_t base = 0; base < sd.chunk_cnt; base += kThreads) {
      const uint32_t c = base + threadIdx.x;
      const uint32_t v = c < sd.chunk_cnt ? A.chunk_cnt[sd.chunk_begin + c] : 0u;
      uint32_t total;
      const uint32_t ex = block_excl_scan(v, s_tmp, total);
      if (c < sd.chunk_cnt) A.chunk_pos[sd.chunk_begin + c] = carry + ex;
      carry += total;
    }
    found = carry;
    // A zero threshold also matches the zero padding behind the tensor; padding sorts last, so
    // it is never emitted, but it must not count as "found".
    if (A.compressor == kThresholdv && __float_as_uint(ss.tau) == 0u) found -= (sd.n_pad - sd.n);
    if (A.compressor == kThresholdv) mode = kModeInOrder;
    else mode = ((uint64_t)found * 16u >= sd.k) ? kModeInOrder : kModeTop;
  }

  uint32_t* gh = A.hist + (size_t)seg * kHistBins;
  if (mode == kModeTop) {
    // suffix sums over the histogram, highest bin first; thread t owns 8 consecutive bins
    constexpr int kPer = kHistBins / kThreads;
    uint32_t h[kPer];
    uint32_t local = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      h[j] = gh[kHistBins - 1 - (threadIdx.x * kPer + j)];
      local += h[j];
    }
    uint32_t total;
    uint32_t running = block_excl_scan(local, s_tmp, total);
    if (threadIdx.x == 0) { s_res[0] = 0; s_res[1] = 0; s_res[2] = 0; }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      if (running < kk && running + h[j] >= kk) {
        s_res[0] = kHistBins - 1 - (threadIdx.x * kPer + j);
        s_res[1] = kk - running;
        s_res[2] = h[j];
      }
      running += h[j];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t k_rem = s_res[1], n_cand = s_res[2];
      uint32_t off = atomicAdd(A.cand_cursor, n_cand);
      if (k_rem == 0 || off + n_cand > A.cand_cap) {  // histogram incomplete or scratch too small
        set_status(A.status, kBadCandidate);
        k_rem = 0; off = 0; mode = kModeNone;
      }
      w->mode = mode;
      w->thr_bin = s_res[0];
      w->k_rem = k_rem;
      w->cand_off = off;
      w->cand_cnt = 0;
      w->out_cursor = 0;
      w->found = 0;
      w->max_saved = w->max_bits;
      w->max_bits = 0;
      w->tau_bits = 0;
      if (b16 && ss.inited) {   // under-filled: "must drop less" (thresholdv16.cpp:245-248)
        ss.tau *= 0.99f;
        A.state[seg] = ss;
      }
    }
  } else if (threadIdx.x == 0) {
    w->mode = mode;
    w->thr_bin = 0;
    w->k_rem = 0;
    w->cand_off = 0;
    w->cand_cnt = 0;
    w->out_cursor = 0;
    w->found = found;
    w->tau_bits = __float_as_uint(ss.tau);
    const float max_abs = __uint_as_float(w->max_bits);
    w->max_saved = w->max_bits;
    w->max_bits = 0;
    if (A.compressor == kThresholdv) {   // AIMD of thresholdv.cpp:70-76
      if (sd.k > found) ss.tau *= 0.99f;
      else if (sd.k < found) ss.tau = ss.tau + 0.01f * ((float)found / (float)sd.k) * max_abs;
    } else {                              // over-filled: thresholdv16.cpp:249-252
      ss.tau += ss.tau_inc;
    }
    A.state[seg] = ss;
  }
  // the histogram row is consumed; clear it for the next select
  for (int b = threadIdx.x; b < kHistBins; b += kThreads) gh[b] = 0;
}

// ------------------------------------------------------------------------------------------------
// pass 2
// ------------------------------------------------------------------------------------------------
template <bool B16>
__global__ void __launch_bounds__(kThreads) k_pass2(SelectArgs A) {
  __shared__ uint32_t s_tmp[kThreads / 32 + 1];
  if (ld_volatile_u32(A.status) != kOk) return;

  const Chunk ch = A.chunks[blockIdx.x];
  const SegDesc sd = A.segs[ch.seg];
  SegWork* wp = &A.work[ch.seg];
  const uint32_t mode = wp->mode;
  if (mode == kModeNone) return;
  const uint32_t thr_bin = wp->thr_bin;
  const uint32_t tau_bits = wp->tau_bits;
  const uint32_t cand_off = wp->cand_off;
  const uint32_t epoch = *A.epoch;
  const uint64_t slot_off = (uint64_t)(epoch & 1u) * A.slot_stride + sd.out_off;
  const uint32_t kk = B16 ? (sd.k + 15u) / 16u : sd.k;
  const uint32_t base_pos = A.chunk_pos[blockIdx.x];
  float* r = A.resid + ch.start;
  const int lane = threadIdx.x & 31;
  bool emitted = false;
  uint32_t running = 0;

  const uint32_t len_up = (ch.len + kPerIter - 1) / kPerIter * kPerIter;
  for (uint32_t i = threadIdx.x * 4; i < len_up; i += kPerIter) {
    const bool act = i < ch.len;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (act) a = *reinterpret_cast<const float4*>(r + i);
    const uint32_t gi = ch.start + i;   // bucket offset of a.x

    if (!B16) {
      const float av[4] = {a.x, a.y, a.z, a.w};
      uint32_t key[4];
      bool sel[4], cnd[4];
      uint32_t n_sel = 0, n_cnd = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        key[j] = key_bits(av[j]);
        if (mode == kModeTop) {
          const uint32_t bin = key[j] >> kHistShift;
          sel[j] = act && bin > thr_bin;
          cnd[j] = act && bin == thr_bin;
        } else {
          sel[j] = act && key[j] >= tau_bits;
          cnd[j] = false;
        }
        n_sel += sel[j];
        n_cnd += cnd[j];
      }
      uint32_t pos = 0;
      if (mode == kModeTop) {
        if (__any_sync(0xffffffffu, n_sel != 0)) {
          const uint32_t incl = warp_incl_scan(n_sel);
          uint32_t base = 0;
          if (lane == 31) base = atomicAdd(&wp->out_cursor, incl);
          base = __shfl_sync(0xffffffffu, base, 31);
          pos = base + incl - n_sel;
        }
        if (__any_sync(0xffffffffu, n_cnd != 0)) {
          const uint32_t incl = warp_incl_scan(n_cnd);
          uint32_t base = 0;
          if (lane == 31) base = atomicAdd(&wp->cand_cnt, incl);
          base = __shfl_sync(0xffffffffu, base, 31);
          uint32_t cpos = cand_off + base + incl - n_cnd;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (cnd[j]) A.cand[cpos++] = make_uint2(gi + j, key[j]);
        }
      } else {
        uint32_t total;
        const uint32_t ex = block_excl_scan(n_sel, s_tmp, total);
        pos = base_pos + running + ex;
        running += total;
      }
      if (n_sel) {
        float out[4] = {a.x, a.y, a.z, a.w};
        bool any = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (sel[j]) {
            if (pos < kk) {   // ordered mode truncates at k; the rest stays in the residual
              emit_entry(A, slot_off, pos, gi + j, av[j]);
              out[j] = 0.f;
              any = true;
            }
            ++pos;
          }
        }
        if (any) {
          *reinterpret_cast<float4*>(r + i) = make_float4(out[0], out[1], out[2], out[3]);
          emitted = true;
        }
      }
    } else {
      const uint32_t key = __float_as_uint(quad_l1(a));
      const bool leader = (lane & 3) == 0;
      bool sel, cnd = false;
      if (mode == kModeTop) {
        const uint32_t bin = key >> kHistShift;
        sel = act && bin > thr_bin;
        cnd = act && bin == thr_bin;
      } else {
        sel = act && key >= tau_bits;
      }
      const uint32_t n_sel = (leader && sel) ? 1u : 0u;
      uint32_t pos = 0;
      if (mode == kModeTop) {
        if (__any_sync(0xffffffffu, n_sel != 0)) {
          const uint32_t incl = warp_incl_scan(n_sel);
          uint32_t base = 0;
          if (lane == 31) base = atomicAdd(&wp->out_cursor, incl);
          base = __shfl_sync(0xffffffffu, base, 31);
          pos = base + incl - n_sel;
        }
        const uint32_t n_cnd = (leader && cnd) ? 1u : 0u;
        if (__any_sync(0xffffffffu, n_cnd != 0)) {
          const uint32_t incl = warp_incl_scan(n_cnd);
          uint32_t base = 0;
          if (lane == 31) base = atomicAdd(&wp->cand_cnt, incl);
          base = __shfl_sync(0xffffffffu, base, 31);
          if (n_cnd) A.cand[cand_off + base + incl - 1] = make_uint2(gi >> 4, key);
        }
      } else {
        uint32_t total;
        const uint32_t ex = block_excl_scan(n_sel, s_tmp, total);
        pos = base_pos + running + ex;
        running += total;
      }
      pos = __shfl_sync(0xffffffffu, pos, lane & ~3);   // block position from the quad leader
      if (sel && pos < kk) {
        const float av[4] = {a.x, a.y, a.z, a.w};
        const uint32_t e0 = pos * 16u + (uint32_t)(lane & 3) * 4u;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (e0 + j < sd.k) emit_entry(A, slot_off, e0 + j, gi + j, av[j]);
        // A truncated last block still leaves the residual exact: only emitted elements are zeroed.
        float4 o = a;
        if (e0 + 0 < sd.k) o.x = 0.f;
        if (e0 + 1 < sd.k) o.y = 0.f;
        if (e0 + 2 < sd.k) o.z = 0.f;
        if (e0 + 3 < sd.k) o.w = 0.f;
        *reinterpret_cast<float4*>(r + i) = o;
        emitted = true;
      }
    }
  }
  if (emitted) __threadfence_system();
}

// ------------------------------------------------------------------------------------------------
// candidates + completion
// ------------------------------------------------------------------------------------------------
constexpr int kCandThreads = 512;

__global__ void __launch_bounds__(kCandThreads) k_cand(SelectArgs A) {
  __shared__ uint32_t s_hist[1024];
  __shared__ uint32_t s_tmp[kCandThreads / 32 + 1];
  __shared__ uint32_t s_res[4];

  const uint32_t seg = blockIdx.x;
  const uint32_t tid = threadIdx.x;
  const SegDesc sd = A.segs[seg];
  SegWork* wp = &A.work[seg];
  const uint32_t epoch = *A.epoch;
  const bool ok = ld_volatile_u32(A.status) == kOk;
  const bool b16 = A.compressor == kThresholdv16;
  const uint32_t kk = b16 ? (sd.k + 15u) / 16u : sd.k;
  const uint64_t slot_off = (uint64_t)(epoch & 1u) * A.slot_stride + sd.out_off;
  const uint32_t mode = wp->mode;

  if (ok && mode == kModeTop) {
    const uint32_t c = wp->cand_cnt;
    const uint2* cand = A.cand + wp->cand_off;
    uint32_t rem = wp->k_rem, ties = 0;
    uint32_t prefix = 0, mask = 0;
    // two 10-bit digits over the low 20 key bits, largest first
    for (int pass = 0; pass < 2; ++pass) {
      const int shift = 10 - 10 * pass;
      for (int b = tid; b < 1024; b += kCandThreads) s_hist[b] = 0;
      __syncthreads();
      for (uint32_t i = tid; i < c; i += kCandThreads) {
        const uint32_t low = cand[i].y & 0xFFFFFu;
        if ((low & mask) == prefix) atomicAdd(&s_hist[(low >> shift) & 1023u], 1u);
      }
      __syncthreads();
      const uint32_t h0 = s_hist[1023 - 2 * tid], h1 = s_hist[1022 - 2 * tid];
      uint32_t total;
      const uint32_t ex = block_excl_scan(h0 + h1, s_tmp, total);
      if (ex < rem && ex + h0 >= rem) {
        s_res[0] = 1023 - 2 * tid; s_res[1] = rem - ex; s_res[2] = h0;
      } else if (ex + h0 < rem && ex + h0 + h1 >= rem) {
        s_res[0] = 1022 - 2 * tid; s_res[1] = rem - ex - h0; s_res[2] = h1;
      }
      __syncthreads();
      prefix |= s_res[0] << shift;
      mask |= 1023u << shift;
      rem = s_res[1];
      ties = s_res[2];
      __syncthreads();
    }
    const uint32_t t_key = (wp->thr_bin << kHistShift) | prefix;
    // among equal keys take the lowest item ids: radix select on the id, smallest first
    uint32_t id_thr = 0xFFFFFFFFu;
    if (rem < ties) {
      uint32_t ipre = 0, imask = 0, irem = rem;
      for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int b = tid; b < 256; b += kCandThreads) s_hist[b] = 0;
        __syncthreads();
        for (uint32_t i = tid; i < c; i += kCandThreads) {
          const uint2 e = cand[i];
          if (e.y == t_key && (e.x & imask) == ipre) atomicAdd(&s_hist[(e.x >> shift) & 255u], 1u);
        }
        __syncthreads();
        const uint32_t h = tid < 256 ? s_hist[tid] : 0u;
        uint32_t total;
        const uint32_t ex = block_excl_scan(h, s_tmp, total);
        if (tid < 256 && ex < irem && ex + h >= irem) { s_res[0] = tid; s_res[1] = irem - ex; }
        __syncthreads();
        ipre |= s_res[0] << shift;
        imask |= 255u << shift;
        irem = s_res[1];
        __syncthreads();
      }
      id_thr = ipre;
    }
    // threshold-v16: the lowest-ranked taken block goes last and may be truncated
    uint32_t last_id = id_thr;
    if (b16 && rem >= ties) {
      uint32_t mxid = 0;
      for (uint32_t i = tid; i < c; i += kCandThreads) {
        const uint2 e = cand[i];
        if (e.y == t_key) mxid = max(mxid, e.x);
      }
      last_id = block_max_u32(mxid, s_tmp);
    }
    bool emitted = false;
    for (uint32_t i = tid; i < c; i += kCandThreads) {
      const uint2 e = cand[i];
      const bool take = e.y > t_key || (e.y == t_key && e.x <= id_thr);
      if (!take) continue;
      emitted = true;
      if (!b16) {
        const uint32_t pos = atomicAdd(&wp->out_cursor, 1u);
        if (pos < kk) {
          emit_entry(A, slot_off, pos, e.x, A.resid[e.x]);
          A.resid[e.x] = 0.f;
        }
      } else {
        const bool is_last = (e.y == t_key && e.x == last_id);
        const uint32_t pos = is_last ? kk - 1 : atomicAdd(&wp->out_cursor, 1u);
        if (pos < kk) {
          const uint32_t base = e.x * 16u;
          for (uint32_t j = 0; j < 16u; ++j) {
            if (pos * 16u + j < sd.k) {
              emit_entry(A, slot_off, pos * 16u + j, base + j, A.resid[base + j]);
              A.resid[base + j] = 0.f;
            }
          }
        }
      }
    }
    if (emitted) __threadfence_system();
    if (tid == 0 && A.compressor != kTopk) {
      SegState ss = A.state[seg];
      if (!ss.inited) {
        // first threshold = the smallest selected key (thresholdv.cpp:27-37 takes the next one
        // down; the first AIMD step below is the one the reference applies right away)
        const float t0 = __uint_as_float(t_key);
        if (b16) {
          ss.tau_inc = 0.01f * t0;
          ss.tau = t0 + ss.tau_inc;
        } else {
          const float max_abs = __uint_as_float(wp->max_saved);
          ss.tau = t0 + 0.01f * ((float)(sd.k + 1) / (float)sd.k) * max_abs;
          ss.tau_inc = 0.f;
        }
        ss.inited = 1;
        A.state[seg] = ss;
      }
    }
  } else if (ok && mode == kModeInOrder && !b16 && wp->found < sd.k) {
    // threshold-v may under-fill (thresholdv.cpp:82): pad the fixed-size stream
    for (uint32_t p = wp->found + tid; p < sd.k; p += kCandThreads)
      emit_entry(A, slot_off, p, kSentinelIdx, 0.f);
    __threadfence_system();
  }

  // completion: the last CTA publishes the arrival flags and advances the epoch
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(A.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *A.done_ctr = 0;
      __threadfence_system();
      if (A.publish && ld_volatile_u32(A.status) == kOk) {
        for (int p = 0; p < A.world; ++p)
          st_release_sys_u64(A.flag[p] + (size_t)(epoch & 1u) * A.flag_slot_stride, (uint64_t)epoch);
      }
      *A.epoch = epoch + 1;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// random-k: k pseudo-random positions per segment (the reference's variant is dead code,
// backend/src/compress/randomk.cpp:125-164); counter-based generator, one CTA per segment.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

__global__ void __launch_bounds__(kThreads) k_randomk(SelectArgs A, uint32_t seed) {
  // Sampling is without replacement by construction: position j of the stream reads element
  // (start + j * stride) mod n with stride coprime to n, so no index repeats inside a stream.
  const uint32_t seg = blockIdx.x;
  const SegDesc sd = A.segs[seg];
  const uint32_t epoch = *A.epoch;
  const bool ok = ld_volatile_u32(A.status) == kOk;
  const uint64_t slot_off = (uint64_t)(epoch & 1u) * A.slot_stride + sd.out_off;
  if (ok) {
    const uint32_t h = mix32(seed ^ mix32(epoch * 0x9E3779B9u + seg));
    const uint32_t start = h % sd.n;
    uint32_t stride = (mix32(h) % sd.n) | 1u;
    // make stride coprime to n (n may be even or share odd factors): fall back to 1
    {
      uint32_t a = stride, b = sd.n;
      while (b) { const uint32_t t = a % b; a = b; b = t; }
      if (a != 1u) stride = 1u;
    }
    for (uint32_t j = threadIdx.x; j < sd.k; j += kThreads) {
      const uint32_t rel = (uint32_t)(((uint64_t)start + (uint64_t)j * stride) % sd.n);
      const uint32_t gi = sd.off + rel;
      emit_entry(A, slot_off, j, gi, A.resid[gi]);
      A.resid[gi] = 0.f;
    }
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(A.done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *A.done_ctr = 0;
      __threadfence_system();
      if (A.publish && ld_volatile_u32(A.status) == kOk) {
        for (int p = 0; p < A.world; ++p)
          st_release_sys_u64(A.flag[p] + (size_t)(epoch & 1u) * A.flag_slot_stride, (uint64_t)epoch);
      }
      *A.epoch = epoch + 1;
    }
  }
}

// Dense a = g + r, r <- a, g <- 0 without selection (first stage of random-k).
__global__ void __launch_bounds__(kThreads) k_ef_only(SelectArgs A) {
  const Chunk ch = A.chunks[blockIdx.x];
  const SegDesc sd = A.segs[ch.seg];
  const uint32_t seg_rel = ch.start - sd.off;
  const bool tab = A.grad_tab != nullptr;
  float* g = tab ? A.grad_tab[ch.seg] + seg_rel : A.grad + ch.start;
  const uint32_t g_valid = tab ? (sd.n > seg_rel ? min(ch.len, sd.n - seg_rel) : 0u) : ch.len;
  float* r = A.resid + ch.start;
  if (blockIdx.x == 0 && threadIdx.x == 0 && A.use_acks) {
    const uint32_t epoch = *A.epoch;
    if (epoch > 2) {
      for (int p = 0; p < A.world; ++p)
        if (!wait_ge_bounded(A.ack_local + (size_t)(epoch & 1u) * A.world + p, (uint64_t)epoch - 2u, A.timeout_ns)) {
          set_status(A.status, kTimeoutAck);
          break;
        }
    }
  }
  for (uint32_t i = threadIdx.x * 4; i < ch.len; i += kPerIter) {
    float4 a = *reinterpret_cast<const float4*>(r + i);
    const float4 gv = load4_guarded(g, i, g_valid);
    a.x += gv.x; a.y += gv.y; a.z += gv.z; a.w += gv.w;
    if (!(a.x == a.x)) a.x = 0.f;
    if (!(a.y == a.y)) a.y = 0.f;
    if (!(a.z == a.z)) a.z = 0.f;
    if (!(a.w == a.w)) a.w = 0.f;
    *reinterpret_cast<float4*>(r + i) = a;
    if (A.zero_grad) store4_guarded(g, i, g_valid, make_float4(0.f, 0.f, 0.f, 0.f));
  }
}

// ------------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------------
cudaError_t launch_select(const SelectArgs& A, uint32_t randomk_seed, cudaStream_t stream) {
  if (A.n_chunks == 0 || A.n_segs == 0) return cudaSuccess;
  if (A.world > kMaxWorld) return cudaErrorInvalidValue;
  if (A.compressor == kRandomk) {
    k_ef_only<<<A.n_chunks, kThreads, 0, stream>>>(A);
    k_randomk<<<A.n_segs, kThreads, 0, stream>>>(A, randomk_seed);
    return cudaGetLastError();
  }
  const bool b16 = A.compressor == kThresholdv16;
  if (b16) k_pass1<true><<<A.n_chunks, kThreads, 0, stream>>>(A);
  else     k_pass1<false><<<A.n_chunks, kThreads, 0, stream>>>(A);
  k_plan<<<A.n_segs, kThreads, 0, stream>>>(A);
  if (b16) k_pass2<true><<<A.n_chunks, kThreads, 0, stream>>>(A);
  else     k_pass2<false><<<A.n_chunks, kThreads, 0, stream>>>(A);
  k_cand<<<A.n_segs, kCandThreads, 0, stream>>>(A);
  return cudaGetLastError();
}

}  // namespace st
