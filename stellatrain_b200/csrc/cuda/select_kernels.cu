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

// Gradients are read once: streaming loads and stores (evict-first) keep them from pushing the
// residual, which pass 2 reads again, out of L2.
__device__ __forceinline__ float4 load4_guarded(const float* p, uint32_t i, uint32_t valid) {
  if (i + 4 <= valid) return __ldcs(reinterpret_cast<const float4*>(p + i));
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i + 0 < valid) v.x = p[i + 0];
  if (i + 1 < valid) v.y = p[i + 1];
  if (i + 2 < valid) v.z = p[i + 2];
  return v;
}

__device__ __forceinline__ void store4_guarded(float* p, uint32_t i, uint32_t valid, float4 v) {
  if (i + 4 <= valid) {
    __stcs(reinterpret_cast<float4*>(p + i), v);
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
// histogram window
// ------------------------------------------------------------------------------------------------
struct HistWindow {
  uint32_t base, shift;
};

__device__ __forceinline__ HistWindow window_of(const SegState& ss) {
  HistWindow w;
  w.base = ss.hist_shift ? ss.hist_base : 0u;
  w.shift = ss.hist_shift ? ss.hist_shift : (uint32_t)kHistShift;
  return w;
}

// Monotone in key, so "bin > b" implies "key above every key of bin b".
__device__ __forceinline__ uint32_t bin_of(uint32_t key, const HistWindow& w) {
  if (key < w.base) return 0u;
  const uint32_t b = (key - w.base) >> w.shift;
  return b < (uint32_t)(kHistBins - 1) ? b : (uint32_t)(kHistBins - 1);
}

// Window for the next select: 2048 bins of 2^13 key units (2^-10 relative) centred on `key`,
// i.e. one octave to either side; keys outside fall into the two end bins.
__device__ __forceinline__ void centre_window(SegState& ss, uint32_t key) {
  const uint32_t half = (uint32_t)(kHistBins / 2) << kFineShift;
  ss.hist_shift = kFineShift;
  ss.hist_base = key > half ? key - half : 0u;
}

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
  const HistWindow win = window_of(ss);

  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *A.cand_cursor = 0;
    if (A.stamps != nullptr) A.stamps[0] = global_timer_ns();
  }
  if (sd.reserved & kSegSkip) {
    // a tensor another rank of the group is responsible for: only clear the consumed gradient
    if (A.zero_grad && A.grad_tab == nullptr) {
      float* gz = A.grad + ch.start;
      for (uint32_t i = threadIdx.x * 4; i < ch.len; i += kPerIter)
        *reinterpret_cast<float4*>(gz + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (threadIdx.x == 0) A.chunk_cnt[blockIdx.x] = 0;
    return;
  }
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

  // Bin 0 is never counted (plan derives it from the item count) and the top bin is counted in a
  // register: with a window centred on the threshold these two bins hold most items, and counting
  // them with shared-memory atomics would serialise on two addresses.
  uint32_t cnt = 0, mx = 0, top = 0;
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
        const uint32_t key[4] = {key_bits(a.x), key_bits(a.y), key_bits(a.z), key_bits(a.w)};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (need_hist) {
            const uint32_t b = bin_of(key[j], win);
            if (b == (uint32_t)(kHistBins - 1)) ++top;
            else if (b != 0u) atomicAdd(&s_hist[b], 1u);
          }
          if (need_count) cnt += (key[j] >= tau_bits);
          mx = max(mx, key[j]);
        }
      }
    } else {
      const uint32_t key = __float_as_uint(quad_l1(a));
      if (act && (threadIdx.x & 3) == 0) {
        if (need_hist) {
          const uint32_t b = bin_of(key, win);
          if (b == (uint32_t)(kHistBins - 1)) ++top;
          else if (b != 0u) atomicAdd(&s_hist[b], 1u);
        }
        if (need_count) cnt += (key >= tau_bits);
      }
    }
  }
  __syncthreads();
  uint32_t total, top_total = 0;
  if (need_hist) {
    uint32_t* gh = A.hist + (size_t)ch.seg * kHistBins;
    for (int b = threadIdx.x; b < kHistBins; b += kThreads) {
      const uint32_t h = s_hist[b];
      if (h) atomicAdd(&gh[b], h);
    }
    block_excl_scan(top, s_tmp, top_total);
    if (threadIdx.x == 0 && top_total) atomicAdd(&gh[kHistBins - 1], top_total);
  }
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
  const uint32_t n_items = b16 ? sd.n_pad / 16u : sd.n_pad;

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

  uint32_t* gh_skip = A.hist + (size_t)seg * kHistBins;
  if (sd.reserved & kSegSkip) {
    if (threadIdx.x == 0) { w->mode = kModeNone; w->k_rem = 0; w->cand_cnt = 0; w->out_cursor = 0; w->found = 0; }
    for (int b = threadIdx.x; b < kHistBins; b += kThreads) gh_skip[b] = 0;
    return;
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
    // bin 0 is not counted by pass 1: it holds whatever the other bins do not
    if (threadIdx.x == kThreads - 1) h[kPer - 1] = n_items > total ? n_items - total : 0u;
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
      centre_window(ss, __float_as_uint(ss.tau));   // keep the fallback histogram centred
    }
    A.state[seg] = ss;
  }
  // the histogram row is consumed; clear it for the next select
  for (int b = threadIdx.x; b < kHistBins; b += kThreads) gh[b] = 0;
}

// ------------------------------------------------------------------------------------------------
// pass 2
// ------------------------------------------------------------------------------------------------
constexpr uint32_t kQueueCap = 1024;   // per-CTA staging of selected / candidate items (16 KB: four CTAs fit one SM)
constexpr uint32_t kP2PerThread = 16;  // consecutive elements per thread: one block of threshold-v16
constexpr uint32_t kP2PerIter = kThreads * kP2PerThread;

// Every thread owns 16 consecutive elements per iteration (four independent 16-byte loads in
// flight), and the CTA needs one scan per 4096 elements to turn per-thread counts into stream
// positions.  Ordered mode writes at chunk_pos + rank; unordered mode stages items in shared memory
// and reserves positions with ONE global atomic per flush, so that stores into peer memory are
// consecutive and the per-segment cursor is not hammered by every warp.
template <bool B16>
__global__ void __launch_bounds__(kThreads, 4) k_pass2(SelectArgs A) {
  __shared__ uint32_t s_tmp[kThreads / 32 + 1];
  __shared__ uint2 s_sel[B16 ? 1 : kQueueCap];      // element mode: (idx, value bits)
  __shared__ uint32_t s_selb[B16 ? kQueueCap : 1];  // block mode: block ids
  __shared__ uint2 s_cnd[kQueueCap];                // (item id, key)
  __shared__ uint32_t s_base[2];
  extern __shared__ __align__(128) float s_dyn[];            // two stages of the TMA pipeline
  float (*s_tile)[kP2PerIter] = reinterpret_cast<float (*)[kP2PerIter]>(s_dyn);
  __shared__ __align__(8) uint64_t s_bar[2];
  if (ld_volatile_u32(A.status) != kOk) return;

  // The tiles need nothing but the chunk's place: start their copies first, so that they travel while the
  // tensor's descriptor, work record and threshold state (a second level of dependent loads) are fetched.
  const Chunk ch = A.chunks[blockIdx.x];
  float* r = A.resid + ch.start;
  const uint32_t n_tiles = (ch.len + kP2PerIter - 1) / kP2PerIter;
  auto issue_tile = [&](uint32_t t) {     // thread 0 only
    const uint32_t elems = min(kP2PerIter, ch.len - t * kP2PerIter);
    mbar_expect_tx(&s_bar[t & 1u], elems * 4u);
    bulk_load(&s_tile[t & 1u][0], r + (size_t)t * kP2PerIter, elems * 4u, &s_bar[t & 1u]);
  };
  if (threadIdx.x == 0) {
    mbar_init(&s_bar[0], 1);
    mbar_init(&s_bar[1], 1);
    mbar_init_fence();
    issue_tile(0);
    if (n_tiles > 1) issue_tile(1);
  }
  __syncthreads();   // the barriers are initialised before anyone waits on them

  const SegDesc sd = A.segs[ch.seg];
  SegWork* wp = &A.work[ch.seg];
  const uint32_t mode = wp->mode;
  if (mode == kModeNone) {
    // nothing to do for this tensor, but no copy into this CTA's shared memory may outlive it
    mbar_wait_bounded(&s_bar[0], 0u);
    if (n_tiles > 1) mbar_wait_bounded(&s_bar[1], 0u);
    return;
  }
  const uint32_t thr_bin = wp->thr_bin;
  const uint32_t tau_bits = wp->tau_bits;
  const uint32_t cand_off = wp->cand_off;
  const HistWindow win = window_of(A.state[ch.seg]);
  const uint32_t epoch = *A.epoch;
  const uint64_t slot_off = (uint64_t)(epoch & 1u) * A.slot_stride + sd.out_off;
  const int dest = dest_of(A, sd);
  const uint32_t nb = narrow_base_of(sd);
  const uint32_t kk = B16 ? (sd.k + 15u) / 16u : sd.k;
  const uint32_t base_pos = A.chunk_pos[blockIdx.x];
  uint32_t running = 0;
  uint32_t fill_sel = 0, fill_cnd = 0;   // uniform over the CTA
  // key range of the threshold bin: [key_lo, key_hi); keys are below 2^31, so 2^31 stands for "none above"
  const uint64_t lo64 = thr_bin == 0u ? 0ull : (uint64_t)win.base + ((uint64_t)thr_bin << win.shift);
  const uint64_t hi64 = thr_bin == (uint32_t)(kHistBins - 1) ? 0x80000000ull
                                                              : (uint64_t)win.base + ((uint64_t)(thr_bin + 1u) << win.shift);
  const uint32_t key_lo = (uint32_t)(lo64 < 0x80000000ull ? lo64 : 0x80000000ull);
  const uint32_t key_hi = (uint32_t)(hi64 < 0x80000000ull ? hi64 : 0x80000000ull);

  auto emit_block = [&](uint32_t pos, uint32_t gi0) {   // one 16-element block at block position pos
#pragma unroll 4
    for (uint32_t e = 0; e < 16u; ++e) {
      const uint32_t p = pos * 16u + e;
      if (p < sd.k) {
        const float a = A.resid[gi0 + e], sv = wire_value(nb, a);
        emit_entry(A, dest, nb, slot_off, p, gi0 + e, sv);
        A.resid[gi0 + e] = a - sv;
      }
    }
  };

  auto flush = [&]() {
    __syncthreads();
    if (threadIdx.x == 0) {
      s_base[0] = fill_sel ? atomicAdd(&wp->out_cursor, fill_sel) : 0u;
      s_base[1] = fill_cnd ? atomicAdd(&wp->cand_cnt, fill_cnd) : 0u;
    }
    __syncthreads();
    const uint32_t b_sel = s_base[0], b_cnd = s_base[1];
    if (!B16) {
      for (uint32_t j = threadIdx.x; j < fill_sel; j += kThreads) {
        const uint2 e = s_sel[j];
        if (b_sel + j < kk) emit_entry(A, dest, nb, slot_off, b_sel + j, e.x, __uint_as_float(e.y));
      }
    } else {
      for (uint32_t t = threadIdx.x; t < fill_sel * 16u; t += kThreads) {
        const uint32_t q = t >> 4, e = t & 15u;
        const uint32_t gi = s_selb[q] * 16u + e;
        const uint32_t p = (b_sel + q) * 16u + e;
        if (p < sd.k) {
          const float a = A.resid[gi], sv = wire_value(nb, a);
          emit_entry(A, dest, nb, slot_off, p, gi, sv);
          A.resid[gi] = a - sv;
        }
      }
    }
    for (uint32_t j = threadIdx.x; j < fill_cnd; j += kThreads) A.cand[cand_off + b_cnd + j] = s_cnd[j];
    fill_sel = 0;
    fill_cnd = 0;
    __syncthreads();
  };

  // Tiles of 4096 elements travel global -> shared by TMA bulk copies, two in flight (started above).
  for (uint32_t tile = 0; tile < n_tiles; ++tile) {
    const uint32_t it = tile * kP2PerIter;
    const uint32_t i = it + threadIdx.x * kP2PerThread;
    const bool act = i < ch.len;   // chunk lengths are multiples of 16: a thread is all in or all out
    // The exit on a copy that never lands is taken by the whole CTA or by nobody: the scans below contain
    // barriers, and a copy into this CTA's shared memory must not be in flight when the CTA retires.
    const bool landed = mbar_wait_bounded(&s_bar[tile & 1u], (tile >> 1) & 1u);
    if (!__syncthreads_and(landed)) {
      if (threadIdx.x == 0) {
        set_status(A.status, kTimeoutFlag);   // cannot happen for a valid source; never spin forever
        // tile + 1 was started together with this one (or when tile - 1 was consumed): wait for it too, bounded
        if (tile + 1 < n_tiles) mbar_wait_bounded(&s_bar[(tile + 1) & 1u], ((tile + 1) >> 1) & 1u);
        if (!landed) mbar_wait_bounded(&s_bar[tile & 1u], (tile >> 1) & 1u);
      }
      __syncthreads();
      return;
    }
    float v[16];
    if (act) {
      const float4* src = reinterpret_cast<const float4*>(&s_tile[tile & 1u][threadIdx.x * kP2PerThread]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 a = src[q];
        v[4 * q + 0] = a.x; v[4 * q + 1] = a.y; v[4 * q + 2] = a.z; v[4 * q + 3] = a.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = 0.f;
    }
    const uint32_t gi = ch.start + i;   // bucket offset of v[0]

    uint32_t sel_mask = 0, cnd_mask = 0, bkey = 0;
    if (!B16) {
      // "bin > thr_bin" and "bin == thr_bin" as two key comparisons (bin_of is monotone), and a
      // whole-thread early out: almost every thread holds nothing at or above the threshold bin
      const uint32_t cut = (mode == kModeTop) ? key_lo : tau_bits;
      uint32_t kmax = 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) kmax = max(kmax, key_bits(v[j]));
      if (act && kmax >= cut) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t key = key_bits(v[j]);
          if (mode == kModeTop) {
            sel_mask |= (uint32_t)(key >= key_hi) << j;
            cnd_mask |= (uint32_t)(key >= key_lo && key < key_hi) << j;
          } else {
            sel_mask |= (uint32_t)(key >= tau_bits) << j;
          }
        }
      }
    } else {
      float g[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        g[q] = (fabsf(v[4 * q]) + fabsf(v[4 * q + 1])) + (fabsf(v[4 * q + 2]) + fabsf(v[4 * q + 3]));
      bkey = __float_as_uint((g[0] + g[1]) + (g[2] + g[3]));   // same tree as quad_l1
      if (mode == kModeTop) {
        const uint32_t bin = bin_of(bkey, win);
        sel_mask = act && bin > thr_bin;
        cnd_mask = act && bin == thr_bin;
      } else {
        sel_mask = act && bkey >= tau_bits;
      }
    }
    const uint32_t n_sel = __popc(sel_mask), n_cnd = __popc(cnd_mask);
    uint32_t total;
    const uint32_t ex = block_excl_scan(n_sel | (n_cnd << 16), s_tmp, total);
    const uint32_t t_sel = total & 0xffffu, t_cnd = total >> 16;
    // every thread has copied its part of the stage into registers (the scan's barriers are behind
    // those reads): the stage can take the tile after next
    if (threadIdx.x == 0 && tile + 2 < n_tiles) issue_tile(tile + 2);

    if (mode == kModeTop) {
      if (fill_sel + t_sel > kQueueCap || fill_cnd + t_cnd > kQueueCap) flush();
      const bool direct = t_sel > kQueueCap || t_cnd > kQueueCap;   // dense selection: bypass the queue
      uint32_t p = fill_sel + (ex & 0xffffu), q = fill_cnd + (ex >> 16);
      if (direct) {
        __syncthreads();
        if (threadIdx.x == 0) {
          s_base[0] = atomicAdd(&wp->out_cursor, t_sel);
          s_base[1] = atomicAdd(&wp->cand_cnt, t_cnd);
        }
        __syncthreads();
        p = s_base[0] + (ex & 0xffffu);
        q = cand_off + s_base[1] + (ex >> 16);
      }
      if (!B16) {
        if (sel_mask | cnd_mask) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (sel_mask >> j & 1u) {
              const float sv = wire_value(nb, v[j]);
              if (direct) { if (p < kk) emit_entry(A, dest, nb, slot_off, p, gi + j, sv); }
              else s_sel[p] = make_uint2(gi + j, __float_as_uint(sv));
              ++p;
              v[j] -= sv;   // exactly zero unless the wire format rounds
            }
            if (cnd_mask >> j & 1u) {
              const uint2 c = make_uint2(gi + j, key_bits(v[j]));
              if (direct) A.cand[q] = c; else s_cnd[q] = c;
              ++q;
            }
          }
          if (sel_mask) {
#pragma unroll
            for (int qd = 0; qd < 4; ++qd)
              *reinterpret_cast<float4*>(r + i + 4 * qd) = make_float4(v[4 * qd], v[4 * qd + 1], v[4 * qd + 2], v[4 * qd + 3]);
          }
        }
      } else {
        if (sel_mask) {
          if (direct) emit_block(p, gi);
          else s_selb[p] = gi >> 4;
        }
        if (cnd_mask) {
          const uint2 c = make_uint2(gi >> 4, bkey);
          if (direct) A.cand[q] = c; else s_cnd[q] = c;
        }
      }
      if (!direct) {
        fill_sel += t_sel;
        fill_cnd += t_cnd;
      }
    } else {
      uint32_t pos = base_pos + running + (ex & 0xffffu);
      running += t_sel;
      if (sel_mask) {
        if (!B16) {
          bool any = false;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (sel_mask >> j & 1u) {
              if (pos < kk) {   // ordered mode truncates at k; the rest stays in the residual
                const float sv = wire_value(nb, v[j]);
                emit_entry(A, dest, nb, slot_off, pos, gi + j, sv);
                v[j] -= sv;
                any = true;
              }
              ++pos;
            }
          }
          if (any) {
#pragma unroll
            for (int qd = 0; qd < 4; ++qd)
              *reinterpret_cast<float4*>(r + i + 4 * qd) = make_float4(v[4 * qd], v[4 * qd + 1], v[4 * qd + 2], v[4 * qd + 3]);
          }
        } else if (pos < kk) {
          // a truncated last block still leaves the residual exact: only emitted elements are zeroed
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (pos * 16u + j < sd.k) {
              const float sv = wire_value(nb, v[j]);
              emit_entry(A, dest, nb, slot_off, pos * 16u + j, gi + j, sv);
              v[j] -= sv;
            }
          }
#pragma unroll
          for (int qd = 0; qd < 4; ++qd)
            *reinterpret_cast<float4*>(r + i + 4 * qd) = make_float4(v[4 * qd], v[4 * qd + 1], v[4 * qd + 2], v[4 * qd + 3]);
        }
      }
    }
  }
  if (mode == kModeTop && (fill_sel | fill_cnd)) flush();
  // No fence here: the arrival flag is published by the last kernel of the chain, and a kernel
  // boundary on the stream already orders these stores before anything that kernel does.
}

// ------------------------------------------------------------------------------------------------
// candidates + completion
// ------------------------------------------------------------------------------------------------
// Debug checks: hand every destination the sum over the entries this select stored into it, and clear
// the accumulators for the next select.  Called by the one thread that publishes the arrival flags, before
// them (their release orders these stores too).
__device__ __forceinline__ void publish_checksums(const SelectArgs& A, uint32_t epoch) {
  if (A.stamps != nullptr) {
    A.stamps[1] = global_timer_ns();
    A.stamps[4] = epoch;
  }
  if (A.cksum_acc == nullptr) return;
  for (int p = 0; p < A.world; ++p) {
    const uint32_t sum = atomicAdd(A.cksum_acc + (A.owner_mode ? p : 0), 0u);
    if (A.cksum[p] != nullptr) A.cksum[p][(size_t)(epoch & 1u) * A.cksum_slot_stride] = sum;
  }
  for (int p = 0; p < kMaxWorld; ++p) A.cksum_acc[p] = 0u;
  __threadfence_system();
}

constexpr int kCandThreads = 1024;
constexpr int kCandIlp = 4;   // independent loads in flight per thread

// Called by a whole CTA of kCandThreads threads.  Among cand[0..c) takes the `rem` largest keys (equal keys: lowest
// item id first; 1 <= rem <= c) and emits them: stream positions come from wp->out_cursor, except that the
// lowest-ranked taken block of threshold-v16 goes to `last_pos`, where it may be cut off at sd.k.  Returns the key
// of the lowest-ranked taken item.  s_hist: 2048 words, s_tmp: kCandThreads / 32 + 1 words, s_res: 4 words.
__device__ __forceinline__ uint32_t take_top(const SelectArgs& A, const SegDesc& sd, SegWork* wp, const uint2* cand,
                                             uint32_t c, uint32_t rem, bool b16, uint32_t kk, uint32_t last_pos,
                                             uint64_t slot_off, int dest, uint32_t nb, uint32_t* s_hist,
                                             uint32_t* s_tmp, uint32_t* s_res) {
  const uint32_t tid = threadIdx.x;
  uint32_t ties = 0;
  uint32_t prefix = 0, mask = 0;
  // radix select over the full 31-bit key, largest first: digits of 11, 11 and 9 bits
  const int shifts[3] = {20, 9, 0};
  const uint32_t widths[3] = {2048u, 2048u, 512u};
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = shifts[pass];
    const uint32_t nbins = widths[pass];
    for (uint32_t b = tid; b < nbins; b += kCandThreads) s_hist[b] = 0;
    __syncthreads();
    for (uint32_t i0 = tid; i0 < c; i0 += kCandThreads * kCandIlp) {
      uint32_t key[kCandIlp];
#pragma unroll
      for (int u = 0; u < kCandIlp; ++u) {
        const uint32_t i = i0 + u * kCandThreads;
        key[u] = i < c ? cand[i].y : 0xFFFFFFFFu;
      }
#pragma unroll
      for (int u = 0; u < kCandIlp; ++u)
        if (key[u] != 0xFFFFFFFFu && (key[u] & mask) == prefix) atomicAdd(&s_hist[(key[u] >> shift) & (nbins - 1)], 1u);
    }
    __syncthreads();
    // thread t owns bins nbins-1-2t and nbins-2-2t (descending)
    const uint32_t h0 = 2 * tid < nbins ? s_hist[nbins - 1 - 2 * tid] : 0u;
    const uint32_t h1 = 2 * tid + 1 < nbins ? s_hist[nbins - 2 - 2 * tid] : 0u;
    uint32_t total;
    const uint32_t ex = block_excl_scan(h0 + h1, s_tmp, total);
    if (ex < rem && ex + h0 >= rem) {
      s_res[0] = nbins - 1 - 2 * tid; s_res[1] = rem - ex; s_res[2] = h0;
    } else if (ex + h0 < rem && ex + h0 + h1 >= rem) {
      s_res[0] = nbins - 2 - 2 * tid; s_res[1] = rem - ex - h0; s_res[2] = h1;
    }
    __syncthreads();
    prefix |= s_res[0] << shift;
    mask |= (nbins - 1) << shift;
    rem = s_res[1];
    ties = s_res[2];
    __syncthreads();
  }
  const uint32_t t_key = prefix;
  // among equal keys take the lowest item ids: radix select on the id, smallest first
  uint32_t id_thr = 0xFFFFFFFFu;
  if (rem < ties) {
    uint32_t ipre = 0, imask = 0, irem = rem;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (uint32_t b = tid; b < 256; b += kCandThreads) s_hist[b] = 0;
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
  for (uint32_t i = tid; i < c; i += kCandThreads) {
    const uint2 e = cand[i];
    const bool take = e.y > t_key || (e.y == t_key && e.x <= id_thr);
    if (!take) continue;
    if (!b16) {
      const uint32_t pos = atomicAdd(&wp->out_cursor, 1u);
      if (pos < kk) {
        const float a = A.resid[e.x], sv = wire_value(nb, a);
        emit_entry(A, dest, nb, slot_off, pos, e.x, sv);
        A.resid[e.x] = a - sv;
      }
    } else {
      const bool is_last = (e.y == t_key && e.x == last_id);
      const uint32_t pos = is_last ? last_pos : atomicAdd(&wp->out_cursor, 1u);
      if (pos < kk) {
        const uint32_t base = e.x * 16u;
        for (uint32_t j = 0; j < 16u; ++j) {
          if (pos * 16u + j < sd.k) {
            const float a = A.resid[base + j], sv = wire_value(nb, a);
            emit_entry(A, dest, nb, slot_off, pos * 16u + j, base + j, sv);
            A.resid[base + j] = a - sv;
          }
        }
      }
    }
  }
  return t_key;
}

// Completion of a select chain, called by thread 0 of every CTA of its last kernel after a CTA barrier: the last
// CTA publishes the arrival flags and advances the epoch.  The CTA barrier orders the CTA's stores before this
// thread's system-scope fence, the counter orders the CTAs.
__device__ __forceinline__ void finish_select(const SelectArgs& A, uint32_t epoch) {
  __threadfence_system();
  const uint32_t prev = atomicAdd(A.done_ctr, 1u);
  if (prev == gridDim.x - 1) {
    *A.done_ctr = 0;
    __threadfence_system();
    publish_checksums(A, epoch);
    if (A.publish && ld_volatile_u32(A.status) == kOk) {
      for (int p = 0; p < A.world; ++p)
        st_release_sys_u64(A.flag[p] + (size_t)(epoch & 1u) * A.flag_slot_stride, (uint64_t)epoch);
    }
    *A.epoch = epoch + 1;
  }
}

__global__ void __launch_bounds__(kCandThreads) k_cand(SelectArgs A) {
  __shared__ uint32_t s_hist[2048];
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
  const int dest = dest_of(A, sd);
  const uint32_t nb = narrow_base_of(sd);
  const uint32_t mode = wp->mode;

  if (ok && mode == kModeTop) {
    const uint32_t t_key = take_top(A, sd, wp, A.cand + wp->cand_off, wp->cand_cnt, wp->k_rem, b16, kk, kk - 1u, slot_off,
                                    dest, nb, s_hist, s_tmp, s_res);
    if (tid == 0) {
      SegState ss = A.state[seg];
      // Next select: centre the histogram on the threshold just found, unless it fell off the
      // window (the distribution moved by more than an octave), then start coarse again.
      const uint32_t tb = wp->thr_bin;
      if (tb == 0u || tb == (uint32_t)(kHistBins - 1)) { ss.hist_shift = 0; ss.hist_base = 0; }
      else centre_window(ss, t_key);
      if (A.compressor != kTopk && !ss.inited) {
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
      }
      A.state[seg] = ss;
    }
  } else if (ok && mode == kModeInOrder && !b16 && wp->found < sd.k) {
    // threshold-v may under-fill (thresholdv.cpp:82): pad the fixed-size stream
    for (uint32_t p = wp->found + tid; p < sd.k; p += kCandThreads)
      emit_entry(A, dest, nb, slot_off, p, kSentinelIdx, 0.f);
  }

  __syncthreads();
  if (tid == 0) {
    wp->cand_cnt = 0;      // the one-pass select appends its near-miss blocks behind a zero count
    wp->found = 0;
    finish_select(A, epoch);
  }
}

// ------------------------------------------------------------------------------------------------
// one-pass select of the threshold modes
// ------------------------------------------------------------------------------------------------
// Threshold-v and threshold-v16 know their threshold before they look at the data (it persists per tensor,
// backend/src/compress/thresholdv.cpp:44-52, backend/src/compress/thresholdv16.cpp:81-97), so once a tensor has
// one the select needs a single pass over gradient and residual:
//   fused   a = g + r, r <- a; items at or over the threshold are counted per chunk, the chunks of a tensor chain
//           their counts (decoupled look-back, one 64-bit word per chunk) so that every item learns its position in
//           index order, and the first k of them go straight into the destinations' receive areas and are cleared
//           in r.  Blocks just under the threshold are noted as candidates for the fill.
//   finish  per tensor: threshold-v pads an under-filled stream; threshold-v16 completes it with the best of
//           the rejected blocks (backend/src/compress/thresholdv16.cpp:261-293: its heap), taken from the noted
//           candidates or, when those do not suffice, from a scan of the whole tensor by this CTA, so the
//           stream always holds exactly what the two-pass chain would have chosen; then the
//           threshold steps (AIMD) and the last CTA publishes the arrival flags.
// 12 bytes per element cross HBM (read g, read r, write r) against 16 to 20 of the two-pass chain.
constexpr int kFusedMaxIter = 16;                              // iterations of kPerIter elements per chunk
constexpr uint32_t kFusedMaxChunk = kFusedMaxIter * kPerIter;  // 16384 elements
constexpr uint32_t kLookbackPolls = 1u << 20;                  // bound of every wait on a predecessor chunk
constexpr float kWindowDefault = 0.05f;                        // candidates: keys in [tau * (1 - window), tau)

__device__ __forceinline__ uint64_t ld_relaxed_gpu_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_relaxed_gpu_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// State word of a chunk: select epoch (so that a word of an earlier select never counts) | kind | item count.
// kind 1: the chunk's own count; kind 2: the count of the chunk and of all chunks of the tensor before it.
__device__ __forceinline__ uint64_t chunk_word(uint32_t epoch, uint32_t kind, uint32_t value) {
  return ((uint64_t)epoch << 32) | ((uint64_t)kind << 30) | (uint64_t)value;
}

// Run by warp 0 of a chunk's CTA.  Publishes the chunk's count, then walks back over the chunks of the tensor,
// 32 at a time, adding counts until one carries an inclusive prefix.  Returns the number of items of the tensor
// in front of this chunk.  Every wait is bounded: *good is false when a predecessor never published, and the
// chunk then still publishes a prefix so that the chunks behind it do not wait for it in turn.
__device__ __forceinline__ uint32_t chunk_lookback(uint64_t* state, uint32_t first, uint32_t mine, uint32_t epoch,
                                                   uint32_t total, bool* good) {
  const uint32_t lane = threadIdx.x & 31u;
  if (mine == first) {
    if (lane == 0) st_relaxed_gpu_u64(state + mine, chunk_word(epoch, 2u, total));
    *good = true;
    return 0u;
  }
  if (lane == 0) st_relaxed_gpu_u64(state + mine, chunk_word(epoch, 1u, total));
  uint32_t base = 0;
  bool ok = true;
  uint32_t j = mine;   // chunks [first, j) are not accounted for yet
  while (j > first) {
    uint32_t kind = 2u, val = 0u;   // lanes that reach past the tensor's first chunk stand for "prefix 0"
    if (j - first > lane) {
      const uint64_t* p = state + (j - 1u - lane);
      uint64_t w = ld_relaxed_gpu_u64(p);
      for (uint32_t polls = 0; (uint32_t)(w >> 32) != epoch && polls < kLookbackPolls; ++polls) {
        __nanosleep(64);
        w = ld_relaxed_gpu_u64(p);
      }
      if ((uint32_t)(w >> 32) != epoch) ok = false;
      else { kind = (uint32_t)(w >> 30) & 3u; val = (uint32_t)w & 0x3FFFFFFFu; }
    }
    const uint32_t has_prefix = __ballot_sync(0xffffffffu, kind == 2u);
    const uint32_t upto = has_prefix ? (uint32_t)__ffs((int)has_prefix) - 1u : 31u;
    base += __reduce_add_sync(0xffffffffu, lane <= upto ? val : 0u);
    if (has_prefix) break;
    j -= 32u;
  }
  ok = __all_sync(0xffffffffu, ok);
  if (lane == 0) st_relaxed_gpu_u64(state + mine, chunk_word(epoch, 2u, base + total));
  *good = ok;
  return base;
}

// The receive slot about to be overwritten was last used two epochs ago; every destination must have consumed
// it.  One thread calls this right before its CTA stores into the destinations.
__device__ __forceinline__ bool acks_arrived(const SelectArgs& A, uint32_t epoch) {
  if (!A.use_acks || epoch <= 2u) return true;
  const uint64_t want = (uint64_t)epoch - 2u;
  for (int p = 0; p < A.world; ++p) {
    if (!wait_ge_bounded(A.ack_local + (size_t)(epoch & 1u) * A.world + p, want, A.timeout_ns)) {
      set_status(A.status, kTimeoutAck);
      return false;
    }
  }
  return true;
}

template <bool B16>
__global__ void __launch_bounds__(kThreads, 8) k_fused(SelectArgs A) {
  constexpr int kWarps = kThreads / 32;
  __shared__ uint32_t s_cnt[kFusedMaxIter * kWarps];        // items over the threshold per (iteration, warp)
  __shared__ uint32_t s_tmp[kWarps + 1];
  __shared__ uint2 s_cnd[B16 ? kFusedMaxChunk / 16 : 1];    // near-miss blocks of this chunk: (block id, key)
  __shared__ uint32_t s_word[6];   // [0] candidates staged, [1] items in front of the chunk, [2] candidate base, [3] may emit,
                                   // [4] selected blocks staged, [5] unused
  // Selected blocks wait here, values and all, until their stream positions are known: the emission then needs no
  // second walk over the chunk and no second read of r.  A chunk holds kStage blocks over the threshold only when the
  // threshold is far too low; it then falls back to walking the chunk again.
  constexpr uint32_t kStage = B16 ? 48u : 1u;
  __shared__ float4 s_sval[kStage * 4];     // the block's 16 values, one float4 per lane of the block
  __shared__ uint2 s_smeta[kStage];         // (offset of the block in the chunk, cell << 8 | blocks of lower lanes in the cell)

  // The chunk's place is all the first loads need: they are on their way while the tensor's descriptor, threshold
  // and gradient pointer (a second level of dependent loads) are fetched.
  const Chunk ch = A.chunks[blockIdx.x];
  float* r = A.resid + ch.start;
  const uint32_t i0 = threadIdx.x * 4;
  float4 r_next = make_float4(0.f, 0.f, 0.f, 0.f), g_next = r_next;
  if (i0 < ch.len) r_next = *reinterpret_cast<const float4*>(r + i0);
  const SegDesc sd = A.segs[ch.seg];
  const SegState ss = A.state[ch.seg];
  SegWork* wp = &A.work[ch.seg];
  const uint32_t epoch = *A.epoch;
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;

  if (blockIdx.x == 0 && threadIdx.x == 0 && A.stamps != nullptr) A.stamps[0] = global_timer_ns();
  if (sd.reserved & kSegSkip) {
    // a tensor another rank of the group is responsible for: only clear the consumed gradient
    if (A.zero_grad && A.grad_tab == nullptr) {
      float* gz = A.grad + ch.start;
      for (uint32_t i = threadIdx.x * 4; i < ch.len; i += kPerIter)
        *reinterpret_cast<float4*>(gz + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    return;
  }
  if (threadIdx.x == 0) { s_word[0] = 0; s_word[4] = 0; }

  const uint32_t seg_rel = ch.start - sd.off;
  const bool tab = A.grad_tab != nullptr;
  float* g = tab ? A.grad_tab[ch.seg] + seg_rel : A.grad + ch.start;
  const uint32_t g_valid = tab ? (sd.n > seg_rel ? min(ch.len, sd.n - seg_rel) : 0u) : ch.len;
  const bool add = !A.skip_ef;
  if (add && i0 < ch.len) g_next = load4_guarded(g, i0, g_valid);
  // a tensor without a threshold yet selects nothing here: the finishing kernel then takes the exact top items
  const uint32_t tau_bits = ss.inited ? __float_as_uint(ss.tau) : 0xFFFFFFFFu;
  const uint32_t kk = B16 ? (sd.k + 15u) / 16u : sd.k;
  const bool collect = B16 && ss.inited;
  float window = __uint_as_float(ss.reserved[0]);
  if (!(window > 0.f && window <= 1.f)) window = kWindowDefault;
  const uint32_t lo_bits = collect ? __float_as_uint(fmaxf(ss.tau * (1.f - window), 0.f)) : 0xFFFFFFFFu;
  const uint32_t n_iter = (ch.len + kPerIter - 1) / kPerIter;   // the launcher guarantees <= kFusedMaxIter
  __syncthreads();   // s_word[0] is cleared before anyone stages a candidate

  uint32_t selbits = 0;   // B16: bit `it` = this lane's block of iteration `it` is over the threshold
  uint64_t selmask = 0;   // element mode: 4 bits per iteration
  uint32_t mx = 0;
  for (uint32_t it = 0; it < n_iter; ++it) {
    const uint32_t i = it * kPerIter + threadIdx.x * 4;
    const bool act = i < ch.len;
    float4 a = r_next;
    const float4 gv = g_next;
    {
      // the loads of the next iteration leave before this iteration's values are touched
      const uint32_t in = i + kPerIter;
      if (it + 1 < n_iter && in < ch.len) {
        r_next = *reinterpret_cast<const float4*>(r + in);
        if (add) g_next = load4_guarded(g, in, g_valid);
      }
    }
    if (act && add) {
      a.x += gv.x; a.y += gv.y; a.z += gv.z; a.w += gv.w;
      // NaN policy: a NaN is dropped (neither sent nor kept), so it cannot poison the residual.
      if (!(a.x == a.x)) a.x = 0.f;
      if (!(a.y == a.y)) a.y = 0.f;
      if (!(a.z == a.z)) a.z = 0.f;
      if (!(a.w == a.w)) a.w = 0.f;
      *reinterpret_cast<float4*>(r + i) = a;
      if (A.zero_grad) store4_guarded(g, i, g_valid, make_float4(0.f, 0.f, 0.f, 0.f));
    }
    if (!act) a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (B16) {
      const uint32_t key = __float_as_uint(quad_l1(a));   // the same value in the four lanes of a block
      const bool sel = act && key >= tau_bits;
      const uint32_t leaders = __ballot_sync(0xffffffffu, sel) & 0x11111111u;
      if (lane == 0) s_cnt[it * kWarps + warp] = __popc(leaders);
      selbits |= (uint32_t)sel << it;
      if (leaders) {
        uint32_t slot = 0;
        if (sel && (lane & 3u) == 0u) slot = atomicAdd(&s_word[4], 1u);
        slot = __shfl_sync(0xffffffffu, slot, lane & ~3u);
        if (sel && slot < kStage) {
          s_sval[slot * 4u + (lane & 3u)] = a;
          if ((lane & 3u) == 0u)
            s_smeta[slot] = make_uint2(i, ((it * kWarps + warp) << 8) | __popc(leaders & ((1u << lane) - 1u)));
        }
      }
      if (collect && act && !sel && (lane & 3u) == 0u && key >= lo_bits && key != 0u) {
        const uint32_t slot = atomicAdd(&s_word[0], 1u);
        s_cnd[slot] = make_uint2((ch.start + i) >> 4, key);
      }
    } else {
      const uint32_t key[4] = {key_bits(a.x), key_bits(a.y), key_bits(a.z), key_bits(a.w)};
      uint32_t m4 = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // the zero padding behind the tensor never counts, whatever the threshold
        if (act && seg_rel + i + j < sd.n) {
          m4 |= (uint32_t)(key[j] >= tau_bits) << j;
          mx = max(mx, key[j]);
        }
      }
      const uint32_t n = __reduce_add_sync(0xffffffffu, (uint32_t)__popc(m4));
      if (lane == 0) s_cnt[it * kWarps + warp] = n;
      selmask |= (uint64_t)m4 << (4u * it);
    }
  }
  __syncthreads();

  // positions: exclusive prefix over (iteration, warp) cells in index order, then over the chunks of the tensor
  const uint32_t n_cells = n_iter * kWarps;
  uint32_t total;
  const uint32_t cell = threadIdx.x < n_cells ? s_cnt[threadIdx.x] : 0u;
  const uint32_t cell_ex = block_excl_scan(cell, s_tmp, total);
  if (threadIdx.x < n_cells) s_cnt[threadIdx.x] = cell_ex;
  if (!B16) {
    mx = block_max_u32(mx, s_tmp);
    if (threadIdx.x == 0 && mx) atomicMax(&wp->max_bits, mx);
  }
  if (warp == 0) {
    bool good;
    const uint32_t base = chunk_lookback(A.chunk_state, sd.chunk_begin, blockIdx.x, epoch, total, &good);
    if (lane == 0) {
      if (!good) set_status(A.status, kTimeoutScan);
      s_word[1] = base;
      if (B16) s_word[2] = s_word[0] ? atomicAdd(&wp->cand_cnt, s_word[0]) : 0u;
      if (blockIdx.x == sd.chunk_begin + sd.chunk_cnt - 1u) wp->found = base + total;
      bool may = total != 0u && base < kk && ld_volatile_u32(A.status) == kOk;
      if (may) may = acks_arrived(A, epoch);
      s_word[3] = may ? 1u : 0u;
    }
  }
  __syncthreads();

  if (B16 && s_word[0]) {
    uint2* region = A.cand + (sd.off >> 4);   // one slot per block of the tensor: can never overflow
    const uint32_t cb = s_word[2];
    for (uint32_t j = threadIdx.x; j < s_word[0]; j += kThreads) region[cb + j] = s_cnd[j];
  }
  if (!s_word[3]) return;

  const uint32_t base = s_word[1];
  const uint64_t slot_off = (uint64_t)(epoch & 1u) * A.slot_stride + sd.out_off;
  const int dest = dest_of(A, sd);
  const uint32_t nb = narrow_base_of(sd);
  if (B16 && s_word[4] <= kStage) {
    // one thread per lane of a staged block
    const uint32_t n_staged = s_word[4];
    for (uint32_t j = threadIdx.x; j < n_staged * 4u; j += kThreads) {
      const uint32_t b = j >> 2, q = j & 3u;
      const uint2 meta = s_smeta[b];
      const uint32_t pos = base + s_cnt[meta.y >> 8] + (meta.y & 0xFFu);
      if (pos >= kk) continue;   // beyond the budget: the block stays in the residual
      const float4 a = s_sval[j];
      float v[4] = {a.x, a.y, a.z, a.w};
      const uint32_t p0 = pos * 16u + q * 4u, i = meta.x + q * 4u;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (p0 + e < sd.k) {   // a truncated last block leaves the residual exact: only emitted elements are cleared
          const float sv = wire_value(nb, v[e]);
          emit_entry(A, dest, nb, slot_off, p0 + e, ch.start + i + e, sv);
          v[e] -= sv;
        }
      }
      *reinterpret_cast<float4*>(r + i) = make_float4(v[0], v[1], v[2], v[3]);
    }
    return;
  }
  for (uint32_t it = 0; it < n_iter; ++it) {
    const uint32_t i = it * kPerIter + threadIdx.x * 4;
    if (B16) {
      const bool sel = (selbits >> it) & 1u;
      const uint32_t leaders = __ballot_sync(0xffffffffu, sel) & 0x11111111u;
      if (!sel) continue;
      const uint32_t before = __popc(leaders & ((1u << (lane & ~3u)) - 1u));   // blocks of lower lanes
      const uint32_t pos = base + s_cnt[it * kWarps + warp] + before;
      if (pos >= kk) continue;   // beyond the budget: the block stays in the residual
      float4 a = *reinterpret_cast<const float4*>(r + i);
      float v[4] = {a.x, a.y, a.z, a.w};
      const uint32_t p0 = pos * 16u + (lane & 3u) * 4u;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (p0 + e < sd.k) {   // a truncated last block leaves the residual exact: only emitted elements are cleared
          const float sv = wire_value(nb, v[e]);
          emit_entry(A, dest, nb, slot_off, p0 + e, ch.start + i + e, sv);
          v[e] -= sv;
        }
      }
      *reinterpret_cast<float4*>(r + i) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      const uint32_t m4 = (uint32_t)(selmask >> (4u * it)) & 15u;
      const uint32_t n = __popc(m4);
      uint32_t pos = base + s_cnt[it * kWarps + warp] + warp_incl_scan(n) - n;
      if (!m4 || pos >= kk) continue;
      float4 a = *reinterpret_cast<const float4*>(r + i);
      float v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (m4 >> j & 1u) {
          if (pos < kk) {   // ordered mode truncates at k; the rest stays in the residual
            const float sv = wire_value(nb, v[j]);
            emit_entry(A, dest, nb, slot_off, pos, ch.start + i + j, sv);
            v[j] -= sv;
          }
          ++pos;
        }
      }
      // the padding of the tensor's last float4 is zero and stays zero
      *reinterpret_cast<float4*>(r + i) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}

__global__ void __launch_bounds__(kCandThreads) k_finish(SelectArgs A) {
  __shared__ uint32_t s_hist[2048];
  __shared__ uint32_t s_tmp[kCandThreads / 32 + 1];
  __shared__ uint32_t s_res[4];
  __shared__ uint32_t s_n[2];   // [0] candidates found by the scan, [1] acknowledgements arrived
  __shared__ uint32_t s_in[3];  // found, noted candidates, "has a threshold" as read by thread 0

  const uint32_t seg = blockIdx.x;
  const uint32_t tid = threadIdx.x;
  const SegDesc sd = A.segs[seg];
  SegWork* wp = &A.work[seg];
  const uint32_t epoch = *A.epoch;
  const bool ok = ld_volatile_u32(A.status) == kOk;
  const bool b16 = A.compressor == kThresholdv16;
  const uint32_t kk = b16 ? (sd.k + 15u) / 16u : sd.k;
  const uint64_t slot_off = (uint64_t)(epoch & 1u) * A.slot_stride + sd.out_off;
  const int dest = dest_of(A, sd);
  const uint32_t nb = narrow_base_of(sd);

  if (ok && !(sd.reserved & kSegSkip)) {
    // Thread 0 rewrites the tensor's state and work record at the end: everything the CTA branches on is read
    // once, handed out through shared memory, and a barrier stands between the last read and the first write.
    if (tid == 0) {
      s_in[0] = wp->found;
      s_in[1] = wp->cand_cnt;
      s_in[2] = A.state[seg].inited;
    }
    __syncthreads();
    SegState ss = A.state[seg];
    ss.inited = s_in[2];
    const uint32_t found = s_in[0];            // items at or over the threshold in the whole tensor
    const uint32_t c_win = s_in[1];            // near-miss blocks the one-pass kernel noted
    const bool short_of = found < kk;
    uint32_t t_key = 0;
    bool scanned = false;
    if (short_of) {
      if (tid == 0) s_n[1] = acks_arrived(A, epoch) ? 1u : 0u;
      __syncthreads();
      if (s_n[1]) {
        if (!b16) {
          // threshold-v may under-fill (thresholdv.cpp:82): pad the fixed-size stream
          for (uint32_t p = found + tid; p < sd.k; p += kCandThreads)
            emit_entry(A, dest, nb, slot_off, p, kSentinelIdx, 0.f);
        } else {
          const uint32_t need = kk - found, n_blocks = sd.n_pad / 16u;
          uint2* cand = A.cand + (sd.off >> 4);
          uint32_t c = min(c_win, n_blocks);   // the candidate region holds one slot per block of the tensor
          if (!ss.inited || c < need) {
            // every block that still holds something is a candidate: the blocks over the threshold were all
            // emitted (the stream is short of them) and are zero in the residual by now
            scanned = true;
            if (tid == 0) s_n[0] = 0;
            __syncthreads();
            constexpr uint32_t kRound = kCandThreads / 4;   // blocks per round, four lanes each
            const float* src = A.resid + sd.off + (tid & 3u) * 4u;
            for (uint32_t b0 = 0; b0 < n_blocks; b0 += 4u * kRound) {
              float4 a[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {   // four independent loads in flight
                const uint32_t b = b0 + u * kRound + (tid >> 2);
                a[u] = b < n_blocks ? *reinterpret_cast<const float4*>(src + (size_t)b * 16u) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const uint32_t b = b0 + u * kRound + (tid >> 2);
                const uint32_t key = __float_as_uint(quad_l1(a[u]));
                if (b < n_blocks && (tid & 3u) == 0u && key != 0u) {
                  const uint32_t slot = atomicAdd(&s_n[0], 1u);
                  cand[slot] = make_uint2((sd.off >> 4) + b, key);
                }
              }
            }
            __syncthreads();
            c = s_n[0];
          }
          const uint32_t take = min(need, c);
          if (take && c <= (uint32_t)kCandThreads) {
            // few candidates: every thread ranks one of them against all others in shared memory (larger key
            // first, equal keys by lower block id), and rank q goes to stream position found + q
            uint2* s_one = reinterpret_cast<uint2*>(s_hist);       // kCandThreads pairs
            uint32_t* s_take = s_hist;                              // reused once the ranks are known
            const uint2 mine = tid < c ? __ldcg(cand + tid) : make_uint2(0u, 0u);
            s_one[tid] = mine;
            __syncthreads();
            uint32_t rank = 0;
            if (tid < c) {
              for (uint32_t j = 0; j < c; ++j) {
                const uint2 o = s_one[j];
                rank += (o.y > mine.y || (o.y == mine.y && o.x < mine.x)) ? 1u : 0u;
              }
            }
            __syncthreads();
            if (tid < c && rank < take) s_take[rank] = mine.x;
            if (tid < c && rank == take - 1u) s_res[0] = mine.y;
            __syncthreads();
            t_key = s_res[0];
            for (uint32_t e = tid; e < take * 16u; e += kCandThreads) {
              const uint32_t q = e >> 4, j = e & 15u;
              const uint32_t p = (found + q) * 16u + j;
              if (p < sd.k) {   // only the lowest-ranked block can be cut off
                const uint32_t gi = s_take[q] * 16u + j;
                const float a = A.resid[gi], sv = wire_value(nb, a);
                emit_entry(A, dest, nb, slot_off, p, gi, sv);
                A.resid[gi] = a - sv;
              }
            }
          } else if (take) {
            if (tid == 0) wp->out_cursor = found;
            __syncthreads();
            t_key = take_top(A, sd, wp, cand, c, take, true, kk, found + take - 1u, slot_off, dest, nb, s_hist, s_tmp, s_res);
          }
          // fewer blocks with anything in them than the budget: the rest of the stream says "no entry"
          for (uint32_t p = (found + take) * 16u + tid; p < sd.k; p += kCandThreads)
            emit_entry(A, dest, nb, slot_off, p, kSentinelIdx, 0.f);
        }
      }
    }
    __syncthreads();   // every thread is past its reads of the state and of the work record
    if (tid == 0) {
      if (!b16) {
        const float max_abs = __uint_as_float(wp->max_bits);
        if (ss.inited) {   // AIMD of thresholdv.cpp:70-76
          if (sd.k > found) ss.tau *= 0.99f;
          else if (sd.k < found) ss.tau = ss.tau + 0.01f * ((float)found / (float)sd.k) * max_abs;
        }
      } else if (!ss.inited) {
        if (short_of && s_n[1]) {   // first threshold: the smallest selected key plus the first additive step
          const float t0 = __uint_as_float(t_key);
          ss.tau_inc = 0.01f * t0;
          ss.tau = t0 + ss.tau_inc;
          ss.inited = 1;
        }
      } else {
        if (short_of) ss.tau *= 0.99f;      // "must drop less" (thresholdv16.cpp:245-248)
        else ss.tau += ss.tau_inc;          // thresholdv16.cpp:249-252
        {
          // Keep a sixteenth to a quarter of the budget in near-miss blocks, and at least twice what this fill took:
          // the additive and multiplicative steps of the threshold move the count of blocks over it by a few per
          // cent, which is all a fill ever needs, and ranking the candidates costs time in proportion to their number.
          float w = __uint_as_float(ss.reserved[0]);
          if (!(w > 0.f && w <= 1.f)) w = kWindowDefault;
          const uint32_t needed = short_of ? kk - found : 0u;
          if (scanned) w *= 2.f;
          else if (c_win < kk / 16u + 8u || c_win < 2u * needed) w *= 1.5f;
          else if (c_win > kk / 4u + 32u) w *= 0.75f;
          ss.reserved[0] = __float_as_uint(fminf(fmaxf(w, 1e-3f), 1.f));
        }
      }
      A.state[seg] = ss;
      wp->cand_cnt = 0;
      wp->found = 0;
      wp->max_bits = 0;
    }
  }

  __syncthreads();
  if (tid == 0) finish_select(A, epoch);
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
  const int dest = dest_of(A, sd);
  const uint32_t nb = narrow_base_of(sd);
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
      const float a = A.resid[gi], sv = wire_value(nb, a);
      emit_entry(A, dest, nb, slot_off, j, gi, sv);
      A.resid[gi] = a - sv;
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
      publish_checksums(A, epoch);
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
  if (blockIdx.x == 0 && threadIdx.x == 0 && A.stamps != nullptr) A.stamps[0] = global_timer_ns();
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
bool fused_select_possible(const SelectArgs& A, uint32_t max_chunk_len) {
  return (A.compressor == kThresholdv || A.compressor == kThresholdv16) && A.chunk_state != nullptr &&
         max_chunk_len <= kFusedMaxChunk && A.n_total < (1u << 30);
}

cudaError_t launch_select_fused(const SelectArgs& A, cudaStream_t stream) {
  if (A.n_chunks == 0 || A.n_segs == 0) return cudaSuccess;
  if (A.world > kMaxWorld || A.chunk_state == nullptr) return cudaErrorInvalidValue;
  if (A.compressor == kThresholdv16) k_fused<true><<<A.n_chunks, kThreads, 0, stream>>>(A);
  else if (A.compressor == kThresholdv) k_fused<false><<<A.n_chunks, kThreads, 0, stream>>>(A);
  else return cudaErrorInvalidValue;
  k_finish<<<A.n_segs, kCandThreads, 0, stream>>>(A);
  return cudaGetLastError();
}

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
  constexpr int kTileBytes = 2 * kP2PerIter * sizeof(float);
  {
    // opt in to more than 48 KB of shared memory, once per device
    static bool ready[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !ready[dev]) {
      e = cudaFuncSetAttribute(k_pass2<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileBytes);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(k_pass2<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileBytes);
      if (e != cudaSuccess) return e;
      ready[dev] = true;
    }
  }
  if (b16) k_pass2<true><<<A.n_chunks, kThreads, kTileBytes, stream>>>(A);
  else     k_pass2<false><<<A.n_chunks, kThreads, kTileBytes, stream>>>(A);
  k_cand<<<A.n_segs, kCandThreads, 0, stream>>>(A);
  return cudaGetLastError();
}

}  // namespace st
