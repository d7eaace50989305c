// Top-k selection without any device allocation: see noalloc_entry.h for who needs this and what
// it costs.  The selection itself is the same four-kernel chain the engine uses for a bucket
// (select_kernels.cu), run on a one-tensor "bucket" whose every table lives in the array below.
#include "noalloc_entry.h"

#include <mutex>
#include <stdio.h>

#include "launchers.h"

namespace {

constexpr uint32_t kMaxElems = ST_NOALLOC_MAX_ELEMS;
constexpr uint32_t kChunkElems = 16384;
constexpr uint32_t kMaxChunks = kMaxElems / kChunkElems;

// Layout of the working memory.  Offsets are multiples of 256 bytes.
struct Layout {
  static constexpr size_t resid = 0;                                          // kMaxElems floats
  static constexpr size_t cand = resid + sizeof(float) * kMaxElems;           // kMaxElems (id,key) pairs
  static constexpr size_t hist = cand + sizeof(uint2) * kMaxElems;            // kHistBins words
  static constexpr size_t chunks = hist + sizeof(uint32_t) * st::kHistBins;   // kMaxChunks Chunk records
  static constexpr size_t chunk_cnt = chunks + sizeof(st::Chunk) * kMaxChunks;
  static constexpr size_t chunk_pos = chunk_cnt + 256;
  static constexpr size_t seg = chunk_pos + 256;
  static constexpr size_t state = seg + 256;
  static constexpr size_t work = state + 256;
  static constexpr size_t control = work + 256;   // [0] epoch [1] done counter [2] status [3] candidate cursor
  static constexpr size_t end = control + 256;
};
static_assert(Layout::end <= ST_NOALLOC_SCRATCH_BYTES, "scratch array too small for its layout");
static_assert(sizeof(uint32_t) * kMaxChunks <= 256, "chunk counters must fit their slot");

// The working memory.  In host code this name is only a handle for cudaGetSymbolAddress; it is
// not a device address and must never be handed to a kernel as one.
static __device__ __align__(256) unsigned char g_scratch[ST_NOALLOC_SCRATCH_BYTES];

// Everything that must not carry over from the previous call is rewritten here: the private copy
// of the values (NaN -> 0, padding -> 0), histogram, tables and counters.
__global__ void __launch_bounds__(256) k_noalloc_setup(const float* values, uint32_t n, uint32_t n_pad, uint32_t k,
                                                       uint32_t n_chunks) {
  float* resid = reinterpret_cast<float*>(g_scratch + Layout::resid);
  const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t i = tid; i < n_pad; i += stride) {
    float v = i < n ? values[i] : 0.f;
    if (!(v == v)) v = 0.f;
    resid[i] = v;
  }
  uint32_t* hist = reinterpret_cast<uint32_t*>(g_scratch + Layout::hist);
  for (uint32_t i = tid; i < (uint32_t)st::kHistBins; i += stride) hist[i] = 0;
  st::Chunk* chunks = reinterpret_cast<st::Chunk*>(g_scratch + Layout::chunks);
  uint32_t* chunk_cnt = reinterpret_cast<uint32_t*>(g_scratch + Layout::chunk_cnt);
  uint32_t* chunk_pos = reinterpret_cast<uint32_t*>(g_scratch + Layout::chunk_pos);
  for (uint32_t c = tid; c < n_chunks; c += stride) {
    const uint32_t start = c * kChunkElems;
    st::Chunk ch;
    ch.seg = 0; ch.start = start; ch.len = min(kChunkElems, n_pad - start); ch.reserved = 0;
    chunks[c] = ch;
    chunk_cnt[c] = 0;
    chunk_pos[c] = 0;
  }
  if (tid == 0) {
    st::SegDesc sd;
    sd.off = 0; sd.n = n; sd.n_pad = n_pad; sd.k = k; sd.out_off = 0; sd.chunk_begin = 0; sd.chunk_cnt = n_chunks;
    sd.reserved = 0;
    *reinterpret_cast<st::SegDesc*>(g_scratch + Layout::seg) = sd;
    st::SegState ss = {};   // no threshold, coarse histogram window
    *reinterpret_cast<st::SegState*>(g_scratch + Layout::state) = ss;
    uint32_t* work = reinterpret_cast<uint32_t*>(g_scratch + Layout::work);
    for (uint32_t i = 0; i < sizeof(st::SegWork) / 4; ++i) work[i] = 0;
    uint32_t* ctl = reinterpret_cast<uint32_t*>(g_scratch + Layout::control);
    ctl[0] = 1; ctl[1] = 0; ctl[2] = 0; ctl[3] = 0;
  }
}

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_base[kMaxDevices] = {};   // device address of g_scratch, per device ordinal
thread_local char g_err[256] = "";

int fail(int code, const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess) snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
  else snprintf(g_err, sizeof(g_err), "%s", what);
  return code;
}

}  // namespace

extern "C" const char* st_noalloc_last_error(void) { return g_err; }

extern "C" int st_noalloc_status(uint32_t* status_out, cudaStream_t stream) {
  if (status_out == nullptr) return fail(ST_NOALLOC_ERR_BAD_ARG, "status_out must not be null");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ST_NOALLOC_ERR_CUDA, "cudaGetDevice", e);
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (dev >= 0 && dev < kMaxDevices) base = g_base[dev];
  }
  if (base == nullptr) return fail(ST_NOALLOC_ERR_BAD_ARG, "no selection has run on this device yet");
  // a plain copy into the caller's memory: nothing is allocated here either
  e = cudaMemcpyAsync(status_out, base + Layout::control + 2 * sizeof(uint32_t), sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(ST_NOALLOC_ERR_CUDA, "reading the status word", e);
  g_err[0] = 0;
  return ST_NOALLOC_OK;
}

extern "C" int st_topk_select_noalloc(const float* values, uint32_t n, uint32_t k, void* out_pairs,
                                      cudaStream_t stream) {
  if (n > kMaxElems) {
    snprintf(g_err, sizeof(g_err), "n = %u exceeds the built-in limit of %u elements", n, kMaxElems);
    return ST_NOALLOC_ERR_TOO_LARGE;
  }
  if (values == nullptr || out_pairs == nullptr || n == 0 || k == 0 || k > n)
    return fail(ST_NOALLOC_ERR_BAD_ARG, "need non-null buffers and 1 <= k <= n");
  if ((reinterpret_cast<uintptr_t>(values) & 3u) || (reinterpret_cast<uintptr_t>(out_pairs) & 7u))
    return fail(ST_NOALLOC_ERR_BAD_ARG, "values must be 4-byte aligned and out_pairs 8-byte aligned");

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ST_NOALLOC_ERR_CUDA, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(ST_NOALLOC_ERR_BAD_ARG, "device ordinal out of range");
  unsigned char* base = nullptr;
  {
    // Once per device, with that device current: ask the runtime where the array lives there.
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_base[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_scratch);
      if (e != cudaSuccess) return fail(ST_NOALLOC_ERR_CUDA, "cudaGetSymbolAddress", e);
      g_base[dev] = static_cast<unsigned char*>(p);
    }
    base = g_base[dev];
  }

  const uint32_t n_pad = (n + 15u) / 16u * 16u;
  const uint32_t n_chunks = (n_pad + kChunkElems - 1) / kChunkElems;
  int grid = (int)((n_pad + 1023u) / 1024u);
  if (grid > 148 * 4) grid = 148 * 4;
  k_noalloc_setup<<<grid, 256, 0, stream>>>(values, n, n_pad, k, n_chunks);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(ST_NOALLOC_ERR_CUDA, "setup launch", e);

  st::SelectArgs A = {};
  A.grad = nullptr;
  A.grad_tab = nullptr;
  A.resid = reinterpret_cast<float*>(base + Layout::resid);
  A.segs = reinterpret_cast<const st::SegDesc*>(base + Layout::seg);
  A.state = reinterpret_cast<st::SegState*>(base + Layout::state);
  A.work = reinterpret_cast<st::SegWork*>(base + Layout::work);
  A.chunks = reinterpret_cast<const st::Chunk*>(base + Layout::chunks);
  A.chunk_cnt = reinterpret_cast<uint32_t*>(base + Layout::chunk_cnt);
  A.chunk_pos = reinterpret_cast<uint32_t*>(base + Layout::chunk_pos);
  A.hist = reinterpret_cast<uint32_t*>(base + Layout::hist);
  A.cand = reinterpret_cast<uint2*>(base + Layout::cand);
  uint32_t* ctl = reinterpret_cast<uint32_t*>(base + Layout::control);
  A.cand_cursor = ctl + 3;
  A.cand_cap = kMaxElems;
  A.n_segs = 1;
  A.n_chunks = n_chunks;
  A.n_total = n_pad;
  A.compressor = st::kTopk;
  A.zero_grad = 0;
  A.skip_ef = 1;                 // the private copy already holds the values
  A.world = 1;
  A.rank = 0;
  A.out[0] = static_cast<uint2*>(out_pairs);
  A.out_mc = nullptr;
  A.slot_stride = 0;             // a single output area, whatever the epoch's parity
  A.flag_slot_stride = 0;
  A.ack_local = nullptr;
  A.use_acks = 0;
  A.publish = 0;
  A.epoch = ctl + 0;
  A.done_ctr = ctl + 1;
  A.status = ctl + 2;
  A.timeout_ns = 0;
  e = st::launch_select(A, 0u, stream);
  if (e != cudaSuccess) return fail(ST_NOALLOC_ERR_CUDA, "select launch", e);
  g_err[0] = 0;
  return ST_NOALLOC_OK;
}
