// Shared host/device plain-data types of the GPU-resident sparse data-parallel path.
//
// One "bucket" is a flat fp32 range that holds several parameter tensors ("segments"), each
// starting on a 16-element (64-byte) boundary and zero-padded to a multiple of 16.  All per-tensor
// semantics of the reference engine (k per tensor: backend/src/engine/modules/compress.cpp:44-52,
// threshold per tensor: backend/src/compress/thresholdv16.cpp:81-97) live in the segment tables.
#pragma once
#include <stdint.h>

namespace st {

constexpr int kMaxWorld = 16;          // peers addressable by one kernel launch
constexpr int kHistBits = 11;          // first radix digit: exponent + 3 mantissa bits of |x|
constexpr int kHistBins = 1 << kHistBits;
constexpr int kHistShift = 31 - kHistBits;  // shift of the coarse window
constexpr int kFineShift = 13;              // shift of the window centred on the previous threshold
constexpr uint32_t kSentinelIdx = 0xFFFFFFFFu;  // "no entry" marker in an (idx,val) stream

enum Compressor : uint32_t { kTopk = 0, kThresholdv = 1, kThresholdv16 = 2, kRandomk = 3 };
enum SegMode : uint32_t { kModeNone = 0, kModeInOrder = 1, kModeTop = 2 };

// Status word written by kernels, read by the host. 0 means success; the first error wins.
enum Status : uint32_t {
  kOk = 0,
  kTimeoutAck = 1,    // a peer did not acknowledge the previous use of a receive slot in time
  kTimeoutFlag = 2,   // a peer's stream did not arrive in time
  kBadIndex = 3,      // a received index is outside the bucket
  kBadCandidate = 4,  // candidate scratch exhausted (cannot happen with a correctly sized scratch)
  kBadSize = 5,       // request exceeds a compiled-in limit
  kBadChecksum = 6,   // debug checks: a received stream does not add up to what its source sent
  kTimeoutScan = 7,   // one-pass select: a chunk never saw the item count of the chunk in front of it
};

struct SegDesc {          // static per segment (re-uploaded when the compression ratio changes)
  uint32_t off;           // first element inside the bucket, multiple of 16
  uint32_t n;             // valid elements
  uint32_t n_pad;         // n rounded up to 16
  uint32_t k;             // entries this rank emits for the segment
  uint32_t out_off;       // position of the segment's first entry in the bucket's stream
  uint32_t chunk_begin;   // first chunk of the segment in the chunk table
  uint32_t chunk_cnt;     // number of chunks
  uint32_t reserved;      // flags: kSegSkip
};

constexpr uint32_t kSegSkip = 1u;   // this rank does not own the tensor (grouped mode): emit nothing, keep no residual
// Partitioned optimiser state: bits 8..15 of SegDesc.reserved name the rank that keeps the tensor's
// optimiser state, receives every rank's entries for it and writes the new parameter values back.
// Narrow wire format: a tensor of fewer than 65536 (padded) elements whose descriptor carries this flag
// sends 4-byte entries, (index relative to the tensor : 16 | bf16 value : 16), packed at the start of the
// tensor's region of the stream; 0xFFFFFFFF is "no entry".  Role of the reference's u16 index and fp16 value
// wire casts (backend/src/engine/comm_manager.cpp:487-571, 579-583), with an unsigned index.
constexpr uint32_t kSegNarrow = 2u;
constexpr uint32_t kNarrowLimit = 65536u;
constexpr uint32_t kNotNarrow = 0xFFFFFFFFu;
constexpr uint32_t kSegOwnerShift = 8u;
constexpr uint32_t kSegOwnerMask = 0xFFu;

struct SegState {         // persistent per segment, saved in checkpoints
  float tau;              // threshold (element magnitude or 16-block L1 norm)
  float tau_inc;          // additive step of threshold-v16
  uint32_t inited;        // 0 until the first threshold was measured
  // Histogram window of the next select: bin(key) = clamp((key - hist_base) >> hist_shift, 0, 2047).
  // hist_shift == 0 means "coarse": base 0, shift 20 (exponent + 3 mantissa bits).  After a select
  // the window is centred on the k-th largest key found, so that in steady state the bin that
  // holds the next threshold is 2^-10 wide (relative) and the candidate set is tiny.
  uint32_t hist_base;
  uint32_t hist_shift;
  // reserved[0]: float bits of the one-pass select's candidate window (blocks with a key in
  // [tau * (1 - window), tau) are noted for the fill); 0 = not set yet.
  uint32_t reserved[3];
};

struct SegWork {          // scratch per segment, valid within one select
  uint32_t mode;          // SegMode
  uint32_t thr_bin;       // histogram bin that contains the k-th largest key
  uint32_t k_rem;         // items still to be taken from that bin
  uint32_t cand_off;      // start of the segment's candidate range in the candidate scratch
  uint32_t cand_cnt;      // candidates appended so far
  uint32_t out_cursor;    // items appended to the stream so far (unordered mode)
  uint32_t found;         // items over the threshold (ordered mode)
  uint32_t max_bits;      // running max |x| of the segment as float bits (reset by plan)
  uint32_t max_saved;     // max |x| of the current select
  uint32_t tau_bits;      // threshold the current select was counted with
  uint32_t reserved[2];
};

struct Chunk {            // unit of work of the streaming passes; never spans two segments
  uint32_t seg;
  uint32_t start;         // bucket offset, multiple of 16
  uint32_t len;           // elements, multiple of 16
  uint32_t reserved;
};

// Hyper-parameters and counters of the sparse optimisers, resident on the device so that a step
// captured in a CUDA graph sees later changes (learning-rate schedules, step counters).
struct OptState {
  float lr, momentum, dampening, weight_decay;
  float beta1, beta2, eps, reserved0;
  uint32_t nesterov, maximize, amsgrad, smart_momentum;
  uint32_t tick;          // calls so far + 1 (Adam bias correction; reference optim/adam.cpp:30-43)
  uint32_t first;         // 1 until the first SGD call happened (reference optim/sgd.cpp:41-50)
  uint32_t kind;          // 0 = SGD, 1 = Adam
  uint32_t reserved1;
};

struct SelectArgs {
  float* grad;                 // flat gradients of the bucket (used when grad_tab is null)
  float* const* grad_tab;      // optional per-segment gradient pointers
  float* resid;                // error-feedback residual, flat
  const SegDesc* segs;
  SegState* state;
  SegWork* work;
  const Chunk* chunks;
  uint32_t* chunk_cnt;         // items over the threshold per chunk
  uint32_t* chunk_pos;         // exclusive prefix of chunk_cnt inside the segment
  uint64_t* chunk_state;       // one-pass select: per chunk (epoch | kind | items), see chunk_word(); or null
  uint32_t* hist;              // [n_segs][kHistBins]
  uint2* cand;                 // candidate scratch: (item id, key)
  uint32_t* cand_cursor;       // bump pointer into cand
  uint32_t cand_cap;
  uint32_t n_segs, n_chunks, n_total;
  uint32_t compressor;         // Compressor
  uint32_t zero_grad;          // write zeros over consumed gradients
  uint32_t skip_ef;            // 1: the residual already holds g + r (re-selection), skip the add
  // exchange
  int32_t world, rank;
  uint2* out[kMaxWorld];       // per destination: its receive area for source `rank`, slot 0
  uint2* out_mc;               // multicast alias of the same area (NVLS), or null
  uint64_t slot_stride;        // entries between slot 0 and slot 1 of a receive area
  uint64_t* flag[kMaxWorld];   // per destination: its arrival flag for source `rank`, slot 0
  uint64_t flag_slot_stride;   // u64 words between the flags of slot 0 and slot 1
  const uint64_t* ack_local;   // [2][world] acknowledgements written by the destinations
  uint32_t use_acks;           // wait for acknowledgements before overwriting a slot
  uint32_t publish;            // publish arrival flags when the stream is complete
  uint32_t owner_mode;         // 1: a segment's entries go only to the rank named in its descriptor
  // Debug checks (null = off): every emitted entry adds a hash of (index, value bits) to cksum_acc[dest]
  // (cksum_acc[0] when the entry goes to everyone); the last kernel of the chain stores the sums into the
  // destinations' checksum words before it publishes the arrival flags.
  uint32_t* cksum_acc;         // [kMaxWorld], device memory of this rank
  uint32_t* cksum[kMaxWorld];  // per destination: its checksum word for source `rank`, slot 0 ([2][world] u32)
  uint64_t cksum_slot_stride;
  uint32_t* epoch;             // select epoch of this bucket (starts at 1)
  uint32_t* done_ctr;          // CTA completion counter of the last kernel of the chain
  uint32_t* status;            // Status
  uint64_t timeout_ns;
  // Device clock (globaltimer, ns) of the latest chain, or null: [0] select start, [1] select end (stream
  // complete, flags published), [2] apply start (first stream seen), [3] apply end, [4] epoch of the
  // select, [5] epoch of the apply.  Feeds the telemetry (push duration, exposed wait).
  uint64_t* stamps;
};

struct ApplyArgs {
  uint2* recv;                 // [2 slots][world][cap] received streams (local memory)
  uint64_t slot_stride;        // entries per slot (= world * cap)
  uint32_t cap;                // entries per source
  uint32_t n_total;            // elements in the bucket
  int32_t world, rank;
  const uint64_t* flag_local;  // [2][world] arrival flags written by the sources
  uint64_t* ack[kMaxWorld];    // per source: its acknowledgement word for consumer `rank`, slot 0
  uint64_t ack_slot_stride;
  uint32_t use_flags;          // wait on arrival flags (0 when a library collective filled recv)
  uint32_t use_acks;
  const float* weight;         // [2][world] weight of each source in the merge (default 1/world), row = epoch & 1:
                               // two rows let the host switch weights at a named iteration without draining the
                               // pipeline (the row of an epoch is rewritten between the applies of epochs e - 2 and e)
  // One 16-byte record per element of the state range: {x: dense accumulator, zero outside a scatter/apply
  // pair; y: bits of the last epoch at which the element was updated; z: momentum buffer (SGD) or first
  // moment (Adam); w: second moment (Adam)}.  Interleaved so that an update touches one 32-byte sector of
  // state instead of four: entries hit random elements and the apply kernel is bound by DRAM transactions.
  float4* rec;
  float* param;
  float* vmax;                 // AMSGrad maximum, or null
  uint32_t* last;              // smart momentum: step of the last touch, or null
  OptState* opt;
  uint32_t* epoch;             // apply epoch of this bucket (starts at 1)
  const uint32_t* sel_epoch;   // select epoch: an apply with epoch >= *sel_epoch has nothing to consume
  uint32_t* done_ctr;
  uint32_t* status;
  uint64_t timeout_ns;
  // Range of stream positions this rank consumes, and the element range its accumulator, stamps and
  // optimiser state cover (acc, stamp, m, v, vmax, last are indexed by idx - state_base).  Replicated
  // state: [0, cap) and [0, n_total).
  uint32_t ent_lo, ent_hi;
  uint32_t state_base, state_len;
  // Partitioned state ("owner mode"): the owner of a tensor applies the update and stores, for every
  // stream position it consumed, either (idx, new parameter value) or the "no entry" marker into the
  // same position of every rank's write-back area; each rank then copies the values into its replica.
  uint32_t owner_mode;
  // Segment table, needed only when some tensors use the narrow wire format (narrow != 0): the receiver
  // finds the tensor of a stream position by binary search over out_off.
  uint32_t narrow;
  uint32_t n_segs;
  const SegDesc* segs;
  // Debug checks (null = off): the scatter adds the same hash over what it reads into rsum[source], the apply
  // compares it with the word the source stored and reports kBadChecksum; with `poison` every consumed entry
  // of a wide stream is overwritten with the "no entry" marker, so a position a source fails to rewrite
  // can never be taken for fresh data.
  // Deterministic merge: the scatter runs once per source, in rank order, so that every replica adds an
  // element's contributions in the same order and replicas stay bit-equal (three or more contributions to
  // one element otherwise round differently from GPU to GPU).  src_first is the source of the current launch.
  uint32_t deterministic;
  uint32_t src_first;
  uint64_t* stamps;                 // see SelectArgs::stamps
  const uint32_t* cksum_local;      // [2][world] written by the sources
  uint32_t* rsum;                   // [world]
  uint32_t poison;
  uint32_t own_lo[kMaxWorld + 1];   // owner o consumes positions [own_lo[o], own_lo[o + 1])
  uint2* wb[kMaxWorld];             // per rank: its write-back area [2][world][cap], slot 0
  uint2* wb_mc;                     // multicast alias of the write-back area, or null
  const uint2* wb_local;            // this rank's write-back area
  uint64_t* pflag[kMaxWorld];       // per rank: its "parameters of owner `rank` have landed" word, slot 0
  const uint64_t* pflag_local;      // [2][world] written by the owners
  uint64_t pflag_slot_stride;
};

// Token bucket of an emulated slow link, resident on the device (k_shape).  The host fills in burst, period and
// the schedule once and zeroes the rest; it reads sent_bytes, waited_ns and the clock origin back for telemetry.
constexpr int kShaperLevels = 64;
struct ShaperState {
  double tokens;            // bytes that may go out without waiting; negative: debt being repaid
  uint64_t last_ns;         // device clock of the last refill, 0 before the first use
  uint64_t t0_ns;           // device clock of the first use: origin of the schedule
  uint64_t sent_bytes;
  uint64_t waited_ns;
  float burst_bytes;
  float period_s;           // duration of one level of the schedule
  uint32_t levels;          // levels in use, <= kShaperLevels
  uint32_t reserved;
  float rate[kShaperLevels];   // bytes per second
};

// Intra-group dense reduction (grouped topologies).
struct GroupArgs {
  float* grad_local;                     // this rank's flat gradients of the bucket (symmetric memory)
  const float* grad_peer[kMaxWorld];     // group-mates' flat gradients, same layout
  int32_t n_mates;
  int32_t mate_slot[kMaxWorld];          // index of mate m in the [group size] flag arrays
  const SegDesc* segs;
  const Chunk* chunks;
  uint32_t n_chunks;
  uint64_t* ready_peer[kMaxWorld];       // mate m's ready word for this rank
  const uint64_t* ready_local;           // [group size] ready words written by the mates
  uint64_t* done_peer[kMaxWorld];
  const uint64_t* done_local;
  const uint32_t* epoch;                 // the bucket's select epoch
  uint32_t* done_ctr;
  uint32_t* status;
  uint64_t timeout_ns;
};

}  // namespace st
