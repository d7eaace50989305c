// Gradient sparsifiers of the CPU tier.
//
// Interface after the reference's Compressor (backend/src/compress/compressor.h:12-33): one call
// compresses one tensor into at most k (index, value) pairs.  Semantics are the ones the GPU kernels
// and the PyTorch oracle implement (stellatrain_b200/ops/oracle.py), so the three tiers can be
// compared entry for entry:
//   top-k          k largest |x|, equal magnitudes towards the lower index (backend/src/compress/topk.cpp
//                  is the intent; the shipped code returns positions of a partitioned copy)
//   threshold-v    all |x| >= tau in index order, at most k; tau adapts AIMD per tensor
//                  (backend/src/compress/thresholdv.cpp:40-83)
//   threshold-v16  aligned 16-element blocks by L1 norm against tau, filled up from the best rejected
//                  blocks when short (backend/src/compress/thresholdv16.cpp:78-295)
//   random-k       k distinct uniformly random positions (backend/src/compress/randomk.cpp:125-164,
//                  dead code in the reference)
// Output is in ascending index order except for the fill-up part of threshold-v16 and random-k.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace stc {

class ThreadPool;

struct ThresholdState {
  float tau = 0.f;
  float tau_inc = 0.f;
  bool inited = false;
};

class Compressor {
 public:
  Compressor(ThreadPool* pool, std::string name) : pool_(pool), name_(std::move(name)) {}
  virtual ~Compressor() = default;
  const std::string& name() const { return name_; }

  // Returns the number of pairs written (<= k).  Indices are offsets into src plus idx_offset.
  virtual size_t compress(const std::string& tensor, const float* src, size_t n, uint32_t k, uint32_t* dst_idx,
                          float* dst_val, int32_t idx_offset = 0) = 0;

  // Per-tensor thresholds, for checkpoints.
  std::map<std::string, ThresholdState> export_state();
  void import_state(const std::map<std::string, ThresholdState>& st);

 protected:
  ThresholdState load_state(const std::string& tensor);
  void store_state(const std::string& tensor, const ThresholdState& st);
  ThreadPool* pool_;
  std::string name_;

 private:
  std::mutex mu_;
  std::map<std::string, ThresholdState> state_;
};

class TopkCompressor : public Compressor {
 public:
  explicit TopkCompressor(ThreadPool* pool) : Compressor(pool, "topk") {}
  size_t compress(const std::string& tensor, const float* src, size_t n, uint32_t k, uint32_t* dst_idx, float* dst_val,
                  int32_t idx_offset = 0) override;
};

class ThresholdvCompressor : public Compressor {
 public:
  explicit ThresholdvCompressor(ThreadPool* pool) : Compressor(pool, "thresholdv") {}
  size_t compress(const std::string& tensor, const float* src, size_t n, uint32_t k, uint32_t* dst_idx, float* dst_val,
                  int32_t idx_offset = 0) override;
};

class Thresholdv16Compressor : public Compressor {
 public:
  explicit Thresholdv16Compressor(ThreadPool* pool) : Compressor(pool, "thresholdv16") {}
  size_t compress(const std::string& tensor, const float* src, size_t n, uint32_t k, uint32_t* dst_idx, float* dst_val,
                  int32_t idx_offset = 0) override;
};

class RandomkCompressor : public Compressor {
 public:
  explicit RandomkCompressor(ThreadPool* pool, uint64_t seed = 0x5DEECE66Dull) : Compressor(pool, "randomk"), seed_(seed) {}
  size_t compress(const std::string& tensor, const float* src, size_t n, uint32_t k, uint32_t* dst_idx, float* dst_val,
                  int32_t idx_offset = 0) override;

 private:
  uint64_t seed_;
  std::mutex mu_;
  std::map<std::string, uint64_t> calls_;
};

std::unique_ptr<Compressor> make_compressor(const std::string& method, ThreadPool* pool);

// Exact selection helper shared by the compressors: writes the positions (ascending) of the `k`
// largest keys, equal keys towards the lower position, and returns the k-th largest key.
uint32_t select_top_keys(const uint32_t* keys, size_t n, size_t k, ThreadPool* pool, std::vector<uint32_t>& out_pos);

// Error feedback around a compressor (backend/src/engine/modules/compress.cpp:139-188):
// acc[i] = grad[i] + resid[i] (NaN -> 0); compress acc; resid = acc with the sent entries zeroed.
size_t compress_with_feedback(Compressor& c, const std::string& tensor, const float* grad, float* resid, size_t n,
                              uint32_t k, uint32_t* dst_idx, float* dst_val, ThreadPool* pool);

}  // namespace stc
