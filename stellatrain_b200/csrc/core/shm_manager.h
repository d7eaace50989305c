// Per-node POSIX shared-memory pool of the CPU tier.
//
// Role of the reference's ShmManager (backend/src/engine/shm_manager.cpp:17-99, 113-187, 190-215,
// 270-381): the node master creates a metadata segment and a data segment named after the session id,
// the other local processes attach, tensors are exchanged between processes as offsets, allocation is
// a bump pointer that never frees, and the data segment can be pinned for CUDA in every process.
// Differences: the node barrier and the counting barriers used by tasks can time out (a dead local
// process becomes an error, not a hang), stale segments of a crashed run with the same session id are
// replaced, and CUDA is reached through dlopen so that the tier also runs on machines without a GPU.
#pragma once
#include <pthread.h>

#include <cstddef>
#include <cstdint>
#include <string>

namespace stc {

struct ShmHeader;   // lives at the start of the metadata segment

class ShmManager {
 public:
  ShmManager(bool master, int64_t session, int local_rank, int local_world, size_t data_bytes, size_t meta_bytes,
             int attach_timeout_ms);
  ~ShmManager();
  ShmManager(const ShmManager&) = delete;

  void* alloc(size_t bytes, size_t align = 64);        // from the data segment; throws bad_alloc when full
  void* alloc_meta(size_t bytes, size_t align = 64);   // from the metadata segment
  void* meta_first() const;                            // address of the first alloc_meta() result, same in every process
  uint64_t offset_of(const void* p) const;
  void* from_offset(uint64_t off) const;
  size_t data_used() const;
  size_t data_bytes() const { return data_bytes_; }

  // All local processes rendezvous; false when the others did not arrive in time.
  bool barrier(int timeout_ms);

  // Counting barrier identified by a 64-bit key (hash of task key and stage).
  //   arrive() registers this process; returns true when it was the last of `parties`.
  //   complete() tells whether all parties have arrived (non-blocking).
  //   depart() releases this process's reference; the last one frees the slot.
  bool arrive(uint64_t key, int parties);
  bool complete(uint64_t key);
  void depart(uint64_t key, int parties);
  // Blocks until some barrier state changed or the time is up (used by the polling manager thread).
  void wait_change(int timeout_ms);

  // cudaHostRegister / cudaHostUnregister of the data segment through a dlopen'ed CUDA runtime.
  bool pin_for_cuda();

  bool master() const { return master_; }
  int local_rank() const { return local_rank_; }
  int local_world() const { return local_world_; }
  static std::string meta_name(int64_t session);
  static std::string data_name(int64_t session);
  static void unlink_session(int64_t session);

 private:
  struct BarrierSlot;
  BarrierSlot* find_slot(uint64_t key, bool create);
  bool master_;
  int64_t session_;
  int local_rank_, local_world_;
  size_t data_bytes_, meta_bytes_;
  ShmHeader* hdr_ = nullptr;
  unsigned char* meta_ = nullptr;
  unsigned char* data_ = nullptr;
  bool pinned_ = false;
  void* cudart_ = nullptr;      // runtime library that registered the data segment
};

}  // namespace stc
