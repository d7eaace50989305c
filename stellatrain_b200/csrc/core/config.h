// Compile-time defaults and limits of the CPU tier.  Values follow the reference's
// backend/src/engine/config.h:6-66 where a counterpart exists; everything that the reference fixes at
// compile time and a user may want to change is also readable from the environment at start-up.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdlib>

namespace stc {
namespace cfg {

constexpr int kWorkersNodeMaster = 32;       // reference config.h:7
constexpr int kWorkersOther = 16;            // reference config.h:8
constexpr size_t kShmMetaBytes = 64ull << 20;   // reference config.h:23
constexpr size_t kShmDataBytes = 4ull << 30;    // reference config.h:24 (one chunk; virtual until touched)
constexpr int kMaxLocalRanks = 8;            // reference MAX_NUM_GPU_PER_NODE
constexpr int kMaxTaskBarriers = 8;          // reference MAX_NUM_BARRIER
constexpr int kMaxNameLen = 63;              // reference task key limit (task.cpp:44-60)
constexpr int kMaxParams = 4096;             // shared parameter table entries
constexpr int kTaskSlots = 32768;            // reference NUM_MAX_CONCURRENT_TASKS
constexpr int kDefaultStaleness = 1;         // reference core.cpp:80
constexpr double kDefaultCompressionRatio = 0.99;   // reference core.cpp:23
constexpr int kBarrierPollMs = 100;          // reference core.cpp:464-484
constexpr int kDefaultTimeoutMs = 30000;     // every blocking wait of the tier gives up after this
constexpr uint16_t kDataPortLo = 10240, kDataPortHi = 49151;   // reference comm_manager.cpp:57-63

inline long env_long(const char* name, long dflt) {
  const char* v = std::getenv(name);
  return v ? std::strtol(v, nullptr, 10) : dflt;
}

}  // namespace cfg
}  // namespace stc
