#include "shm_manager.h"

#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstring>
#include <new>
#include <stdexcept>
#include <thread>

#include "logger.h"

namespace stc {

namespace {
constexpr uint64_t kMagic = 0x5354423230305348ull;   // "STB200SH"
constexpr int kBarrierSlots = 8192;

timespec deadline_after(int ms) {
  timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  ts.tv_sec += ms / 1000;
  ts.tv_nsec += static_cast<long>(ms % 1000) * 1000000L;
  if (ts.tv_nsec >= 1000000000L) { ts.tv_sec += 1; ts.tv_nsec -= 1000000000L; }
  return ts;
}
}  // namespace

struct ShmManager::BarrierSlot {
  uint64_t key;       // 0 = free
  uint32_t arrived;
  uint32_t departed;
};

struct ShmHeader {
  uint64_t magic;
  uint64_t data_bytes, meta_bytes;
  pthread_mutex_t mu;          // process-shared, robust
  pthread_cond_t cv;           // process-shared
  uint64_t data_cursor, meta_cursor;
  uint32_t node_arrived, node_generation;
  uint32_t ready;              // set by the master when the header is initialised
};

static size_t header_bytes() {
  return (sizeof(ShmHeader) + 4095) / 4096 * 4096;
}

std::string ShmManager::meta_name(int64_t s) { return "/stb200-shm-meta-" + std::to_string(s); }
std::string ShmManager::data_name(int64_t s) { return "/stb200-shm-data-" + std::to_string(s); }

void ShmManager::unlink_session(int64_t s) {
  shm_unlink(meta_name(s).c_str());
  shm_unlink(data_name(s).c_str());
}

static unsigned char* map_segment(const std::string& name, size_t bytes, bool create, int timeout_ms) {
  int fd = -1;
  if (create) {
    shm_unlink(name.c_str());   // a crashed run with the same session may have left one behind
    fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) throw std::runtime_error("shm_open(create " + name + "): " + std::strerror(errno));
    if (ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
      close(fd);
      throw std::runtime_error("ftruncate(" + name + "): " + std::strerror(errno));
    }
  } else {
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      fd = shm_open(name.c_str(), O_RDWR, 0600);
      if (fd >= 0) {
        struct stat st;
        if (fstat(fd, &st) == 0 && static_cast<size_t>(st.st_size) >= bytes) break;
        close(fd);
        fd = -1;
      }
      if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms))
        throw std::runtime_error("timed out attaching to " + name + " (is the node master running?)");
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) throw std::runtime_error("mmap(" + name + "): " + std::strerror(errno));
  return static_cast<unsigned char*>(p);
}

ShmManager::ShmManager(bool master, int64_t session, int local_rank, int local_world, size_t data_bytes,
                       size_t meta_bytes, int attach_timeout_ms)
    : master_(master), session_(session), local_rank_(local_rank), local_world_(local_world),
      data_bytes_(data_bytes), meta_bytes_(meta_bytes) {
  const size_t slots_bytes = sizeof(BarrierSlot) * kBarrierSlots;
  if (meta_bytes_ < header_bytes() + slots_bytes + 4096) throw std::invalid_argument("metadata segment too small");
  meta_ = map_segment(meta_name(session), meta_bytes_, master, attach_timeout_ms);
  hdr_ = reinterpret_cast<ShmHeader*>(meta_);
  if (master) {
    std::memset(meta_, 0, header_bytes() + slots_bytes);
    pthread_mutexattr_t ma;
    pthread_mutexattr_init(&ma);
    pthread_mutexattr_setpshared(&ma, PTHREAD_PROCESS_SHARED);
    pthread_mutexattr_setrobust(&ma, PTHREAD_MUTEX_ROBUST);
    pthread_mutex_init(&hdr_->mu, &ma);
    pthread_mutexattr_destroy(&ma);
    pthread_condattr_t ca;
    pthread_condattr_init(&ca);
    pthread_condattr_setpshared(&ca, PTHREAD_PROCESS_SHARED);
    pthread_cond_init(&hdr_->cv, &ca);
    pthread_condattr_destroy(&ca);
    hdr_->data_bytes = data_bytes_;
    hdr_->meta_bytes = meta_bytes_;
    hdr_->data_cursor = 0;
    hdr_->meta_cursor = header_bytes() + slots_bytes;
    hdr_->magic = kMagic;
    data_ = map_segment(data_name(session), data_bytes_, true, attach_timeout_ms);
    __atomic_store_n(&hdr_->ready, 1u, __ATOMIC_RELEASE);
  } else {
    const auto t0 = std::chrono::steady_clock::now();
    while (__atomic_load_n(&hdr_->ready, __ATOMIC_ACQUIRE) != 1u || hdr_->magic != kMagic) {
      if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(attach_timeout_ms))
        throw std::runtime_error("shared-memory header was never initialised by the node master");
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    if (hdr_->data_bytes != data_bytes_ || hdr_->meta_bytes != meta_bytes_)
      throw std::runtime_error("shared-memory sizes differ between local processes");
    data_ = map_segment(data_name(session), data_bytes_, false, attach_timeout_ms);
  }
}

ShmManager::~ShmManager() {
  if (pinned_) {
    using Fn = int (*)(void*);
    if (auto fn = cudart_ ? reinterpret_cast<Fn>(dlsym(cudart_, "cudaHostUnregister")) : nullptr) fn(data_);
  }
  if (data_) munmap(data_, data_bytes_);
  if (meta_) munmap(meta_, meta_bytes_);
  if (master_) unlink_session(session_);
}

static void lock_robust(pthread_mutex_t* mu) {
  const int rc = pthread_mutex_lock(mu);
  if (rc == EOWNERDEAD) pthread_mutex_consistent(mu);   // a local process died holding it
}

void* ShmManager::alloc(size_t bytes, size_t align) {
  lock_robust(&hdr_->mu);
  const uint64_t off = (hdr_->data_cursor + align - 1) / align * align;
  if (off + bytes > data_bytes_) {
    pthread_mutex_unlock(&hdr_->mu);
    throw std::bad_alloc();
  }
  hdr_->data_cursor = off + bytes;
  pthread_mutex_unlock(&hdr_->mu);
  return data_ + off;
}

void* ShmManager::alloc_meta(size_t bytes, size_t align) {
  lock_robust(&hdr_->mu);
  const uint64_t off = (hdr_->meta_cursor + align - 1) / align * align;
  if (off + bytes > meta_bytes_) {
    pthread_mutex_unlock(&hdr_->mu);
    throw std::bad_alloc();
  }
  hdr_->meta_cursor = off + bytes;
  pthread_mutex_unlock(&hdr_->mu);
  return meta_ + off;
}

void* ShmManager::meta_first() const {
  const size_t off = header_bytes() + sizeof(BarrierSlot) * kBarrierSlots;
  return meta_ + (off + 63) / 64 * 64;
}

uint64_t ShmManager::offset_of(const void* p) const {
  const auto* c = static_cast<const unsigned char*>(p);
  if (c < data_ || c >= data_ + data_bytes_) throw std::out_of_range("pointer is not inside the shared data segment");
  return static_cast<uint64_t>(c - data_);
}

void* ShmManager::from_offset(uint64_t off) const {
  if (off >= data_bytes_) throw std::out_of_range("offset beyond the shared data segment");
  return data_ + off;
}

size_t ShmManager::data_used() const { return hdr_->data_cursor; }

bool ShmManager::barrier(int timeout_ms) {
  const timespec dl = deadline_after(timeout_ms);
  lock_robust(&hdr_->mu);
  const uint32_t gen = hdr_->node_generation;
  if (++hdr_->node_arrived == static_cast<uint32_t>(local_world_)) {
    hdr_->node_arrived = 0;
    ++hdr_->node_generation;
    pthread_cond_broadcast(&hdr_->cv);
    pthread_mutex_unlock(&hdr_->mu);
    return true;
  }
  while (hdr_->node_generation == gen) {
    const int rc = pthread_cond_timedwait(&hdr_->cv, &hdr_->mu, &dl);
    if (rc == EOWNERDEAD) pthread_mutex_consistent(&hdr_->mu);
    if (rc == ETIMEDOUT && hdr_->node_generation == gen) {
      --hdr_->node_arrived;   // withdraw, so that a later attempt starts clean
      pthread_mutex_unlock(&hdr_->mu);
      return false;
    }
  }
  pthread_mutex_unlock(&hdr_->mu);
  return true;
}

ShmManager::BarrierSlot* ShmManager::find_slot(uint64_t key, bool create) {
  auto* slots = reinterpret_cast<BarrierSlot*>(meta_ + header_bytes());
  if (key == 0) key = 1;
  size_t h = static_cast<size_t>(key * 0x9E3779B97F4A7C15ull >> 40) % kBarrierSlots;
  BarrierSlot* free_slot = nullptr;
  for (int probe = 0; probe < kBarrierSlots; ++probe) {
    BarrierSlot* s = &slots[(h + probe) % kBarrierSlots];
    if (s->key == key) return s;
    if (s->key == 0) {
      if (!free_slot) free_slot = s;
      break;   // keys are never moved, so the first hole ends the probe sequence
    }
  }
  if (!create) return nullptr;
  if (!free_slot) throw std::runtime_error("barrier table full");
  free_slot->key = key;
  free_slot->arrived = free_slot->departed = 0;
  return free_slot;
}

bool ShmManager::arrive(uint64_t key, int parties) {
  lock_robust(&hdr_->mu);
  BarrierSlot* s = find_slot(key, true);
  const bool last = ++s->arrived == static_cast<uint32_t>(parties);
  if (last) pthread_cond_broadcast(&hdr_->cv);
  pthread_mutex_unlock(&hdr_->mu);
  return last;
}

bool ShmManager::complete(uint64_t key) {
  lock_robust(&hdr_->mu);
  BarrierSlot* s = find_slot(key, false);
  // a slot that is gone was completed and released by everybody else already
  const bool done = s == nullptr || s->arrived >= static_cast<uint32_t>(local_world_);
  pthread_mutex_unlock(&hdr_->mu);
  return done;
}

void ShmManager::depart(uint64_t key, int parties) {
  lock_robust(&hdr_->mu);
  BarrierSlot* s = find_slot(key, false);
  if (s && ++s->departed == static_cast<uint32_t>(parties)) {
    // tombstone-free removal is only safe when the next slot is empty; otherwise keep a
    // reusable marker by zeroing counts and leaving the key (it is never reused: keys carry
    // the iteration number)
    auto* slots = reinterpret_cast<BarrierSlot*>(meta_ + header_bytes());
    const size_t i = static_cast<size_t>(s - slots);
    if (slots[(i + 1) % kBarrierSlots].key == 0) s->key = 0;
    else { s->key = ~0ull - i; s->arrived = s->departed = 0; }
  }
  pthread_mutex_unlock(&hdr_->mu);
}

void ShmManager::wait_change(int timeout_ms) {
  const timespec dl = deadline_after(timeout_ms);
  lock_robust(&hdr_->mu);
  const int rc = pthread_cond_timedwait(&hdr_->cv, &hdr_->mu, &dl);
  if (rc == EOWNERDEAD) pthread_mutex_consistent(&hdr_->mu);
  pthread_mutex_unlock(&hdr_->mu);
}

bool ShmManager::pin_for_cuda() {
  if (pinned_) return true;
  void* lib = dlopen("libcudart.so.12", RTLD_NOW | RTLD_NOLOAD);   // the copy the framework already uses
  if (!lib) lib = dlopen("libcudart.so.12", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libcudart.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return false;
  using Fn = int (*)(void*, size_t, unsigned int);
  auto fn = reinterpret_cast<Fn>(dlsym(lib, "cudaHostRegister"));
  if (!fn) return false;
  const int rc = fn(data_, data_bytes_, 0x02 /* cudaHostRegisterMapped */);
  pinned_ = rc == 0;
  if (pinned_) cudart_ = lib;
  if (!pinned_) LOG_WARN("ShmManager", "cudaHostRegister failed with code " << rc << "; copies will be pageable");
  return pinned_;
}

}  // namespace stc
