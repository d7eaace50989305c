#include "comm_manager.h"

#include <cstdlib>

#include <poll.h>
#include <cstdio>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <stdexcept>

#include "../core/logger.h"
#include "../cpu/array_util.h"

namespace stc {

namespace {

constexpr uint32_t kMagic = 0x32425453u;   // "STB2"

enum MsgType : uint32_t {
  kInitReq = 1, kInitRes, kModelPut, kModelGet, kModelRep, kSyncTime, kStatRep, kBarrier, kOk, kConfigUpd, kGrad,
  kBye,
};

struct FrameHeader {
  uint32_t magic, type, key_len, flags;
  uint64_t payload_len;
};

struct InitReq {            // cf. reference MsgInitReq (backend/src/engine/message.h:10-25)
  uint16_t rank, listen_port, num_gpus, reserved;
  int64_t timestamp_ns;
  char ip[64];
};
struct InitRes {
  uint8_t success;
  uint8_t pad[3];
  uint16_t target_port, target_rank;
  char target_ip[64];
};

int64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

bool send_frame(int fd, uint32_t type, const std::string& key, uint32_t flags, const void* payload, size_t len,
                int timeout_ms) {
  FrameHeader h{kMagic, type, static_cast<uint32_t>(key.size()), flags, len};
  if (!send_all(fd, &h, sizeof(h), timeout_ms)) return false;
  if (!key.empty() && !send_all(fd, key.data(), key.size(), timeout_ms)) return false;
  if (len && !send_all(fd, payload, len, timeout_ms)) return false;
  return true;
}

bool recv_frame(int fd, FrameHeader* h, std::string* key, std::vector<unsigned char>* payload, int timeout_ms) {
  if (!recv_all(fd, h, sizeof(*h), timeout_ms)) return false;
  if (h->magic != kMagic || h->key_len > 4096 || h->payload_len > (1ull << 34)) return false;   // truncated or foreign
  key->resize(h->key_len);
  if (h->key_len && !recv_all(fd, &(*key)[0], h->key_len, timeout_ms)) return false;
  payload->resize(h->payload_len);
  if (h->payload_len && !recv_all(fd, payload->data(), h->payload_len, timeout_ms)) return false;
  return true;
}

}  // namespace

CommManager::CommManager(const std::string& master_addr, uint16_t master_port, int timeout_ms)
    : master_addr_(master_addr), master_port_(master_port), timeout_ms_(timeout_ms) {}

CommManager::~CommManager() {
  stop_ = true;
  tx_cv_.notify_all();
  if (control_fd_ >= 0) {
    std::lock_guard<std::mutex> lk(control_mu_);
    send_frame(control_fd_, kBye, "", 0, nullptr, 0, 200);
  }
  if (push_thread_.joinable()) push_thread_.join();
  // tell the ring successor that the silence that follows is a regular shutdown, not a lost node
  if (push_fd_ >= 0 && !failed_) send_frame(push_fd_, kBye, "", 0, nullptr, 0, 200);
  if (pull_thread_.joinable()) pull_thread_.join();
  if (zmq_) zmq_->close();     // both threads are gone: no socket is in use any more
  close_fd(push_fd_);
  close_fd(pull_fd_);
  close_fd(data_listen_fd_);
  close_fd(control_fd_);
  if (broker_thread_.joinable()) broker_thread_.join();
  close_fd(broker_listen_fd_);
}

void CommManager::set_failed(const std::string& why) {
  std::lock_guard<std::mutex> lk(fail_mu_);
  if (!failed_) {
    failure_ = why;
    failed_ = true;
    LOG_ERROR("CommManager", why);
  }
}

std::string CommManager::failure() const {
  std::lock_guard<std::mutex> lk(fail_mu_);
  return failure_;
}

// ---------------------------------------------------------------- broker (rank 0)
void CommManager::start_server(int world) {
  uint16_t bound = 0;
  broker_listen_fd_ = tcp_listen(master_port_, &bound);
  if (broker_listen_fd_ < 0) throw std::runtime_error("broker cannot listen on port " + std::to_string(master_port_));
  broker_thread_ = std::thread([this, world] { broker_main(world); });
}

void CommManager::broker_main(int world) {
  pthread_setname_np(pthread_self(), "CommBroker");
  struct Client {
    int fd = -1;
    InitReq req{};
    bool registered = false;
  };
  std::vector<Client> clients;
  std::map<std::string, std::vector<unsigned char>> models;             // key -> parameter bytes
  std::map<std::string, std::vector<int>> model_waiters;                // key -> client slots waiting
  std::vector<int> barrier_waiters;
  int registered = 0;
  bool ring_sent = false;

  while (!stop_) {
    std::vector<pollfd> pfds;
    pfds.push_back({broker_listen_fd_, POLLIN, 0});
    for (auto& c : clients) pfds.push_back({c.fd, static_cast<short>(c.fd >= 0 ? POLLIN : 0), 0});
    const int rc = poll(pfds.data(), pfds.size(), 100);
    if (rc <= 0) continue;
    if (pfds[0].revents & POLLIN) {
      const int fd = tcp_accept(broker_listen_fd_, 0);
      if (fd >= 0) {
        Client c;
        c.fd = fd;
        clients.push_back(c);
      }
    }
    for (size_t ci = 0; ci + 1 < pfds.size() && ci < clients.size(); ++ci) {
      if (!(pfds[ci + 1].revents & (POLLIN | POLLHUP | POLLERR))) continue;
      Client& c = clients[ci];
      if (c.fd < 0) continue;
      FrameHeader h;
      std::string key;
      std::vector<unsigned char> payload;
      if (!recv_frame(c.fd, &h, &key, &payload, timeout_ms_)) {
        close_fd(c.fd);   // a node that disappears is simply dropped; its peers time out on data
        continue;
      }
      switch (h.type) {
        case kInitReq: {
          if (payload.size() == sizeof(InitReq)) {
            std::memcpy(&c.req, payload.data(), sizeof(InitReq));
            c.registered = true;
            ++registered;
          }
          break;
        }
        case kModelPut: {
          models[key] = std::move(payload);
          send_frame(c.fd, kOk, key, 0, nullptr, 0, timeout_ms_);
          auto it = model_waiters.find(key);
          if (it != model_waiters.end()) {
            for (int w : it->second)
              if (clients[w].fd >= 0)
                send_frame(clients[w].fd, kModelRep, key, 0, models[key].data(), models[key].size(), timeout_ms_);
            model_waiters.erase(it);
          }
          break;
        }
        case kModelGet: {
          auto it = models.find(key);
          if (it != models.end()) send_frame(c.fd, kModelRep, key, 0, it->second.data(), it->second.size(), timeout_ms_);
          else model_waiters[key].push_back(static_cast<int>(ci));
          break;
        }
        case kSyncTime: {
          const int64_t t = now_ns();
          send_frame(c.fd, kSyncTime, "", 0, &t, sizeof(t), timeout_ms_);
          break;
        }
        case kStatRep: {
          if (payload.size() == sizeof(PeerStat)) {
            PeerStat s;
            std::memcpy(&s, payload.data(), sizeof(s));
            std::lock_guard<std::mutex> lk(stats_mu_);
            stats_[s.rank] = s;
          }
          send_frame(c.fd, kOk, "", 0, nullptr, 0, timeout_ms_);
          break;
        }
        case kBarrier: {
          barrier_waiters.push_back(static_cast<int>(ci));
          if (static_cast<int>(barrier_waiters.size()) == world) {
            for (int w : barrier_waiters)
              if (clients[w].fd >= 0) send_frame(clients[w].fd, kOk, "", 0, nullptr, 0, timeout_ms_);
            barrier_waiters.clear();
          }
          break;
        }
        case kConfigUpd:   // placeholder in the reference too (comm_manager.cpp:312-328)
          send_frame(c.fd, kOk, "", 0, nullptr, 0, timeout_ms_);
          break;
        case kBye:
          close_fd(c.fd);
          break;
        default:
          break;
      }
    }
    if (!ring_sent && registered == world) {
      // ring in rank order: the successor of rank r is rank (r + 1) mod world
      std::map<int, Client*> by_rank;
      for (auto& c : clients)
        if (c.registered) by_rank[c.req.rank] = &c;
      if (static_cast<int>(by_rank.size()) == world) {
        for (auto& kv : by_rank) {
          Client* succ = by_rank[(kv.first + 1) % world];
          InitRes res{};
          res.success = 1;
          res.target_port = succ->req.listen_port;
          res.target_rank = succ->req.rank;
          std::snprintf(res.target_ip, sizeof(res.target_ip), "%s", succ->req.ip);   // always terminated
          send_frame(kv.second->fd, kInitRes, "", 0, &res, sizeof(res), timeout_ms_);
        }
        ring_sent = true;
      }
    }
  }
  for (auto& c : clients) close_fd(c.fd);
}

// ---------------------------------------------------------------- client
bool CommManager::set_data_transport(const std::string& name, const std::string& libzmq_hint) {
  if (name == "tcp") {
    zmq_.reset();
    return true;
  }
  if (name != "zmq") return false;
  std::string why;
  if (!ZmqLibrary::load(libzmq_hint, &why)) {
    LOG_WARN("CommManager", why);
    return false;
  }
  zmq_ = std::make_unique<ZmqLink>();
  return true;
}

bool CommManager::start_client(int rank, int world, int num_gpus) {
  rank_ = rank;
  world_ = world;
  if (!zmq_) {
    const char* env = std::getenv("STELLATRAIN_DATA_TRANSPORT");
    if (env != nullptr && std::string(env) == "zmq" && !set_data_transport("zmq")) {
      set_failed("STELLATRAIN_DATA_TRANSPORT=zmq, but no ZeroMQ library could be loaded (STELLATRAIN_LIBZMQ names one)");
      return false;
    }
  }
  control_fd_ = tcp_connect(master_addr_, master_port_, timeout_ms_);
  if (control_fd_ < 0) { set_failed("cannot reach the broker at " + master_addr_); return false; }
  const std::string my_ip = master_addr_ == "127.0.0.1" || master_addr_ == "localhost" ? "127.0.0.1" : pick_local_ip();
  uint16_t port = 0;
  if (zmq_) {
    port = zmq_->bind_pull(my_ip == "127.0.0.1" ? my_ip : "*");
    if (port == 0) { set_failed("cannot bind a ZeroMQ PULL socket"); return false; }
  } else {
    data_listen_fd_ = tcp_listen(0, &port, true);
    if (data_listen_fd_ < 0) { set_failed("cannot open a data port"); return false; }
  }
  InitReq req{};
  req.rank = static_cast<uint16_t>(rank);
  req.listen_port = port;
  req.num_gpus = static_cast<uint16_t>(num_gpus);
  req.timestamp_ns = now_ns();
  std::strncpy(req.ip, my_ip.c_str(), sizeof(req.ip) - 1);
  FrameHeader h;
  std::string key;
  std::vector<unsigned char> payload;
  {
    std::lock_guard<std::mutex> lk(control_mu_);
    if (!send_frame(control_fd_, kInitReq, "", 0, &req, sizeof(req), timeout_ms_) ||
        !recv_frame(control_fd_, &h, &key, &payload, timeout_ms_) || h.type != kInitRes ||
        payload.size() != sizeof(InitRes)) {
      set_failed("rendezvous with the broker failed (are all " + std::to_string(world) + " nodes up?)");
      return false;
    }
  }
  InitRes res;
  std::memcpy(&res, payload.data(), sizeof(res));
  if (zmq_) {
    if (!zmq_->connect_push(res.target_ip, res.target_port)) { set_failed("cannot connect the ZeroMQ PUSH socket"); return false; }
  } else {
    push_fd_ = tcp_connect(res.target_ip, res.target_port, timeout_ms_);
    pull_fd_ = tcp_accept(data_listen_fd_, timeout_ms_);
    if (push_fd_ < 0 || pull_fd_ < 0) { set_failed("cannot establish the data ring"); return false; }
  }
  LOG_INFO("CommManager", "rank " << rank << " -> rank " << res.target_rank << " at " << res.target_ip << ":" << res.target_port);
  push_thread_ = std::thread([this] { push_main(); });
  pull_thread_ = std::thread([this] { pull_main(); });
  return true;
}

void CommManager::set_tx_fault_hook(std::function<bool(const std::string&, int*)> hook) {
  std::lock_guard<std::mutex> lk(tx_mu_);
  tx_hook_ = std::move(hook);
}

namespace {

void put_values(const float* val, size_t n, int value_format, unsigned char* out) {
  if (value_format == 1) f32_to_f16(val, reinterpret_cast<uint16_t*>(out), n);
  else if (value_format == 2) f32_to_bf16(val, reinterpret_cast<uint16_t*>(out), n);
  else std::memcpy(out, val, n * 4);
}

// true when idx[j .. j+15] is one aligned block: starts at a multiple of 16 and counts up by one
inline bool whole_block_at(const uint32_t* idx, size_t j, size_t count) {
  if (j + 16 > count || (idx[j] & 15u) != 0) return false;
  for (uint32_t d = 1; d < 16; ++d)
    if (idx[j + d] != idx[j] + d) return false;
  return true;
}

}  // namespace

EncodedSparse encode_sparse(const uint32_t* idx, const float* val, size_t count, uint32_t tensor_numel, bool allow_u16,
                            int value_format, bool allow_blocks) {
  EncodedSparse e;
  e.count = static_cast<uint32_t>(count);
  const size_t vsz = value_format == 0 ? 4 : 2;
  if (value_format == 1) e.flags |= kFlagValF16;
  else if (value_format == 2) e.flags |= kFlagValBF16;

  // pass over the indices: where the whole blocks are, and whether the rest fits 16 bits (reference:
  // tensor_numel < 65536, comm_manager.cpp:579-583; the sentinel index used for padding does not fit and
  // keeps the stream wide)
  std::vector<uint32_t> block_at;      // positions j of whole blocks
  bool narrow = allow_u16 && tensor_numel <= 65536;
  bool narrow_blocks = true;
  for (size_t j = 0; j < count;) {
    if (allow_blocks && whole_block_at(idx, j, count)) {
      block_at.push_back(static_cast<uint32_t>(j));
      narrow_blocks = narrow_blocks && (idx[j] >> 4) < 65536u;
      j += 16;
    } else {
      narrow = narrow && idx[j] < 65536u;
      ++j;
    }
  }
  const size_t nb = block_at.size();
  const size_t loose = count - 16 * nb;
  const size_t isz = narrow ? 2 : 4;
  if (narrow) e.flags |= kFlagIdxU16;

  if (nb == 0) {
    e.payload.resize(4 + count * isz + count * vsz);
    unsigned char* p = e.payload.data();
    std::memcpy(p, &e.count, 4);
    p += 4;
    if (narrow) narrow_u32_to_u16(idx, reinterpret_cast<uint16_t*>(p), count);
    else std::memcpy(p, idx, count * 4);
    put_values(val, count, value_format, p + count * isz);
    return e;
  }

  e.flags |= kFlagBlock16;
  if (narrow_blocks) e.flags |= kFlagBlockU16;
  const size_t bsz = narrow_blocks ? 2 : 4;
  e.payload.resize(8 + nb * bsz + loose * isz + count * vsz);
  unsigned char* p = e.payload.data();
  const uint32_t nb32 = static_cast<uint32_t>(nb);
  std::memcpy(p, &e.count, 4);
  std::memcpy(p + 4, &nb32, 4);
  unsigned char* pb = p + 8;
  unsigned char* pi = pb + nb * bsz;
  unsigned char* pv = pi + loose * isz;
  unsigned char* pvl = pv + 16 * nb * vsz;   // values of the loose entries follow those of the blocks
  std::vector<uint32_t> loose_idx;
  std::vector<float> loose_val;
  loose_idx.reserve(loose);
  loose_val.reserve(loose);
  size_t next_block = 0;
  for (size_t j = 0; j < count;) {
    if (next_block < nb && block_at[next_block] == j) {
      const uint32_t id = idx[j] >> 4;
      if (narrow_blocks) {
        const uint16_t id16 = static_cast<uint16_t>(id);
        std::memcpy(pb + next_block * 2, &id16, 2);
      } else {
        std::memcpy(pb + next_block * 4, &id, 4);
      }
      put_values(val + j, 16, value_format, pv + next_block * 16 * vsz);
      ++next_block;
      j += 16;
    } else {
      loose_idx.push_back(idx[j]);
      loose_val.push_back(val[j]);
      ++j;
    }
  }
  if (loose) {
    if (narrow) narrow_u32_to_u16(loose_idx.data(), reinterpret_cast<uint16_t*>(pi), loose);
    else std::memcpy(pi, loose_idx.data(), loose * 4);
    put_values(loose_val.data(), loose, value_format, pvl);
  }
  return e;
}

bool decode_sparse(uint8_t flags, const unsigned char* payload, size_t len, uint32_t tensor_numel,
                   std::vector<uint32_t>* idx, std::vector<float>* val) {
  if (len < 4) return false;
  uint32_t count;
  std::memcpy(&count, payload, 4);
  const size_t isz = (flags & kFlagIdxU16) ? 2 : 4;
  const size_t vsz = (flags & (kFlagValF16 | kFlagValBF16)) ? 2 : 4;
  uint32_t nb = 0;
  size_t head = 4, bsz = 0;
  if (flags & kFlagBlock16) {
    if (len < 8) return false;
    std::memcpy(&nb, payload + 4, 4);
    head = 8;
    bsz = (flags & kFlagBlockU16) ? 2 : 4;
    if (static_cast<uint64_t>(nb) * 16 > count) return false;
  }
  const size_t loose = count - static_cast<size_t>(nb) * 16;
  if (len != head + nb * bsz + loose * isz + static_cast<size_t>(count) * vsz) return false;
  idx->resize(count);
  val->resize(count);
  const unsigned char* pb = payload + head;
  const unsigned char* pi = pb + nb * bsz;
  const unsigned char* pv = pi + loose * isz;
  for (uint32_t b = 0; b < nb; ++b) {
    uint32_t id;
    if (bsz == 2) {
      uint16_t id16;
      std::memcpy(&id16, pb + b * 2, 2);
      id = id16;
    } else {
      std::memcpy(&id, pb + b * 4, 4);
      if (id > 0x0FFFFFFFu) return false;
    }
    for (uint32_t d = 0; d < 16; ++d) (*idx)[static_cast<size_t>(b) * 16 + d] = id * 16 + d;
  }
  uint32_t* li = idx->data() + static_cast<size_t>(nb) * 16;
  if (isz == 2) widen_u16_to_u32(reinterpret_cast<const uint16_t*>(pi), li, loose);
  else if (loose) std::memcpy(li, pi, loose * 4);
  if (flags & kFlagValF16) f16_to_f32(reinterpret_cast<const uint16_t*>(pv), val->data(), count);
  else if (flags & kFlagValBF16) bf16_to_f32(reinterpret_cast<const uint16_t*>(pv), val->data(), count);
  else if (count) std::memcpy(val->data(), pv, static_cast<size_t>(count) * 4);
  if (tensor_numel)
    for (uint32_t j = 0; j < count; ++j)
      if ((*idx)[j] >= tensor_numel && (*idx)[j] != 0xFFFFFFFFu) return false;   // the padding sentinel may travel
  return true;
}

void CommManager::queue_tx(int64_t priority, const std::string& key, const uint32_t* idx, const float* val, size_t count,
                           uint32_t tensor_numel, bool allow_u16, int value_format, bool allow_blocks) {
  auto item = std::make_shared<TxItem>();
  item->priority = priority;
  item->key = key;
  EncodedSparse enc = encode_sparse(idx, val, count, tensor_numel, allow_u16, value_format, allow_blocks);
  item->flags = enc.flags;
  item->payload = std::move(enc.payload);
  {
    std::lock_guard<std::mutex> lk(tx_mu_);
    item->seq = tx_seq_++;
    tx_queue_.push(std::move(item));
  }
  tx_cv_.notify_one();
}

void CommManager::set_tx_rate_limit(double bytes_per_s, size_t burst_bytes) {
  tx_burst_ = std::max<size_t>(burst_bytes, 1);
  tx_rate_ = bytes_per_s > 0 ? bytes_per_s : 0.0;
}

void CommManager::push_main() {
  pthread_setname_np(pthread_self(), "CommPushThread");
  while (!stop_) {
    std::shared_ptr<TxItem> item;
    std::function<bool(const std::string&, int*)> hook;
    {
      std::unique_lock<std::mutex> lk(tx_mu_);
      tx_cv_.wait_for(lk, std::chrono::milliseconds(100), [this] { return stop_ || !tx_queue_.empty(); });
      if (stop_) return;
      if (tx_queue_.empty()) continue;
      item = tx_queue_.top();
      tx_queue_.pop();
      hook = tx_hook_;
    }
    if (hook) {
      int delay = 0;
      if (hook(item->key, &delay)) continue;   // dropped on purpose by a test
      if (delay > 0) std::this_thread::sleep_for(std::chrono::milliseconds(delay));
    }
    const std::vector<unsigned char>& payload = item->payload;
    if (const double rate = tx_rate_.load()) {
      // token bucket: the message leaves when the bucket holds its bytes (or is as full as it gets)
      const double need = static_cast<double>(sizeof(FrameHeader) + item->key.size() + payload.size());
      const double burst = static_cast<double>(tx_burst_.load());
      const auto now = std::chrono::steady_clock::now();
      if (tx_last_.time_since_epoch().count() == 0) { tx_last_ = now; tx_tokens_ = burst; }
      tx_tokens_ = std::min(burst, tx_tokens_ + std::chrono::duration<double>(now - tx_last_).count() * rate);
      tx_last_ = now;
      if (tx_tokens_ < need) {
        const double wait_s = (need - tx_tokens_) / rate;
        const auto until = now + std::chrono::duration_cast<std::chrono::steady_clock::duration>(std::chrono::duration<double>(wait_s));
        while (!stop_ && std::chrono::steady_clock::now() < until)
          std::this_thread::sleep_for(std::min<std::chrono::steady_clock::duration>(until - std::chrono::steady_clock::now(), std::chrono::milliseconds(20)));
        tx_last_ = std::chrono::steady_clock::now();
        tx_tokens_ = 0.0;       // a message larger than the bucket leaves once the bucket's worth plus the rest has accrued
      } else {
        tx_tokens_ -= need;
      }
    }
    const bool sent = zmq_ ? zmq_->send(item->key, item->flags, payload.data(), payload.size(), timeout_ms_)
                           : send_frame(push_fd_, kGrad, item->key, item->flags, payload.data(), payload.size(), timeout_ms_);
    if (!sent) {
      if (!stop_) set_failed("send to the ring successor failed for " + item->key);
      return;
    }
    bytes_sent_ += sizeof(FrameHeader) + item->key.size() + payload.size();
  }
}

void CommManager::pull_main() {
  pthread_setname_np(pthread_self(), "CommPullThread");
  while (!stop_) {
    FrameHeader h{};
    std::string key;
    std::vector<unsigned char> payload;
    if (zmq_) {
      uint8_t flags = 0;
      bool malformed = false;
      if (!zmq_->recv(&key, &flags, &payload, 100, &malformed)) {
        if (malformed && !stop_) { set_failed("malformed ZeroMQ gradient message"); return; }
        continue;     // nothing within the poll interval (ZeroMQ hides connection loss; the engine's own deadlines catch it)
      }
      h.type = kGrad;
      h.flags = flags;
    } else {
      if (!wait_readable(pull_fd_, 100)) continue;
      if (!recv_frame(pull_fd_, &h, &key, &payload, timeout_ms_)) {
        if (!stop_) set_failed("the ring predecessor closed the connection or sent a truncated frame");
        return;
      }
    }
    if (h.type == kBye) {
      LOG_DEBUG("CommManager", "the ring predecessor shut down");
      return;
    }
    if (h.type != kGrad || payload.size() < 4) continue;
    SparseMessage m;
    m.key = key;
    m.flags = static_cast<uint8_t>(h.flags);
    if (!decode_sparse(m.flags, payload.data(), payload.size(), 0, &m.idx, &m.val)) {
      set_failed("malformed gradient frame for " + key);
      return;
    }
    m.wire_bytes = sizeof(FrameHeader) + key.size() + payload.size();
    bytes_recv_ += m.wire_bytes;
    rx_mon_.add(m.wire_bytes);
    std::function<void(SparseMessage&&)> cb;
    {
      std::lock_guard<std::mutex> lk(rx_mu_);
      auto it = posted_.find(key);
      if (it != posted_.end()) {
        cb = std::move(it->second);
        posted_.erase(it);
      } else {
        stash_[key] = std::move(m);   // arrived before its receive was posted
      }
    }
    if (cb) cb(std::move(m));
  }
}

void CommManager::post_recv(const std::string& key, std::function<void(SparseMessage&&)> cb) {
  SparseMessage m;
  bool have = false;
  {
    std::lock_guard<std::mutex> lk(rx_mu_);
    auto it = stash_.find(key);
    if (it != stash_.end()) {
      m = std::move(it->second);
      stash_.erase(it);
      have = true;
    } else {
      posted_[key] = std::move(cb);
    }
  }
  if (have) cb(std::move(m));
}

bool CommManager::cancel_recv(const std::string& key) {
  std::lock_guard<std::mutex> lk(rx_mu_);
  return posted_.erase(key) > 0;
}

size_t CommManager::stashed() const {
  std::lock_guard<std::mutex> lk(rx_mu_);
  return stash_.size();
}

// ---------------------------------------------------------------- control plane
bool CommManager::control_roundtrip(uint32_t type, const std::string& key, const void* payload, size_t payload_len,
                                    std::vector<unsigned char>* reply, int timeout_ms) {
  std::lock_guard<std::mutex> lk(control_mu_);
  if (control_fd_ < 0) return false;
  if (!send_frame(control_fd_, type, key, 0, payload, payload_len, timeout_ms)) return false;
  FrameHeader h;
  std::string rkey;
  std::vector<unsigned char> rp;
  if (!recv_frame(control_fd_, &h, &rkey, &rp, timeout_ms)) return false;
  if (reply) *reply = std::move(rp);
  return true;
}

bool CommManager::send_init_model(const std::string& key, const float* data, size_t n) {
  return control_roundtrip(kModelPut, key, data, n * sizeof(float), nullptr, timeout_ms_);
}

bool CommManager::recv_init_model(const std::string& key, float* data, size_t n) {
  std::vector<unsigned char> reply;
  if (!control_roundtrip(kModelGet, key, nullptr, 0, &reply, timeout_ms_)) return false;
  if (reply.size() != n * sizeof(float)) return false;
  std::memcpy(data, reply.data(), reply.size());
  return true;
}

bool CommManager::global_barrier() { return control_roundtrip(kBarrier, "", nullptr, 0, nullptr, timeout_ms_); }

double CommManager::sync_time(int pings) {
  // offset = server_time - (t_send + t_recv) / 2, smoothed with weights 0.9 / 0.1 (reference 286-311)
  double offset_ms = 0.0;
  bool first = true;
  for (int i = 0; i < pings; ++i) {
    const int64_t t0 = now_ns();
    std::vector<unsigned char> reply;
    if (!control_roundtrip(kSyncTime, "", &t0, sizeof(t0), &reply, timeout_ms_) || reply.size() != sizeof(int64_t)) break;
    const int64_t t1 = now_ns();
    int64_t ts;
    std::memcpy(&ts, reply.data(), sizeof(ts));
    const double off = (static_cast<double>(ts) - (static_cast<double>(t0) + static_cast<double>(t1)) / 2.0) / 1e6;
    offset_ms = first ? off : 0.9 * offset_ms + 0.1 * off;
    first = false;
  }
  return offset_ms;
}

bool CommManager::report_stat(double send_mbps, double recv_mbps) {
  PeerStat s{rank_, send_mbps, recv_mbps, 0.0};
  return control_roundtrip(kStatRep, "", &s, sizeof(s), nullptr, timeout_ms_);
}

std::vector<PeerStat> CommManager::broker_stats() {
  std::lock_guard<std::mutex> lk(stats_mu_);
  std::vector<PeerStat> out;
  for (auto& kv : stats_) out.push_back(kv.second);
  return out;
}

}  // namespace stc
