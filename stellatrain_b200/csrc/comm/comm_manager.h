// Inter-node transport of the CPU tier over plain TCP.
//
// Capabilities of the reference's CommManager (backend/src/engine/comm_manager.cpp:95-335 broker,
// 369-477 client start, 572-602 queueTx, 722-815 push thread, 833-974 pull thread with the
// "arrived before posted" stash, 1022-1077 initial-model relay, 286-311 time sync, 252-284 stat
// reports) with length-prefixed frames instead of ZeroMQ multipart messages (no zmq headers exist on
// the target machines).  Topology is the same: a star for control (every node keeps one connection to
// the broker on rank 0) and a unidirectional ring for gradient data; data messages are keyed, may
// arrive before their receive is posted, and are sent in priority order (smaller first).
// Unlike the reference every blocking call has a deadline, and a send can be dropped or delayed by a
// host-side hook so that failure handling is testable without breaking real links.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <queue>
#include <string>
#include <thread>
#include <vector>

#include "net_util.h"

namespace stc {

constexpr uint8_t kFlagIdxU16 = 0x01;   // reference comm_manager.h:24
constexpr uint8_t kFlagValF16 = 0x02;   // reference comm_manager.h:25
constexpr uint8_t kFlagValBF16 = 0x04;

struct SparseMessage {
  std::string key;
  uint8_t flags = 0;
  std::vector<uint32_t> idx;
  std::vector<float> val;
  size_t wire_bytes = 0;
};

struct PeerStat {       // one line of the broker's link report
  int rank;
  double send_mbps, recv_mbps, clock_offset_ms;
};

class CommManager {
 public:
  CommManager(const std::string& master_addr, uint16_t master_port, int timeout_ms);
  ~CommManager();

  // rank 0 only: start the broker for `world` nodes.
  void start_server(int world);
  // every node (rank 0 included): register with the broker, open the data listener, connect to the
  // ring successor, start the push and pull threads.  Returns false on timeout.
  bool start_client(int rank, int world, int num_gpus);
  int rank() const { return rank_; }
  int world() const { return world_; }

  // ---- gradient data (ring)
  void queue_tx(int64_t priority, const std::string& key, const uint32_t* idx, const float* val, size_t count,
                uint32_t tensor_numel, bool allow_u16 = true, int value_format = 0 /*0 f32, 1 f16, 2 bf16*/);
  // `cb` runs on the pull thread (or immediately on the caller when the message is already here).
  void post_recv(const std::string& key, std::function<void(SparseMessage&&)> cb);
  bool cancel_recv(const std::string& key);

  // ---- control plane (through the broker)
  bool send_init_model(const std::string& key, const float* data, size_t n);
  bool recv_init_model(const std::string& key, float* data, size_t n);
  bool global_barrier();                               // all nodes
  double sync_time(int pings = 16);                    // estimated clock offset to the broker in ms
  bool report_stat(double send_mbps, double recv_mbps);
  std::vector<PeerStat> broker_stats();                // rank 0: latest reports

  // ---- observability and host-side fault injection
  BandwidthMonitor& rx_monitor() { return rx_mon_; }
  uint64_t bytes_sent() const { return bytes_sent_; }
  uint64_t bytes_received() const { return bytes_recv_; }
  size_t stashed() const;
  // return true to drop the message; positive delay_ms stalls the sender before the send
  void set_tx_fault_hook(std::function<bool(const std::string& key, int* delay_ms)> hook);
  bool failed() const { return failed_; }
  std::string failure() const;

 private:
  struct TxItem {
    int64_t priority;
    uint64_t seq;
    std::string key;
    uint8_t flags;
    std::vector<unsigned char> idx_bytes, val_bytes;
    uint32_t count;
  };
  struct TxLater {
    bool operator()(const std::shared_ptr<TxItem>& a, const std::shared_ptr<TxItem>& b) const {
      return a->priority != b->priority ? a->priority > b->priority : a->seq > b->seq;
    }
  };
  void broker_main(int world);
  void push_main();
  void pull_main();
  bool control_roundtrip(uint32_t type, const std::string& key, const void* payload, size_t payload_len,
                         std::vector<unsigned char>* reply, int timeout_ms);
  void set_failed(const std::string& why);

  std::string master_addr_;
  uint16_t master_port_;
  int timeout_ms_;
  int rank_ = -1, world_ = 0;
  std::atomic<bool> stop_{false};
  std::atomic<bool> failed_{false};
  mutable std::mutex fail_mu_;
  std::string failure_;

  // broker
  std::thread broker_thread_;
  int broker_listen_fd_ = -1;
  std::mutex stats_mu_;
  std::map<int, PeerStat> stats_;

  // client
  int control_fd_ = -1;
  std::mutex control_mu_;
  int data_listen_fd_ = -1, pull_fd_ = -1, push_fd_ = -1;
  std::thread push_thread_, pull_thread_;
  std::mutex tx_mu_;
  std::condition_variable tx_cv_;
  std::priority_queue<std::shared_ptr<TxItem>, std::vector<std::shared_ptr<TxItem>>, TxLater> tx_queue_;
  uint64_t tx_seq_ = 0;
  mutable std::mutex rx_mu_;
  std::map<std::string, std::function<void(SparseMessage&&)>> posted_;
  std::map<std::string, SparseMessage> stash_;
  std::function<bool(const std::string&, int*)> tx_hook_;
  BandwidthMonitor rx_mon_;
  std::atomic<uint64_t> bytes_sent_{0}, bytes_recv_{0};
};

}  // namespace stc
