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
#include <chrono>
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
#include "zmq_link.h"

namespace stc {

constexpr uint8_t kFlagIdxU16 = 0x01;   // reference comm_manager.h:24
constexpr uint8_t kFlagValF16 = 0x02;   // reference comm_manager.h:25
constexpr uint8_t kFlagValBF16 = 0x04;
constexpr uint8_t kFlagBlock16 = 0x08;  // part of the entries travels as whole aligned blocks of 16
constexpr uint8_t kFlagBlockU16 = 0x10; // block ids are 16 bits wide (tensors of up to 1,048,576 elements)

struct SparseMessage {
  std::string key;
  uint8_t flags = 0;
  std::vector<uint32_t> idx;
  std::vector<float> val;
  size_t wire_bytes = 0;
};

// Payload of one gradient message.
//
//   plain:  count:u32 | idx[count] (u32, or u16 with kFlagIdxU16) | val[count] (f32, f16 or bf16)
//   blocks: count:u32 | nblocks:u32 | block_id[nblocks] (u32, or u16 with kFlagBlockU16)
//           | idx[count - 16 nblocks] | val[count]
//
// The block form is what threshold-v16 produces most of the time: 16 consecutive indices that start at a
// multiple of 16.  Such a run is sent as one block id (index / 16) followed by its 16 values, which removes
// 15 of 16 indices: 68 bytes instead of 128 for a block of fp32 values (the reference always sends
// (index, value) pairs, backend/src/engine/comm_manager.cpp:748-764).  The encoder moves the whole blocks to
// the front of the message and the loose entries behind them; a receiver that merges by index does not depend
// on the order.  A message without a single whole block is sent in the plain form.
struct EncodedSparse {
  uint8_t flags = 0;
  uint32_t count = 0;
  std::vector<unsigned char> payload;
};
EncodedSparse encode_sparse(const uint32_t* idx, const float* val, size_t count, uint32_t tensor_numel, bool allow_u16,
                            int value_format, bool allow_blocks);
// Returns false when the payload does not have the size its header implies or names an index outside the tensor
// (tensor_numel 0: not checked).
bool decode_sparse(uint8_t flags, const unsigned char* payload, size_t len, uint32_t tensor_numel,
                   std::vector<uint32_t>* idx, std::vector<float>* val);

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

  // Transport of the gradient ring, chosen before start_client: "tcp" (length-prefixed frames on plain sockets, the
  // default) or "zmq" (ZeroMQ PUSH/PULL sockets as in the reference, backend/src/engine/comm_manager.cpp:369-477; the
  // library is opened at run time, `libzmq_hint` may name it).  The control plane stays on framed TCP either way.
  // Also selected by STELLATRAIN_DATA_TRANSPORT=zmq.  Returns false when ZeroMQ cannot be loaded.
  bool set_data_transport(const std::string& name, const std::string& libzmq_hint = "");
  const char* data_transport() const { return zmq_ ? "zmq" : "tcp"; }

  // ---- gradient data (ring)
  void queue_tx(int64_t priority, const std::string& key, const uint32_t* idx, const float* val, size_t count,
                uint32_t tensor_numel, bool allow_u16 = true, int value_format = 0 /*0 f32, 1 f16, 2 bf16*/,
                bool allow_blocks = true);
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
  // Paces the gradient sends of this node to `bytes_per_s` (0: unlimited) with a token bucket of `burst_bytes`: a
  // software stand-in for a slow link between nodes, so that the regime the reference was written for (about
  // 1 Gbit/s between machines) can be reproduced on one host.  Control-plane messages are not paced.
  void set_tx_rate_limit(double bytes_per_s, size_t burst_bytes = 64 << 10);
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
    std::vector<unsigned char> payload;
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
  std::atomic<double> tx_rate_{0.0};            // bytes per second, 0 = unlimited
  std::atomic<size_t> tx_burst_{64 << 10};
  double tx_tokens_ = 0.0;                       // push thread only
  std::chrono::steady_clock::time_point tx_last_{};
  BandwidthMonitor rx_mon_;
  std::atomic<uint64_t> bytes_sent_{0}, bytes_recv_{0};
  std::unique_ptr<ZmqLink> zmq_;                 // set: the ring runs over ZeroMQ PUSH/PULL instead of plain sockets
};

}  // namespace stc
