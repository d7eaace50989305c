// Telemetry client and server shim of the control plane.
//
// Message set of the reference's protobuf schema (backend/src/proto/message.proto:5-88; mirrored PODs in
// backend/src/engine/message.h:74-121): TrainConfig, Measurements, LocalTelemetryInit, Telemetry,
// GlobalTelemetryInit, Instruction, wrapped in typed requests and responses.  protoc is not available
// on the target machines, so the wire form is a fixed little-endian layout behind a 12-byte frame
// header; the Python controller (stellatrain_b200/control/messages.py) reads and writes the same bytes.
// Client behaviour after backend/src/engine/telemetry_client.cpp:5-110 (blocking init, queued reports
// from a worker thread, callback on INSTRUCTION); server shim after telemetry_server.cpp:10-96.
//
// Second transport, the reference's own: a uri that starts with "zmq://" makes client and server speak protobuf
// messages over a ZeroMQ REQ socket (proto_wire.h, ../comm/zmq_link.h; libzmq is opened at run time, the path in
// STELLATRAIN_LIBZMQ or the system's), which is what the reference's controller (batch_rate_alloc.py:283-321) and this
// package's control/zmq_endpoint.py answer.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../comm/zmq_link.h"

namespace stc {

#pragma pack(push, 1)
struct TrainConfig {
  uint32_t ubatch_size;
  uint32_t gradient_accumulation;
  double compression_rate;
};
struct TrainMeasurement {
  double grad_send_thpt_mbps, grad_recv_thpt_mbps, fwd_delay_ms, bwd_delay_ms, bwd_fwd_gap_ms, intra_fwd_gap_ms;
};
struct LocalTelemetryInit {
  uint32_t gpu_id, rank, local_rank;
  char gpu_name[64];
};
struct LocalTelemetry {
  uint32_t gpu_id;
  uint64_t uiter;
  TrainConfig config;
  TrainMeasurement measurement;
};
struct Instruction {
  uint64_t iter_effective_since;
  TrainConfig config;
};
struct TelemetryFrame {
  uint32_t magic, type, payload_len;
};
#pragma pack(pop)

constexpr uint32_t kTelemetryMagic = 0x31545453u;   // "STT1"
enum TelemetryType : uint32_t {
  kTelLocalInit = 1, kTelLocal = 2, kTelGlobalInit = 3, kTelInit = 4, kTelTerminate = 5,
  kTelOk = 100, kTelInstruction = 101,
};

using InstructionCallback = std::function<void(uint64_t iter_effective_since, const TrainConfig&)>;

class TelemetryClient {
 public:
  // uri: "tcp://host:port" or "host:port" (framed TCP), "zmq://host:port" (protobuf over ZeroMQ REQ).  Throws when the
  // controller cannot be reached in time.
  TelemetryClient(const std::string& uri, uint32_t gpu_id, const std::string& gpu_name, uint32_t rank,
                  uint32_t local_rank, int timeout_ms = 5000);
  ~TelemetryClient();
  // Non-blocking: queues one report; `cb` runs on the client's thread if the reply is an instruction.
  void report(uint64_t uiter, const TrainConfig& cfg, const TrainMeasurement& m, InstructionCallback cb = nullptr);
  size_t queued();
  uint64_t sent() const { return st_->sent; }
  bool alive() const { return !st_->dead; }
  // How many clients of this process were destroyed on their own worker thread so far (see State below); for tests.
  static uint64_t destroyed_on_own_thread();

 private:
  // Everything the worker thread touches lives in a block that the thread shares with this object.  A callback may
  // hold the last reference to whatever owns this client (a Python hook whose bound method was passed to report());
  // when the worker releases that callback, this object is destroyed ON the worker thread.  The destructor then cannot
  // join the thread it runs on: it lets the thread go, and the thread finishes on the shared block alone.
  struct State {
    int fd = -1;
    std::unique_ptr<ZmqReq> zmq;      // set instead of fd for the ZeroMQ transport
    uint32_t message_id = 0;
    int timeout_ms = 5000;
    std::mutex mu;
    std::condition_variable cv;
    std::deque<std::pair<LocalTelemetry, InstructionCallback>> queue;
    std::atomic<bool> stop{false}, dead{false};
    std::atomic<uint64_t> sent{0};
  };
  static void worker_main(std::shared_ptr<State> st);
  std::shared_ptr<State> st_;
  uint32_t gpu_id_;
  std::thread worker_;
};

class TelemetryServer {
 public:
  // When `launch_controller` is set the Python controller is started as a child process
  // (`python -m stellatrain_b200.control.controller --port <port>`), as the reference starts its
  // batch_rate_alloc.py with std::system (telemetry_server.cpp:57-73).
  TelemetryServer(const std::string& uri, bool launch_controller, int timeout_ms = 10000);
  ~TelemetryServer();
  bool send_global_telemetry(uint32_t num_nodes, uint32_t num_gpus, const std::vector<uint64_t>& param_counts,
                             bool grad_fp16, bool grad_idx_u16);
  bool terminate();

 private:
  int fd_ = -1;
  std::unique_ptr<ZmqReq> zmq_;
  int timeout_ms_;
  std::thread launcher_;
};

bool parse_uri(const std::string& uri, std::string* host, uint16_t* port);

}  // namespace stc
