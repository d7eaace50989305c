// Telemetry client and server shim of the control plane.
//
// Message set of the reference's protobuf schema (backend/src/proto/message.proto:5-88; mirrored PODs in
// backend/src/engine/message.h:74-121): TrainConfig, Measurements, LocalTelemetryInit, Telemetry,
// GlobalTelemetryInit, Instruction, wrapped in typed requests and responses.  protoc is not available
// on the target machines, so the wire form is a fixed little-endian layout behind a 12-byte frame
// header; the Python controller (stellatrain_b200/control/messages.py) reads and writes the same bytes.
// Client behaviour after backend/src/engine/telemetry_client.cpp:5-110 (blocking init, queued reports
// from a worker thread, callback on INSTRUCTION); server shim after telemetry_server.cpp:10-96.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

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
  // uri: "tcp://host:port" or "host:port".  Throws when the controller cannot be reached in time.
  TelemetryClient(const std::string& uri, uint32_t gpu_id, const std::string& gpu_name, uint32_t rank,
                  uint32_t local_rank, int timeout_ms = 5000);
  ~TelemetryClient();
  // Non-blocking: queues one report; `cb` runs on the client's thread if the reply is an instruction.
  void report(uint64_t uiter, const TrainConfig& cfg, const TrainMeasurement& m, InstructionCallback cb = nullptr);
  size_t queued();
  uint64_t sent() const { return sent_; }
  bool alive() const { return !dead_; }

 private:
  void worker_main();
  int fd_ = -1;
  uint32_t gpu_id_;
  int timeout_ms_;
  std::thread worker_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::pair<LocalTelemetry, InstructionCallback>> queue_;
  std::atomic<bool> stop_{false}, dead_{false};
  std::atomic<uint64_t> sent_{0};
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
  int timeout_ms_;
  std::thread launcher_;
};

bool parse_uri(const std::string& uri, std::string* host, uint16_t* port);

}  // namespace stc
