#include "telemetry.h"

#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include "../comm/net_util.h"
#include "../core/logger.h"

namespace stc {

bool parse_uri(const std::string& uri, std::string* host, uint16_t* port) {
  std::string s = uri;
  const std::string scheme = "tcp://";
  if (s.compare(0, scheme.size(), scheme) == 0) s = s.substr(scheme.size());
  const size_t c = s.rfind(':');
  if (c == std::string::npos) return false;
  *host = s.substr(0, c);
  if (*host == "*" || host->empty()) *host = "127.0.0.1";
  const long p = std::strtol(s.c_str() + c + 1, nullptr, 10);
  if (p <= 0 || p > 65535) return false;
  *port = static_cast<uint16_t>(p);
  return true;
}

static bool send_msg(int fd, uint32_t type, const void* payload, uint32_t len, int timeout_ms) {
  TelemetryFrame f{kTelemetryMagic, type, len};
  return send_all(fd, &f, sizeof(f), timeout_ms) && (len == 0 || send_all(fd, payload, len, timeout_ms));
}

static bool recv_msg(int fd, uint32_t* type, std::vector<unsigned char>* payload, int timeout_ms) {
  TelemetryFrame f;
  if (!recv_all(fd, &f, sizeof(f), timeout_ms) || f.magic != kTelemetryMagic || f.payload_len > (1u << 24)) return false;
  payload->resize(f.payload_len);
  if (f.payload_len && !recv_all(fd, payload->data(), f.payload_len, timeout_ms)) return false;
  *type = f.type;
  return true;
}

TelemetryClient::TelemetryClient(const std::string& uri, uint32_t gpu_id, const std::string& gpu_name, uint32_t rank,
                                 uint32_t local_rank, int timeout_ms)
    : gpu_id_(gpu_id), timeout_ms_(timeout_ms) {
  std::string host;
  uint16_t port;
  if (!parse_uri(uri, &host, &port)) throw std::invalid_argument("bad telemetry uri: " + uri);
  fd_ = tcp_connect(host, port, timeout_ms);
  if (fd_ < 0) throw std::runtime_error("telemetry: cannot reach the controller at " + uri);
  LocalTelemetryInit init{};
  init.gpu_id = gpu_id;
  init.rank = rank;
  init.local_rank = local_rank;
  std::strncpy(init.gpu_name, gpu_name.c_str(), sizeof(init.gpu_name) - 1);
  uint32_t type;
  std::vector<unsigned char> reply;
  if (!send_msg(fd_, kTelLocalInit, &init, sizeof(init), timeout_ms) || !recv_msg(fd_, &type, &reply, timeout_ms)) {
    close_fd(fd_);
    throw std::runtime_error("telemetry: the controller did not acknowledge the registration");
  }
  worker_ = std::thread([this] { worker_main(); });
}

TelemetryClient::~TelemetryClient() {
  stop_ = true;
  cv_.notify_all();
  if (worker_.joinable()) worker_.join();
  close_fd(fd_);
}

void TelemetryClient::report(uint64_t uiter, const TrainConfig& cfg, const TrainMeasurement& m, InstructionCallback cb) {
  LocalTelemetry t{};
  t.gpu_id = gpu_id_;
  t.uiter = uiter;
  t.config = cfg;
  t.measurement = m;
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (queue_.size() > 4096) queue_.pop_front();   // a stalled controller must not grow memory
    queue_.emplace_back(t, std::move(cb));
  }
  cv_.notify_one();
}

size_t TelemetryClient::queued() {
  std::lock_guard<std::mutex> lk(mu_);
  return queue_.size();
}

void TelemetryClient::worker_main() {
  pthread_setname_np(pthread_self(), "TelemetryClient");
  while (!stop_) {
    std::pair<LocalTelemetry, InstructionCallback> item;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait_for(lk, std::chrono::milliseconds(100), [this] { return stop_ || !queue_.empty(); });
      if (stop_) return;
      if (queue_.empty()) continue;
      item = std::move(queue_.front());
      queue_.pop_front();
    }
    uint32_t type;
    std::vector<unsigned char> reply;
    if (!send_msg(fd_, kTelLocal, &item.first, sizeof(item.first), timeout_ms_) || !recv_msg(fd_, &type, &reply, timeout_ms_)) {
      LOG_WARN("TelemetryClient", "controller connection lost; telemetry stops, training continues");
      dead_ = true;
      return;
    }
    ++sent_;
    if (type == kTelInstruction && reply.size() == sizeof(Instruction) && item.second) {
      Instruction ins;
      std::memcpy(&ins, reply.data(), sizeof(ins));
      item.second(ins.iter_effective_since, ins.config);
    }
  }
}

TelemetryServer::TelemetryServer(const std::string& uri, bool launch_controller, int timeout_ms) : timeout_ms_(timeout_ms) {
  std::string host;
  uint16_t port;
  if (!parse_uri(uri, &host, &port)) throw std::invalid_argument("bad telemetry uri: " + uri);
  if (launch_controller) {
    launcher_ = std::thread([port] {
      const std::string cmd = "python -m stellatrain_b200.control.controller --port " + std::to_string(port);
      const int rc = std::system(cmd.c_str());
      if (rc != 0) LOG_WARN("TelemetryServer", "controller exited with status " << rc);
    });
  }
  fd_ = tcp_connect(host, port, timeout_ms);
  if (fd_ < 0) {
    if (launcher_.joinable()) launcher_.detach();
    throw std::runtime_error("telemetry server: controller not reachable at " + uri);
  }
  uint32_t type;
  std::vector<unsigned char> reply;
  if (!send_msg(fd_, kTelInit, nullptr, 0, timeout_ms_) || !recv_msg(fd_, &type, &reply, timeout_ms_))
    throw std::runtime_error("telemetry server: controller did not answer INIT");
}

TelemetryServer::~TelemetryServer() {
  close_fd(fd_);
  if (launcher_.joinable()) launcher_.join();
}

bool TelemetryServer::send_global_telemetry(uint32_t num_nodes, uint32_t num_gpus, const std::vector<uint64_t>& param_counts,
                                            bool grad_fp16, bool grad_idx_u16) {
  std::vector<unsigned char> buf(16 + param_counts.size() * 8);
  const uint32_t n = static_cast<uint32_t>(param_counts.size());
  std::memcpy(buf.data(), &num_nodes, 4);
  std::memcpy(buf.data() + 4, &num_gpus, 4);
  buf[8] = grad_fp16;
  buf[9] = grad_idx_u16;
  buf[10] = buf[11] = 0;
  std::memcpy(buf.data() + 12, &n, 4);
  if (n) std::memcpy(buf.data() + 16, param_counts.data(), static_cast<size_t>(n) * 8);
  uint32_t type;
  std::vector<unsigned char> reply;
  return send_msg(fd_, kTelGlobalInit, buf.data(), static_cast<uint32_t>(buf.size()), timeout_ms_) &&
         recv_msg(fd_, &type, &reply, timeout_ms_);
}

bool TelemetryServer::terminate() {
  uint32_t type;
  std::vector<unsigned char> reply;
  return send_msg(fd_, kTelTerminate, nullptr, 0, timeout_ms_) && recv_msg(fd_, &type, &reply, timeout_ms_);
}

}  // namespace stc
