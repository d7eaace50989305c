#include "telemetry.h"

#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include "../comm/net_util.h"
#include "../core/logger.h"
#include "proto_wire.h"

namespace stc {

// "zmq://host:port" (also "zmq+tcp://"): the ZeroMQ transport; *endpoint becomes "tcp://host:port".
static bool zmq_uri(const std::string& uri, std::string* endpoint) {
  for (const char* scheme : {"zmq://", "zmq+tcp://"}) {
    const std::string sc(scheme);
    if (uri.compare(0, sc.size(), sc) == 0) {
      *endpoint = "tcp://" + uri.substr(sc.size());
      return true;
    }
  }
  return false;
}

static std::unique_ptr<ZmqReq> zmq_connect(const std::string& endpoint, const std::string& what) {
  std::string why;
  if (!ZmqLibrary::load("", &why)) throw std::runtime_error(what + ": " + why);
  auto req = std::make_unique<ZmqReq>();
  if (!req->connect(endpoint)) throw std::runtime_error(what + ": cannot connect a ZeroMQ REQ socket to " + endpoint);
  return req;
}

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
    : st_(std::make_shared<State>()), gpu_id_(gpu_id) {
  st_->timeout_ms = timeout_ms;
  LocalTelemetryInit init{};
  init.gpu_id = gpu_id;
  init.rank = rank;
  init.local_rank = local_rank;
  std::strncpy(init.gpu_name, gpu_name.c_str(), sizeof(init.gpu_name) - 1);
  std::string endpoint;
  if (zmq_uri(uri, &endpoint)) {
    st_->zmq = zmq_connect(endpoint, "telemetry");
    pbwire::Bytes reply;
    uint32_t type = 0;
    bool has = false;
    Instruction ins{};
    if (!st_->zmq->request(pbwire::request_local_init(init), &reply, timeout_ms) ||
        !pbwire::parse_response(reply, &type, &has, &ins) || type == pbwire::kRespInvalid) {
      st_->zmq->close();
      throw std::runtime_error("telemetry: the controller did not acknowledge the registration");
    }
  } else {
    std::string host;
    uint16_t port;
    if (!parse_uri(uri, &host, &port)) throw std::invalid_argument("bad telemetry uri: " + uri);
    st_->fd = tcp_connect(host, port, timeout_ms);
    if (st_->fd < 0) throw std::runtime_error("telemetry: cannot reach the controller at " + uri);
    uint32_t type;
    std::vector<unsigned char> reply;
    if (!send_msg(st_->fd, kTelLocalInit, &init, sizeof(init), timeout_ms) || !recv_msg(st_->fd, &type, &reply, timeout_ms)) {
      close_fd(st_->fd);
      throw std::runtime_error("telemetry: the controller did not acknowledge the registration");
    }
  }
  worker_ = std::thread(worker_main, st_);
}

namespace {
std::atomic<uint64_t> g_destroyed_on_own_thread{0};
}
uint64_t TelemetryClient::destroyed_on_own_thread() { return g_destroyed_on_own_thread.load(); }

TelemetryClient::~TelemetryClient() {
  st_->stop = true;
  st_->cv.notify_all();
  if (worker_.joinable()) {
    if (worker_.get_id() == std::this_thread::get_id()) {
      ++g_destroyed_on_own_thread;
      worker_.detach();          // destroyed from the worker itself (see State): it closes the socket on its way out
      return;
    }
    worker_.join();
  }
  close_fd(st_->fd);
  if (st_->zmq) st_->zmq->close();
}

void TelemetryClient::report(uint64_t uiter, const TrainConfig& cfg, const TrainMeasurement& m, InstructionCallback cb) {
  LocalTelemetry t{};
  t.gpu_id = gpu_id_;
  t.uiter = uiter;
  t.config = cfg;
  t.measurement = m;
  {
    std::lock_guard<std::mutex> lk(st_->mu);
    if (st_->queue.size() > 4096) st_->queue.pop_front();   // a stalled controller must not grow memory
    st_->queue.emplace_back(t, std::move(cb));
  }
  st_->cv.notify_one();
}

size_t TelemetryClient::queued() {
  std::lock_guard<std::mutex> lk(st_->mu);
  return st_->queue.size();
}

void TelemetryClient::worker_main(std::shared_ptr<State> st) {
  pthread_setname_np(pthread_self(), "TelemetryClient");
  bool detached = false;
  while (!st->stop) {
    {
      std::pair<LocalTelemetry, InstructionCallback> item;
      {
        std::unique_lock<std::mutex> lk(st->mu);
        st->cv.wait_for(lk, std::chrono::milliseconds(100), [&st] { return st->stop || !st->queue.empty(); });
        if (st->stop) break;
        if (st->queue.empty()) continue;
        item = std::move(st->queue.front());
        st->queue.pop_front();
      }
      uint32_t type = 0;
      std::vector<unsigned char> reply;
      bool ok, has_instruction = false;
      Instruction ins{};
      if (st->zmq) {
        ok = st->zmq->request(pbwire::request_telemetry(item.first, st->message_id++), &reply, st->timeout_ms) &&
             pbwire::parse_response(reply, &type, &has_instruction, &ins) && type != pbwire::kRespInvalid;
      } else {
        ok = send_msg(st->fd, kTelLocal, &item.first, sizeof(item.first), st->timeout_ms) &&
             recv_msg(st->fd, &type, &reply, st->timeout_ms);
        if (ok && type == kTelInstruction && reply.size() == sizeof(Instruction)) {
          std::memcpy(&ins, reply.data(), sizeof(ins));
          has_instruction = true;
        }
      }
      if (!ok) {
        LOG_WARN("TelemetryClient", "controller connection lost; telemetry stops, training continues");
        st->dead = true;
        break;
      }
      ++st->sent;
      if (has_instruction && item.second) item.second(ins.iter_effective_since, ins.config);
    }   // the callback is released here, which may destroy the client on this very thread
    if (st->stop && st.use_count() == 1) detached = true;
  }
  // queued callbacks may own the client as well: release them before deciding who closes the socket
  std::deque<std::pair<LocalTelemetry, InstructionCallback>> rest;
  {
    std::lock_guard<std::mutex> lk(st->mu);
    rest.swap(st->queue);
  }
  rest.clear();
  if (detached || st.use_count() == 1) {   // the client is gone and could not close the connection itself
    close_fd(st->fd);
    if (st->zmq) st->zmq->close();
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
  std::string endpoint;
  if (zmq_uri(uri, &endpoint)) {
    zmq_ = zmq_connect(endpoint, "telemetry server");
    pbwire::Bytes reply;
    uint32_t type = 0;
    bool has = false;
    Instruction ins{};
    if (!zmq_->request(pbwire::request_plain(pbwire::kReqInit), &reply, timeout_ms_) ||
        !pbwire::parse_response(reply, &type, &has, &ins) || type == pbwire::kRespInvalid)
      throw std::runtime_error("telemetry server: controller did not answer INIT");
    return;
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
  if (zmq_) zmq_->close();
  if (launcher_.joinable()) launcher_.join();
}

bool TelemetryServer::send_global_telemetry(uint32_t num_nodes, uint32_t num_gpus, const std::vector<uint64_t>& param_counts,
                                            bool grad_fp16, bool grad_idx_u16) {
  if (zmq_) {
    pbwire::Bytes reply;
    uint32_t type = 0;
    bool has = false;
    Instruction ins{};
    return zmq_->request(pbwire::request_global_init(num_nodes, num_gpus, param_counts, grad_fp16, grad_idx_u16), &reply,
                         timeout_ms_) &&
           pbwire::parse_response(reply, &type, &has, &ins) && type == pbwire::kRespOk;
  }
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
  if (zmq_) {
    pbwire::Bytes reply;
    uint32_t type = 0;
    bool has = false;
    Instruction ins{};
    return zmq_->request(pbwire::request_plain(pbwire::kReqTerminate), &reply, timeout_ms_) &&
           pbwire::parse_response(reply, &type, &has, &ins);
  }
  uint32_t type;
  std::vector<unsigned char> reply;
  return send_msg(fd_, kTelTerminate, nullptr, 0, timeout_ms_) && recv_msg(fd_, &type, &reply, timeout_ms_);
}

}  // namespace stc
