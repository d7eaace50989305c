#include "zmq_link.h"

#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace stc {

namespace {

// The part of zmq.h (libzmq 4.x, stable ABI) that this file uses.
constexpr int kZmqPull = 7, kZmqPush = 8, kZmqReq = 3;
constexpr int kZmqSndMore = 2;
constexpr int kZmqLinger = 17, kZmqSndHwm = 23, kZmqRcvHwm = 24, kZmqRcvTimeo = 27, kZmqSndTimeo = 28, kZmqLastEndpoint = 32;
struct alignas(8) ZmqMsg { unsigned char opaque[64]; };

struct Api {
  void* (*ctx_new)() = nullptr;
  int (*ctx_term)(void*) = nullptr;
  void* (*socket)(void*, int) = nullptr;
  int (*close)(void*) = nullptr;
  int (*bind)(void*, const char*) = nullptr;
  int (*connect)(void*, const char*) = nullptr;
  int (*setsockopt)(void*, int, const void*, size_t) = nullptr;
  int (*getsockopt)(void*, int, void*, size_t*) = nullptr;
  int (*send)(void*, const void*, size_t, int) = nullptr;
  int (*msg_init)(ZmqMsg*) = nullptr;
  int (*msg_recv)(ZmqMsg*, void*, int) = nullptr;
  void* (*msg_data)(ZmqMsg*) = nullptr;
  size_t (*msg_size)(const ZmqMsg*) = nullptr;
  int (*msg_more)(const ZmqMsg*) = nullptr;
  int (*msg_close)(ZmqMsg*) = nullptr;
  void* handle = nullptr;
};

Api g_api;
std::mutex g_mu;

template <typename F>
bool sym(void* h, const char* name, F* out) {
  *out = reinterpret_cast<F>(dlsym(h, name));
  return *out != nullptr;
}

}  // namespace

bool ZmqLibrary::loaded() {
  std::lock_guard<std::mutex> lk(g_mu);
  return g_api.handle != nullptr;
}

bool ZmqLibrary::load(const std::string& hint, std::string* why) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_api.handle != nullptr) return true;
  std::vector<std::string> names;
  if (const char* env = std::getenv("STELLATRAIN_LIBZMQ")) names.emplace_back(env);
  if (!hint.empty()) names.push_back(hint);
  names.emplace_back("libzmq.so.5");
  names.emplace_back("libzmq.so");
  void* h = nullptr;
  std::string tried;
  for (const auto& n : names) {
    h = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h != nullptr) break;
    tried += (tried.empty() ? "" : ", ") + n;
  }
  if (h == nullptr) {
    if (why) *why = "no ZeroMQ library could be opened (tried " + tried + ")";
    return false;
  }
  Api a;
  const bool ok = sym(h, "zmq_ctx_new", &a.ctx_new) && sym(h, "zmq_ctx_term", &a.ctx_term) && sym(h, "zmq_socket", &a.socket) &&
                  sym(h, "zmq_close", &a.close) && sym(h, "zmq_bind", &a.bind) && sym(h, "zmq_connect", &a.connect) &&
                  sym(h, "zmq_setsockopt", &a.setsockopt) && sym(h, "zmq_getsockopt", &a.getsockopt) &&
                  sym(h, "zmq_send", &a.send) && sym(h, "zmq_msg_init", &a.msg_init) && sym(h, "zmq_msg_recv", &a.msg_recv) &&
                  sym(h, "zmq_msg_data", &a.msg_data) && sym(h, "zmq_msg_size", &a.msg_size) &&
                  sym(h, "zmq_msg_more", &a.msg_more) && sym(h, "zmq_msg_close", &a.msg_close);
  if (!ok) {
    dlclose(h);
    if (why) *why = "the library that was opened does not export the ZeroMQ 4 entry points";
    return false;
  }
  a.handle = h;
  g_api = a;
  return true;
}

ZmqLink::ZmqLink() {
  if (g_api.handle != nullptr) ctx_ = g_api.ctx_new();
}

ZmqLink::~ZmqLink() { close(); }

void ZmqLink::close() {
  if (push_) { g_api.close(push_); push_ = nullptr; }
  if (pull_) { g_api.close(pull_); pull_ = nullptr; }
  if (ctx_) { g_api.ctx_term(ctx_); ctx_ = nullptr; }
}

uint16_t ZmqLink::bind_pull(const std::string& ip) {
  if (ctx_ == nullptr) return 0;
  pull_ = g_api.socket(ctx_, kZmqPull);
  if (pull_ == nullptr) return 0;
  const int zero = 0;
  g_api.setsockopt(pull_, kZmqLinger, &zero, sizeof(zero));
  g_api.setsockopt(pull_, kZmqRcvHwm, &zero, sizeof(zero));      // no limit, as the reference sets it
  const std::string ep = "tcp://" + ip + ":*";
  if (g_api.bind(pull_, ep.c_str()) != 0) return 0;
  char last[256] = {};
  size_t n = sizeof(last);
  if (g_api.getsockopt(pull_, kZmqLastEndpoint, last, &n) != 0) return 0;
  const char* colon = std::strrchr(last, ':');
  return colon ? static_cast<uint16_t>(std::atoi(colon + 1)) : 0;
}

bool ZmqLink::connect_push(const std::string& ip, uint16_t port) {
  if (ctx_ == nullptr) return false;
  push_ = g_api.socket(ctx_, kZmqPush);
  if (push_ == nullptr) return false;
  const int zero = 0;
  g_api.setsockopt(push_, kZmqLinger, &zero, sizeof(zero));
  g_api.setsockopt(push_, kZmqSndHwm, &zero, sizeof(zero));
  const std::string ep = "tcp://" + ip + ":" + std::to_string(port);
  return g_api.connect(push_, ep.c_str()) == 0;
}

bool ZmqLink::send(const std::string& key, uint8_t flags, const unsigned char* payload, size_t len, int timeout_ms) {
  if (push_ == nullptr) return false;
  g_api.setsockopt(push_, kZmqSndTimeo, &timeout_ms, sizeof(timeout_ms));
  if (g_api.send(push_, key.data(), key.size(), kZmqSndMore) < 0) return false;
  if (g_api.send(push_, &flags, 1, kZmqSndMore) < 0) return false;
  return g_api.send(push_, payload, len, 0) >= 0;
}

bool ZmqLink::recv(std::string* key, uint8_t* flags, std::vector<unsigned char>* payload, int timeout_ms, bool* malformed) {
  if (malformed) *malformed = false;
  if (pull_ == nullptr) return false;
  g_api.setsockopt(pull_, kZmqRcvTimeo, &timeout_ms, sizeof(timeout_ms));
  int part = 0;
  bool more = true, ok = true;
  while (more) {
    ZmqMsg m;
    g_api.msg_init(&m);
    if (g_api.msg_recv(&m, pull_, 0) < 0) {
      g_api.msg_close(&m);
      if (part != 0 && malformed) *malformed = true;   // a message that stops between its frames
      return false;
    }
    const unsigned char* d = static_cast<const unsigned char*>(g_api.msg_data(&m));
    const size_t n = g_api.msg_size(&m);
    if (part == 0) key->assign(reinterpret_cast<const char*>(d), n);
    else if (part == 1) { if (n == 1) *flags = d[0]; else ok = false; }
    else if (part == 2) payload->assign(d, d + n);
    more = g_api.msg_more(&m) != 0;
    g_api.msg_close(&m);
    ++part;
  }
  if (part != 3 || !ok) {
    if (malformed) *malformed = true;
    return false;
  }
  return true;
}

ZmqReq::ZmqReq() {
  if (g_api.handle != nullptr) ctx_ = g_api.ctx_new();
}

ZmqReq::~ZmqReq() { close(); }

void ZmqReq::close() {
  if (sock_) { g_api.close(sock_); sock_ = nullptr; }
  if (ctx_) { g_api.ctx_term(ctx_); ctx_ = nullptr; }
}

bool ZmqReq::connect(const std::string& endpoint) {
  if (ctx_ == nullptr) return false;
  sock_ = g_api.socket(ctx_, kZmqReq);
  if (sock_ == nullptr) return false;
  const int zero = 0;
  g_api.setsockopt(sock_, kZmqLinger, &zero, sizeof(zero));
  return g_api.connect(sock_, endpoint.c_str()) == 0;
}

bool ZmqReq::request(const std::vector<unsigned char>& body, std::vector<unsigned char>* reply, int timeout_ms) {
  if (sock_ == nullptr) return false;
  g_api.setsockopt(sock_, kZmqSndTimeo, &timeout_ms, sizeof(timeout_ms));
  g_api.setsockopt(sock_, kZmqRcvTimeo, &timeout_ms, sizeof(timeout_ms));
  if (g_api.send(sock_, body.data(), body.size(), 0) < 0) return false;
  reply->clear();
  bool more = true;
  while (more) {
    ZmqMsg m;
    g_api.msg_init(&m);
    if (g_api.msg_recv(&m, sock_, 0) < 0) {
      g_api.msg_close(&m);
      return false;
    }
    const unsigned char* d = static_cast<const unsigned char*>(g_api.msg_data(&m));
    reply->insert(reply->end(), d, d + g_api.msg_size(&m));
    more = g_api.msg_more(&m) != 0;
    g_api.msg_close(&m);
  }
  return true;
}

}  // namespace stc
