#include "net_util.h"

#include <arpa/inet.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <random>

#include "../core/config.h"

namespace stc {

static bool private_v4(uint32_t host_order) {
  return (host_order >> 24) == 10 || (host_order >> 20) == (172u << 4 | 1) || (host_order >> 16) == (192u << 8 | 168);
}

std::vector<IfAddr> list_interfaces() {
  std::vector<IfAddr> out;
  ifaddrs* ifa = nullptr;
  if (getifaddrs(&ifa) != 0) return out;
  for (ifaddrs* p = ifa; p; p = p->ifa_next) {
    if (!p->ifa_addr || p->ifa_addr->sa_family != AF_INET || !(p->ifa_flags & IFF_UP)) continue;
    const auto* sin = reinterpret_cast<const sockaddr_in*>(p->ifa_addr);
    char buf[INET_ADDRSTRLEN];
    if (!inet_ntop(AF_INET, &sin->sin_addr, buf, sizeof(buf))) continue;
    IfAddr a;
    a.ifname = p->ifa_name;
    a.ip = buf;
    a.loopback = (p->ifa_flags & IFF_LOOPBACK) != 0;
    a.is_private = private_v4(ntohl(sin->sin_addr.s_addr));
    out.push_back(a);
  }
  freeifaddrs(ifa);
  return out;
}

std::string pick_local_ip() {
  if (const char* ip = std::getenv("PUBLIC_IP")) return ip;
  const auto ifs = list_interfaces();
  if (const char* want = std::getenv("IFNAME"))
    for (auto& a : ifs)
      if (a.ifname == want) return a.ip;
  for (auto& a : ifs)
    if (!a.loopback && !a.is_private) return a.ip;
  for (auto& a : ifs)
    if (!a.loopback) return a.ip;
  return "127.0.0.1";
}

// ---------------------------------------------------------------- bandwidth monitor
static int64_t window_index(std::chrono::steady_clock::time_point t) {
  return std::chrono::duration_cast<std::chrono::milliseconds>(t.time_since_epoch()).count() / 100;
}

void BandwidthMonitor::roll(std::chrono::steady_clock::time_point now) {
  const int64_t w = window_index(now);
  while (!windows_.empty() && windows_.front().first <= w - 10) windows_.pop_front();
}

void BandwidthMonitor::add(size_t bytes) {
  const auto now = std::chrono::steady_clock::now();
  std::lock_guard<std::mutex> lk(mu_);
  roll(now);
  const int64_t w = window_index(now);
  if (windows_.empty() || windows_.back().first != w) windows_.emplace_back(w, 0);
  windows_.back().second += bytes;
  total_ += bytes;
}

double BandwidthMonitor::peak_bytes_per_s() {
  std::lock_guard<std::mutex> lk(mu_);
  roll(std::chrono::steady_clock::now());
  size_t mx = 0;
  for (auto& w : windows_) mx = w.second > mx ? w.second : mx;
  return static_cast<double>(mx) * 10.0;
}

double BandwidthMonitor::mean_bytes_per_s() {
  std::lock_guard<std::mutex> lk(mu_);
  roll(std::chrono::steady_clock::now());
  size_t sum = 0;
  for (auto& w : windows_) sum += w.second;
  return static_cast<double>(sum);
}

// ---------------------------------------------------------------- TCP
static void tune(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int buf = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

int tcp_listen(uint16_t port, uint16_t* bound_port, bool any_port_in_range) {
  std::mt19937 rng(static_cast<unsigned>(getpid()) * 2654435761u + static_cast<unsigned>(time(nullptr)));
  for (int attempt = 0; attempt < (any_port_in_range ? 64 : 1); ++attempt) {
    const int fd = socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
    const uint16_t p = any_port_in_range
                           ? static_cast<uint16_t>(cfg::kDataPortLo + rng() % (cfg::kDataPortHi - cfg::kDataPortLo))
                           : port;
    addr.sin_port = htons(p);
    if (bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0 && listen(fd, 64) == 0) {
      socklen_t len = sizeof(addr);
      getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
      if (bound_port) *bound_port = ntohs(addr.sin_port);
      return fd;
    }
    close(fd);
  }
  return -1;
}

bool wait_readable(int fd, int timeout_ms) {
  pollfd p{fd, POLLIN, 0};
  for (;;) {
    const int rc = poll(&p, 1, timeout_ms);
    if (rc > 0) return (p.revents & (POLLIN | POLLHUP | POLLERR)) != 0;
    if (rc == 0) return false;
    if (errno != EINTR) return false;
  }
}

int tcp_accept(int listen_fd, int timeout_ms) {
  if (!wait_readable(listen_fd, timeout_ms)) return -1;
  const int fd = accept(listen_fd, nullptr, nullptr);
  if (fd >= 0) tune(fd);
  return fd;
}

int tcp_connect(const std::string& host, uint16_t port, int timeout_ms) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res) return -1;
  const auto t0 = std::chrono::steady_clock::now();
  int fd = -1;
  for (;;) {
    fd = socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) break;
    if (connect(fd, res->ai_addr, res->ai_addrlen) == 0) break;
    close(fd);
    fd = -1;
    if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms)) break;
    usleep(20000);   // the peer may not be listening yet
  }
  freeaddrinfo(res);
  if (fd >= 0) tune(fd);
  return fd;
}

bool send_all(int fd, const void* buf, size_t len, int timeout_ms) {
  const auto* p = static_cast<const unsigned char*>(buf);
  const auto t0 = std::chrono::steady_clock::now();
  while (len) {
    const ssize_t n = send(fd, p, len, MSG_NOSIGNAL);
    if (n > 0) { p += n; len -= static_cast<size_t>(n); continue; }
    if (n < 0 && (errno == EINTR)) continue;
    if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) {
      if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms)) return false;
      pollfd pf{fd, POLLOUT, 0};
      poll(&pf, 1, 50);
      continue;
    }
    return false;
  }
  return true;
}

bool recv_all(int fd, void* buf, size_t len, int timeout_ms) {
  auto* p = static_cast<unsigned char*>(buf);
  const auto t0 = std::chrono::steady_clock::now();
  while (len) {
    const int left = timeout_ms - static_cast<int>(std::chrono::duration_cast<std::chrono::milliseconds>(
                                      std::chrono::steady_clock::now() - t0).count());
    if (left <= 0 || !wait_readable(fd, left)) return false;
    const ssize_t n = recv(fd, p, len, 0);
    if (n > 0) { p += n; len -= static_cast<size_t>(n); continue; }
    if (n < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    return false;   // closed or error
  }
  return true;
}

void close_fd(int& fd) {
  if (fd >= 0) {
    shutdown(fd, SHUT_RDWR);
    close(fd);
    fd = -1;
  }
}

}  // namespace stc
