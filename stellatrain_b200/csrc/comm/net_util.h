// Small network helpers of the CPU tier: interface discovery (role of backend/src/misc/ipaddr.cpp:14-236,
// env overrides PUBLIC_IP and IFNAME at lines 204-216), a windowed bandwidth monitor
// (backend/src/misc/bandwidth_monitor.h:8-84) and blocking TCP helpers with deadlines.
#pragma once
#include <chrono>
#include <cstddef>
#include <cstdint>
#include <deque>
#include <mutex>
#include <string>
#include <vector>

namespace stc {

struct IfAddr {
  std::string ifname, ip;
  bool loopback = false, is_private = false;
};
std::vector<IfAddr> list_interfaces();
// PUBLIC_IP wins; else the first address of IFNAME; else first public, then private, then loopback.
std::string pick_local_ip();

// Bytes per second over a sliding window of 1 s split into 100 ms sub-windows; reports the busiest
// sub-window (the reference's choice: it estimates the link rate, not the average load).
class BandwidthMonitor {
 public:
  void add(size_t bytes);
  double peak_bytes_per_s();
  double mean_bytes_per_s();
  uint64_t total_bytes() const { return total_; }

 private:
  void roll(std::chrono::steady_clock::time_point now);
  std::mutex mu_;
  std::deque<std::pair<int64_t, size_t>> windows_;   // (sub-window index, bytes)
  uint64_t total_ = 0;
};

// TCP.  All calls return false / -1 on failure or when the deadline passes; none blocks forever.
int tcp_listen(uint16_t port, uint16_t* bound_port, bool any_port_in_range = false);
int tcp_accept(int listen_fd, int timeout_ms);
int tcp_connect(const std::string& host, uint16_t port, int timeout_ms);
bool send_all(int fd, const void* buf, size_t len, int timeout_ms);
bool recv_all(int fd, void* buf, size_t len, int timeout_ms);
bool wait_readable(int fd, int timeout_ms);
void close_fd(int& fd);

}  // namespace stc
