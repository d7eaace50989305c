// ZeroMQ PUSH/PULL link for the gradient ring, the reference's data transport
// (backend/src/engine/comm_manager.cpp:369-477: one PULL socket bound to a port of its own and one PUSH socket
// connected to the ring successor, both with a high-water mark of 0; 722-766 and 833-870: gradient messages as
// multipart messages).  No ZeroMQ headers exist on the target machines, so the library is opened at run time
// (dlopen: the path named by STELLATRAIN_LIBZMQ, a path handed in by the caller such as the libzmq that ships inside
// pyzmq, or the system's libzmq.so.5) and the handful of C entry points used here are declared by hand.
//
// Message layout: [key][flags: 1 byte][payload], three frames.  The payload is this package's sparse payload
// (comm_manager.h: encode_sparse), which extends the reference's (index array, value array) pair with whole blocks
// and 16-bit values; the reference's own layout is four frames, [key][flag][indices][values].
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace stc {

class ZmqLibrary {
 public:
  // Loads the library once per process; `hint` may name a file.  Returns false (and a reason) when none can be loaded.
  static bool load(const std::string& hint, std::string* why);
  static bool loaded();
};

class ZmqLink {
 public:
  ZmqLink();
  ~ZmqLink();
  ZmqLink(const ZmqLink&) = delete;
  ZmqLink& operator=(const ZmqLink&) = delete;

  // PULL side: binds to an ephemeral port of `ip`, returns the port (0 on failure).
  uint16_t bind_pull(const std::string& ip);
  // PUSH side: connects to the successor's PULL socket.
  bool connect_push(const std::string& ip, uint16_t port);

  bool send(const std::string& key, uint8_t flags, const unsigned char* payload, size_t len, int timeout_ms);
  // false on time-out (nothing arrived within timeout_ms) or on a malformed message (*malformed set)
  bool recv(std::string* key, uint8_t* flags, std::vector<unsigned char>* payload, int timeout_ms, bool* malformed);
  void close();

 private:
  void* ctx_ = nullptr;
  void* push_ = nullptr;
  void* pull_ = nullptr;
};

// REQ socket for the control plane (the reference's telemetry client and server talk to the controller's ROUTER socket
// this way, backend/src/engine/telemetry_client.cpp:5-37): one request, one reply.  A request that got no reply in time
// leaves a REQ socket unusable (strict alternation), so the caller gives the connection up after a failure.
class ZmqReq {
 public:
  ZmqReq();
  ~ZmqReq();
  ZmqReq(const ZmqReq&) = delete;
  ZmqReq& operator=(const ZmqReq&) = delete;
  bool connect(const std::string& endpoint);      // "tcp://host:port"
  bool request(const std::vector<unsigned char>& body, std::vector<unsigned char>* reply, int timeout_ms);
  void close();

 private:
  void* ctx_ = nullptr;
  void* sock_ = nullptr;
};

}  // namespace stc
