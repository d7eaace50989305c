#include "proto_wire.h"

#include <cstring>

namespace stc {
namespace pbwire {

namespace {

void varint(Bytes& out, uint64_t v) {
  while (v >= 0x80) {
    out.push_back(static_cast<unsigned char>(v) | 0x80);
    v >>= 7;
  }
  out.push_back(static_cast<unsigned char>(v));
}

void key(Bytes& out, uint32_t field, uint32_t wire) { varint(out, (static_cast<uint64_t>(field) << 3) | wire); }

// proto3 leaves default values (0, 0.0, "", false) out
void put_uint(Bytes& out, uint32_t field, uint64_t v) {
  if (v == 0) return;
  key(out, field, 0);
  varint(out, v);
}

void put_float(Bytes& out, uint32_t field, float v) {
  uint32_t bits;
  std::memcpy(&bits, &v, 4);
  if (bits == 0) return;
  key(out, field, 5);
  for (int i = 0; i < 4; ++i) out.push_back(static_cast<unsigned char>(bits >> (8 * i)));
}

void put_bytes(Bytes& out, uint32_t field, const unsigned char* d, size_t n, bool always) {
  if (n == 0 && !always) return;
  key(out, field, 2);
  varint(out, n);
  out.insert(out.end(), d, d + n);
}

void put_message(Bytes& out, uint32_t field, const Bytes& body) { put_bytes(out, field, body.data(), body.size(), true); }

Bytes train_config(const TrainConfig& c) {
  Bytes b;
  put_uint(b, 1, c.ubatch_size);
  put_uint(b, 2, c.gradient_accumulation);
  put_float(b, 3, static_cast<float>(c.compression_rate));
  return b;
}

Bytes measurements(const TrainMeasurement& m) {
  Bytes b;
  const double v[6] = {m.grad_send_thpt_mbps, m.grad_recv_thpt_mbps, m.fwd_delay_ms, m.bwd_delay_ms, m.bwd_fwd_gap_ms,
                       m.intra_fwd_gap_ms};
  for (uint32_t i = 0; i < 6; ++i) put_float(b, i + 1, static_cast<float>(v[i]));
  return b;
}

// ---- reading
struct Reader {
  const unsigned char* p;
  const unsigned char* end;
  bool ok = true;

  uint64_t varint() {
    uint64_t v = 0;
    for (int shift = 0; shift <= 63; shift += 7) {
      if (p >= end) { ok = false; return 0; }
      const unsigned char b = *p++;
      v |= static_cast<uint64_t>(b & 0x7F) << shift;
      if (!(b & 0x80)) return v;
    }
    ok = false;
    return 0;
  }
};

// Calls fn(field, wire, value, data, len) for every field; unknown wire types end the message as malformed.
template <typename Fn>
bool each_field(const unsigned char* d, size_t n, Fn fn) {
  Reader r{d, d + n};
  while (r.ok && r.p < r.end) {
    const uint64_t k = r.varint();
    if (!r.ok) return false;
    const uint32_t field = static_cast<uint32_t>(k >> 3), wire = static_cast<uint32_t>(k & 7);
    if (wire == 0) {
      const uint64_t v = r.varint();
      if (!r.ok) return false;
      fn(field, wire, v, nullptr, 0);
    } else if (wire == 5 || wire == 1) {
      const size_t w = wire == 5 ? 4 : 8;
      if (static_cast<size_t>(r.end - r.p) < w) return false;
      uint64_t v = 0;
      for (size_t i = 0; i < w; ++i) v |= static_cast<uint64_t>(r.p[i]) << (8 * i);
      r.p += w;
      fn(field, wire, v, nullptr, 0);
    } else if (wire == 2) {
      const uint64_t len = r.varint();
      if (!r.ok || static_cast<uint64_t>(r.end - r.p) < len) return false;
      fn(field, wire, 0, r.p, static_cast<size_t>(len));
      r.p += len;
    } else {
      return false;
    }
  }
  return r.ok;
}

float as_float(uint64_t bits) {
  const uint32_t b = static_cast<uint32_t>(bits);
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}

bool parse_train_config(const unsigned char* d, size_t n, TrainConfig* c) {
  *c = TrainConfig{0, 0, 0.0};
  return each_field(d, n, [c](uint32_t f, uint32_t w, uint64_t v, const unsigned char*, size_t) {
    if (f == 1 && w == 0) c->ubatch_size = static_cast<uint32_t>(v);
    else if (f == 2 && w == 0) c->gradient_accumulation = static_cast<uint32_t>(v);
    else if (f == 3 && w == 5) c->compression_rate = as_float(v);
  });
}

}  // namespace

Bytes request_plain(uint32_t type) {
  Bytes b;
  put_uint(b, 1, type);
  return b;
}

Bytes request_local_init(const LocalTelemetryInit& init) {
  Bytes m;
  put_uint(m, 1, init.gpu_id);
  put_uint(m, 2, init.rank);
  const size_t n = strnlen(init.gpu_name, sizeof(init.gpu_name));
  put_bytes(m, 3, reinterpret_cast<const unsigned char*>(init.gpu_name), n, false);
  put_uint(m, 4, init.local_rank);
  Bytes b;
  put_uint(b, 1, kReqLocalInit);
  put_message(b, 3, m);
  return b;
}

Bytes request_telemetry(const LocalTelemetry& t, uint32_t message_id) {
  Bytes m;
  put_uint(m, 1, t.gpu_id);
  put_uint(m, 2, message_id);
  put_uint(m, 3, t.uiter);
  put_message(m, 4, train_config(t.config));
  put_message(m, 5, measurements(t.measurement));
  Bytes b;
  put_uint(b, 1, kReqLocalTelemetry);
  put_message(b, 4, m);
  return b;
}

Bytes request_global_init(uint32_t num_nodes, uint32_t num_gpus, const std::vector<uint64_t>& param_counts, bool grad_fp16,
                          bool grad_idx_u16) {
  Bytes packed;
  for (uint64_t c : param_counts) varint(packed, c);
  Bytes m;
  put_uint(m, 1, num_nodes);
  put_uint(m, 2, num_gpus);
  put_bytes(m, 3, packed.data(), packed.size(), false);      // repeated uint32, packed as proto3 writes it
  put_uint(m, 4, grad_fp16 ? 1 : 0);
  put_uint(m, 5, grad_idx_u16 ? 1 : 0);
  Bytes b;
  put_uint(b, 1, kReqGlobalInit);
  put_message(b, 2, m);
  return b;
}

bool parse_response(const Bytes& body, uint32_t* type, bool* has_instruction, Instruction* ins) {
  *type = kRespInvalid;
  *has_instruction = false;
  const unsigned char* idata = nullptr;
  size_t ilen = 0;
  bool seen = false;
  if (!each_field(body.data(), body.size(), [&](uint32_t f, uint32_t w, uint64_t v, const unsigned char* d, size_t n) {
        if (f == 1 && w == 0) *type = static_cast<uint32_t>(v);
        else if (f == 2 && w == 2) { idata = d; ilen = n; seen = true; }
      }))
    return false;
  if (*type != kRespInstruction || !seen) return true;
  bool valid = false, cfg_ok = true;
  Instruction out{};
  if (!each_field(idata, ilen, [&](uint32_t f, uint32_t w, uint64_t v, const unsigned char* d, size_t n) {
        if (f == 3 && w == 0) out.iter_effective_since = v;
        else if (f == 4 && w == 0) valid = v != 0;
        else if (f == 5 && w == 2) cfg_ok = parse_train_config(d, n, &out.config);
      }) || !cfg_ok)
    return false;
  if (valid) {
    *ins = out;
    *has_instruction = true;
  }
  return true;
}

}  // namespace pbwire
}  // namespace stc
