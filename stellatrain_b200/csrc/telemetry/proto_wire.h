// The reference's telemetry schema in protocol-buffers wire format (backend/src/proto/message.proto:5-88), written and
// read by hand: varints, 32-bit floats and length-delimited fields are all the schema needs, and no protoc exists on the
// target machines.  Same bytes as stellatrain_b200/control/protobuf_wire.py, which is checked against the protobuf run
// time.  Used by the ZeroMQ transport of TelemetryClient / TelemetryServer (telemetry.h).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "telemetry.h"

namespace stc {
namespace pbwire {

using Bytes = std::vector<unsigned char>;

// Request.Type / Response.Type (message.proto:58-65, 77-81)
enum : uint32_t { kReqInit = 1, kReqGlobalInit = 2, kReqLocalInit = 3, kReqLocalTelemetry = 4, kReqTerminate = 5 };
enum : uint32_t { kRespInvalid = 0, kRespOk = 1, kRespInstruction = 2 };

Bytes request_plain(uint32_t type);                                        // INIT, TERMINATE
Bytes request_local_init(const LocalTelemetryInit& init);
Bytes request_telemetry(const LocalTelemetry& t, uint32_t message_id);
Bytes request_global_init(uint32_t num_nodes, uint32_t num_gpus, const std::vector<uint64_t>& param_counts, bool grad_fp16,
                          bool grad_idx_u16);

// Returns false on a malformed message.  *has_instruction: the reply carries an instruction marked valid.
bool parse_response(const Bytes& body, uint32_t* type, bool* has_instruction, Instruction* ins);

}  // namespace pbwire
}  // namespace stc
