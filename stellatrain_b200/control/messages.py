"""Telemetry wire format shared with the native client (``csrc/telemetry/telemetry.h``).

Message set of the reference's protobuf schema (backend/src/proto/message.proto:5-88): TrainConfig,
Measurements, LocalTelemetryInit, Telemetry, GlobalTelemetryInit, Instruction, inside typed requests and
responses.  ``protoc`` is not available where this runs, so the layout is fixed little-endian behind a
12-byte frame header ``<magic u32><type u32><payload_len u32>``.
"""
from __future__ import annotations

import socket
import struct
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

MAGIC = 0x31545453  # "STT1"
LOCAL_INIT, LOCAL, GLOBAL_INIT, INIT, TERMINATE = 1, 2, 3, 4, 5
OK, INSTRUCTION = 100, 101

_FRAME = struct.Struct("<III")
_TRAIN_CONFIG = struct.Struct("<IId")
_MEASUREMENT = struct.Struct("<6d")
_LOCAL_INIT = struct.Struct("<III64s")
_LOCAL = struct.Struct("<IQ" + "IId" + "6d")
_INSTRUCTION = struct.Struct("<Q" + "IId")


@dataclass
class TrainConfig:
    ubatch_size: int = 0
    gradient_accumulation: int = 1
    compression_rate: float = 0.99


@dataclass
class Measurement:
    grad_send_thpt_mbps: float = 0.0
    grad_recv_thpt_mbps: float = 0.0
    fwd_delay_ms: float = 0.0
    bwd_delay_ms: float = 0.0
    bwd_fwd_gap_ms: float = 0.0
    intra_fwd_gap_ms: float = 0.0

    def as_tuple(self) -> Tuple[float, ...]:
        return (self.grad_send_thpt_mbps, self.grad_recv_thpt_mbps, self.fwd_delay_ms, self.bwd_delay_ms,
                self.bwd_fwd_gap_ms, self.intra_fwd_gap_ms)


@dataclass
class LocalInit:
    gpu_id: int
    rank: int
    local_rank: int
    gpu_name: str


@dataclass
class LocalTelemetry:
    gpu_id: int
    uiter: int
    config: TrainConfig
    measurement: Measurement


@dataclass
class GlobalInit:
    num_nodes: int
    num_gpus: int
    grad_fp16: bool
    grad_idx_u16: bool
    param_counts: List[int] = field(default_factory=list)


@dataclass
class Instruction:
    iter_effective_since: int
    config: TrainConfig


def pack_frame(mtype: int, payload: bytes = b"") -> bytes:
    return _FRAME.pack(MAGIC, mtype, len(payload)) + payload


def pack_local_init(m: LocalInit) -> bytes:
    return pack_frame(LOCAL_INIT, _LOCAL_INIT.pack(m.gpu_id, m.rank, m.local_rank, m.gpu_name.encode()[:63]))


def pack_local(m: LocalTelemetry) -> bytes:
    c = m.config
    return pack_frame(LOCAL, _LOCAL.pack(m.gpu_id, m.uiter, c.ubatch_size, c.gradient_accumulation, c.compression_rate,
                                         *m.measurement.as_tuple()))


def pack_global_init(m: GlobalInit) -> bytes:
    body = struct.pack("<IIBBHI", m.num_nodes, m.num_gpus, int(m.grad_fp16), int(m.grad_idx_u16), 0, len(m.param_counts))
    body += struct.pack(f"<{len(m.param_counts)}Q", *m.param_counts)
    return pack_frame(GLOBAL_INIT, body)


def pack_instruction(m: Instruction) -> bytes:
    c = m.config
    return pack_frame(INSTRUCTION, _INSTRUCTION.pack(m.iter_effective_since, c.ubatch_size, c.gradient_accumulation,
                                                     c.compression_rate))


def parse(mtype: int, payload: bytes):
    if mtype == LOCAL_INIT:
        gid, rank, lrank, name = _LOCAL_INIT.unpack(payload)
        return LocalInit(gid, rank, lrank, name.split(b"\0", 1)[0].decode(errors="replace"))
    if mtype == LOCAL:
        v = _LOCAL.unpack(payload)
        return LocalTelemetry(v[0], v[1], TrainConfig(v[2], v[3], v[4]), Measurement(*v[5:11]))
    if mtype == GLOBAL_INIT:
        nn, ng, f16, u16, _, n = struct.unpack_from("<IIBBHI", payload, 0)
        counts = list(struct.unpack_from(f"<{n}Q", payload, 16))
        return GlobalInit(nn, ng, bool(f16), bool(u16), counts)
    if mtype == INSTRUCTION:
        v = _INSTRUCTION.unpack(payload)
        return Instruction(v[0], TrainConfig(v[1], v[2], v[3]))
    return None


def recv_exact(sock: socket.socket, n: int) -> Optional[bytes]:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            return None
        buf += chunk
    return bytes(buf)


def recv_frame(sock: socket.socket) -> Optional[Tuple[int, bytes]]:
    head = recv_exact(sock, _FRAME.size)
    if head is None:
        return None
    magic, mtype, n = _FRAME.unpack(head)
    if magic != MAGIC or n > (1 << 24):
        raise ValueError("malformed telemetry frame")
    payload = recv_exact(sock, n) if n else b""
    if payload is None:
        return None
    return mtype, payload
