"""The reference's telemetry schema in protocol-buffers wire format, without ``protoc``.

The reference serialises its control messages with protobuf (backend/src/proto/message.proto:5-88: ``TrainConfig``,
``Measurements``, ``GlobalTelemetryInit``, ``LocalTelemetryInit``, ``Telemetry``, ``Instruction`` inside ``Request``
and ``Response``) and moves them over ZeroMQ REQ/ROUTER sockets (backend/src/engine/telemetry_client.cpp:5-110,
backend/src/engine/batch_rate_alloc.py:283-321).  This package's own transport uses fixed little-endian frames
(``messages.py``); this module states the same eight messages in proto3 wire format, so that the controller can
also answer a client built from the reference, and this package's hooks can report to the reference's controller
(``zmq_endpoint.py``).

Only what the schema needs is implemented: varints (wire type 0), 32-bit floats (wire type 5) and length-delimited
fields (wire type 2: strings, sub-messages, packed ``repeated uint32``).  Unknown fields are skipped, as the format
asks; proto3 default values are not written.
"""
from __future__ import annotations

import struct
from typing import Dict, Iterator, List, Tuple

from . import messages as M

# Request.Type / Response.Type (message.proto:58-65, 77-81)
REQ_INVALID, REQ_INIT, REQ_GLOBAL_TELEMETRY_INIT, REQ_LOCAL_TELEMETRY_INIT, REQ_LOCAL_TELEMETRY, REQ_TERMINATE = range(6)
RESP_INVALID, RESP_OK, RESP_INSTRUCTION = range(3)


# ------------------------------------------------------------------------------------------------ primitives
def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    shift = result = 0
    while True:
        if pos >= len(buf) or shift > 63:
            raise ValueError("truncated or oversized varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7


def _key(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def _uint(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(int(v)) if v else b""


def _float(field: int, v: float) -> bytes:
    raw = struct.pack("<f", float(v))
    return _key(field, 5) + raw if raw != b"\0\0\0\0" else b""


def _bytes(field: int, v: bytes, always: bool = False) -> bytes:
    return _key(field, 2) + _varint(len(v)) + v if (v or always) else b""


def fields(buf: bytes) -> Iterator[Tuple[int, int, object]]:
    """(field number, wire type, value) of every field of a serialised message; value is an int (wire types 0, 1, 5
    as raw little-endian integers) or bytes (wire type 2)."""
    pos = 0
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, pos = _read_varint(buf, pos)
        elif wire == 1:
            if pos + 8 > len(buf):
                raise ValueError("truncated 64-bit field")
            v, pos = int.from_bytes(buf[pos:pos + 8], "little"), pos + 8
        elif wire == 2:
            n, pos = _read_varint(buf, pos)
            if pos + n > len(buf):
                raise ValueError("truncated length-delimited field")
            v, pos = bytes(buf[pos:pos + n]), pos + n
        elif wire == 5:
            if pos + 4 > len(buf):
                raise ValueError("truncated 32-bit field")
            v, pos = int.from_bytes(buf[pos:pos + 4], "little"), pos + 4
        else:
            raise ValueError(f"unsupported wire type {wire}")
        yield field, wire, v


def _as_float(raw: int) -> float:
    return struct.unpack("<f", struct.pack("<I", raw & 0xFFFFFFFF))[0]


def _collect(buf: bytes) -> Dict[int, List[Tuple[int, object]]]:
    out: Dict[int, List[Tuple[int, object]]] = {}
    for f, w, v in fields(buf):
        out.setdefault(f, []).append((w, v))
    return out


def _last(d: Dict[int, List[Tuple[int, object]]], field: int, default=0):
    return d[field][-1][1] if field in d else default


# ------------------------------------------------------------------------------------------------ messages
def encode_train_config(c: M.TrainConfig) -> bytes:
    return _uint(1, c.ubatch_size) + _uint(2, c.gradient_accumulation) + _float(3, c.compression_rate)


def decode_train_config(buf: bytes) -> M.TrainConfig:
    d = _collect(buf)
    return M.TrainConfig(int(_last(d, 1)), int(_last(d, 2)), _as_float(int(_last(d, 3))))


def encode_measurements(m: M.Measurement) -> bytes:
    return b"".join(_float(i + 1, v) for i, v in enumerate(m.as_tuple()))


def decode_measurements(buf: bytes) -> M.Measurement:
    d = _collect(buf)
    return M.Measurement(*[_as_float(int(_last(d, i))) for i in range(1, 7)])


def encode_global_init(g: M.GlobalInit) -> bytes:
    packed = b"".join(_varint(int(n)) for n in g.param_counts)
    return (_uint(1, g.num_nodes) + _uint(2, g.num_gpus) + _bytes(3, packed) + _uint(4, int(g.grad_fp16)) +
            _uint(5, int(g.grad_idx_u16)))


def decode_global_init(buf: bytes) -> M.GlobalInit:
    d = _collect(buf)
    counts: List[int] = []
    for wire, v in d.get(3, []):
        if wire == 2:                      # packed (what proto3 writes)
            pos = 0
            while pos < len(v):
                n, pos = _read_varint(v, pos)
                counts.append(n)
        else:                              # one element per field (allowed on the wire)
            counts.append(int(v))
    return M.GlobalInit(int(_last(d, 1)), int(_last(d, 2)), bool(_last(d, 4)), bool(_last(d, 5)), counts)


def encode_local_init(m: M.LocalInit, local_world_size: int = 0, max_batch_size: int = 0) -> bytes:
    return (_uint(1, m.gpu_id) + _uint(2, m.rank) + _bytes(3, m.gpu_name.encode()) + _uint(4, m.local_rank) +
            _uint(5, local_world_size) + _uint(6, max_batch_size))


def decode_local_init(buf: bytes) -> Tuple[M.LocalInit, int, int]:
    """(init, local_world_size, max_batch_size)."""
    d = _collect(buf)
    name = _last(d, 3, b"")
    init = M.LocalInit(int(_last(d, 1)), int(_last(d, 2)), int(_last(d, 4)), bytes(name).decode(errors="replace"))
    return init, int(_last(d, 5)), int(_last(d, 6))


def encode_telemetry(t: M.LocalTelemetry, message_id: int = 0) -> bytes:
    return (_uint(1, t.gpu_id) + _uint(2, message_id) + _uint(3, t.uiter) + _bytes(4, encode_train_config(t.config), True) +
            _bytes(5, encode_measurements(t.measurement), True))


def decode_telemetry(buf: bytes) -> Tuple[M.LocalTelemetry, int]:
    """(telemetry, message_id)."""
    d = _collect(buf)
    cfg = decode_train_config(bytes(_last(d, 4, b"")))
    meas = decode_measurements(bytes(_last(d, 5, b"")))
    return M.LocalTelemetry(int(_last(d, 1)), int(_last(d, 3)), cfg, meas), int(_last(d, 2))


def encode_instruction(i: M.Instruction, client_id: int = 0, message_id: int = 0, valid: bool = True) -> bytes:
    return (_uint(1, client_id) + _uint(2, message_id) + _uint(3, i.iter_effective_since) + _uint(4, int(valid)) +
            _bytes(5, encode_train_config(i.config), True))


def decode_instruction(buf: bytes) -> Tuple[M.Instruction, bool]:
    """(instruction, valid)."""
    d = _collect(buf)
    return M.Instruction(int(_last(d, 3)), decode_train_config(bytes(_last(d, 5, b"")))), bool(_last(d, 4))


# ------------------------------------------------------------------------------------------------ envelopes
def encode_request(rtype: int, payload=None, **kw) -> bytes:
    """``Request{type, oneof payload}``: payload is a GlobalInit, LocalInit or LocalTelemetry matching ``rtype``."""
    out = _uint(1, rtype)
    if rtype == REQ_GLOBAL_TELEMETRY_INIT:
        out += _bytes(2, encode_global_init(payload), True)
    elif rtype == REQ_LOCAL_TELEMETRY_INIT:
        out += _bytes(3, encode_local_init(payload, **kw), True)
    elif rtype == REQ_LOCAL_TELEMETRY:
        out += _bytes(4, encode_telemetry(payload, **kw), True)
    return out


def decode_request(buf: bytes) -> Tuple[int, object]:
    """(type, payload): payload is a GlobalInit, a LocalInit, a LocalTelemetry, or None."""
    d = _collect(buf)
    rtype = int(_last(d, 1))
    if rtype == REQ_GLOBAL_TELEMETRY_INIT and 2 in d:
        return rtype, decode_global_init(bytes(_last(d, 2)))
    if rtype == REQ_LOCAL_TELEMETRY_INIT and 3 in d:
        return rtype, decode_local_init(bytes(_last(d, 3)))[0]
    if rtype == REQ_LOCAL_TELEMETRY and 4 in d:
        return rtype, decode_telemetry(bytes(_last(d, 4)))[0]
    return rtype, None


def encode_response(rtype: int, instruction: M.Instruction = None, client_id: int = 0) -> bytes:
    out = _uint(1, rtype)
    if rtype == RESP_INSTRUCTION and instruction is not None:
        out += _bytes(2, encode_instruction(instruction, client_id=client_id), True)
    return out


def decode_response(buf: bytes) -> Tuple[int, object]:
    """(type, Instruction or None); an instruction that is not marked valid counts as none."""
    d = _collect(buf)
    rtype = int(_last(d, 1))
    if rtype == RESP_INSTRUCTION and 2 in d:
        inst, valid = decode_instruction(bytes(_last(d, 2)))
        return rtype, inst if valid else None
    return rtype, None
