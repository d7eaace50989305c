"""The reference's control-plane wire format: protobuf messages (hand-coded codec) over ZeroMQ REQ/ROUTER."""
import struct
import time

import pytest

from stellatrain_b200.control import messages as M
from stellatrain_b200.control import protobuf_wire as PB


def test_train_config_bytes_are_the_proto3_encoding():
    # field 1 varint 32, field 2 varint 1, field 3 fixed32 float 0.99: written out by hand from the format's rules
    want = bytes([0x08, 0x20, 0x10, 0x01, 0x1D]) + struct.pack("<f", 0.99)
    assert PB.encode_train_config(M.TrainConfig(32, 1, 0.99)) == want
    back = PB.decode_train_config(want)
    assert (back.ubatch_size, back.gradient_accumulation) == (32, 1) and back.compression_rate == pytest.approx(0.99, rel=1e-6)
    # proto3 leaves default values out; multi-byte varints
    assert PB.encode_train_config(M.TrainConfig(0, 0, 0.0)) == b""
    assert PB.encode_train_config(M.TrainConfig(300, 0, 0.0)) == bytes([0x08, 0xAC, 0x02])


def test_request_and_response_envelopes_round_trip():
    t = M.LocalTelemetry(5, 1234, M.TrainConfig(48, 2, 0.95), M.Measurement(100.5, 99.25, 7.0, 14.5, 0.75, 0.125))
    body = PB.encode_request(PB.REQ_LOCAL_TELEMETRY, t, message_id=9)
    assert body[:2] == bytes([0x08, 0x04]) and body[2] == 0x22          # type = LOCAL_TELEMETRY, then field 4, length-delimited
    rtype, got = PB.decode_request(body)
    assert rtype == PB.REQ_LOCAL_TELEMETRY and got.gpu_id == 5 and got.uiter == 1234
    assert got.config.ubatch_size == 48 and got.config.gradient_accumulation == 2
    assert got.measurement.as_tuple() == (100.5, 99.25, 7.0, 14.5, 0.75, 0.125)

    g = M.GlobalInit(2, 8, False, True, [9408, 64, 2359296, 100])
    rtype, got = PB.decode_request(PB.encode_request(PB.REQ_GLOBAL_TELEMETRY_INIT, g))
    assert rtype == PB.REQ_GLOBAL_TELEMETRY_INIT and got == g

    li = M.LocalInit(3, 1, 2, "NVIDIA B200")
    rtype, got = PB.decode_request(PB.encode_request(PB.REQ_LOCAL_TELEMETRY_INIT, li, local_world_size=4, max_batch_size=64))
    assert rtype == PB.REQ_LOCAL_TELEMETRY_INIT and got == li

    inst = M.Instruction(77, M.TrainConfig(24, 1, 0.875))
    rtype, got = PB.decode_response(PB.encode_response(PB.RESP_INSTRUCTION, inst, client_id=3))
    assert rtype == PB.RESP_INSTRUCTION and got.iter_effective_since == 77 and got.config.ubatch_size == 24
    assert PB.decode_response(PB.encode_response(PB.RESP_OK)) == (PB.RESP_OK, None)
    assert PB.decode_request(PB.encode_request(PB.REQ_TERMINATE)) == (PB.REQ_TERMINATE, None)


def test_decoder_skips_unknown_fields_and_rejects_truncation():
    body = PB.encode_train_config(M.TrainConfig(7, 1, 0.5)) + bytes([0x78, 0x05]) + bytes([0x82, 0x01, 0x02, 0xAA, 0xBB])
    c = PB.decode_train_config(body)       # field 15 (varint) and field 16 (bytes) are not in the schema
    assert c.ubatch_size == 7 and c.compression_rate == 0.5
    with pytest.raises(ValueError):
        list(PB.fields(bytes([0x0A, 0x05, 0x01])))      # announces 5 bytes, carries 1
    with pytest.raises(ValueError):
        list(PB.fields(bytes([0x08, 0x80])))            # varint without its last byte


def test_controller_answers_protobuf_clients_over_zeromq():
    pytest.importorskip("zmq")
    from stellatrain_b200.control.controller import Controller
    from stellatrain_b200.control.zmq_endpoint import (ZmqControllerEndpoint, ZmqTelemetryClient, send_global_init,
                                                       send_terminate)

    ctl = Controller(port=0, host="127.0.0.1", adapt=False).start()
    ep = ZmqControllerEndpoint(ctl, "tcp://127.0.0.1:0").start()
    got = []
    try:
        assert send_global_init(ep.uri, M.GlobalInit(1, 2, False, False, [1000, 2000]))
        assert ctl.optimizer is not None and ctl.optimizer.num_gpus == 2
        clients = [ZmqTelemetryClient(ep.uri, gid, "NVIDIA B200", 0, gid) for gid in (0, 1)]
        assert sorted(ctl.clients) == [0, 1] and ctl.clients[1].gpu_name == "NVIDIA B200"
        ctl.clients[1].pending.put(M.Instruction(40, M.TrainConfig(20, 1, 0.9)))
        for it in range(6):
            for c in clients:
                c.report(it, M.TrainConfig(16, 1, 0.99), M.Measurement(10.0, 10.0, 5.0, 10.0, 1.0, 0.0),
                         lambda since, cfg, who=c.gpu_id: got.append((who, since, cfg.ubatch_size, round(cfg.compression_rate, 4))))
        deadline = time.time() + 5.0
        while (ctl.latest_iter < 5 or not got) and time.time() < deadline:
            time.sleep(0.02)
        assert ctl.latest_iter >= 5 and len(ctl.scoreboard) == 2
        assert float(ctl.scoreboard.loc[0, "bwd_ms"]) == pytest.approx(10.0)
        assert got == [(1, 40, 20, 0.9)]                   # the queued instruction went to client 1, once
        for c in clients:
            c.close()
        assert send_terminate(ep.uri) and ctl.stop.is_set()
    finally:
        ep.close()
        ctl.close()
