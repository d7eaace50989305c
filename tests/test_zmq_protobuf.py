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


def _schema_classes():
    """The reference's schema (backend/src/proto/message.proto:5-88) stated as a descriptor for the protobuf run time,
    so that the real library serialises and parses next to the hand-written codec.  No protoc involved."""
    pb2 = pytest.importorskip("google.protobuf.descriptor_pb2")
    from google.protobuf import descriptor_pool, message_factory

    F = pb2.FieldDescriptorProto
    fd = pb2.FileDescriptorProto(name="fasterdp_message_test.proto", package="fasterdp_test", syntax="proto3")

    def msg(name, fields, enums=()):
        m = fd.message_type.add(name=name)
        for ename, values in enums:
            e = m.enum_type.add(name=ename)
            for i, v in enumerate(values):
                e.value.add(name=v, number=i)
        for fname, number, ftype, extra in fields:
            f = m.field.add(name=fname, number=number, type=ftype, label=extra.get("label", F.LABEL_OPTIONAL))
            if "type_name" in extra:
                f.type_name = extra["type_name"]
            if "oneof" in extra:
                if not m.oneof_decl:
                    m.oneof_decl.add(name="payload")
                f.oneof_index = 0
        return m

    u32, f32, boolean, string, message, enum = F.TYPE_UINT32, F.TYPE_FLOAT, F.TYPE_BOOL, F.TYPE_STRING, F.TYPE_MESSAGE, F.TYPE_ENUM
    pkg = ".fasterdp_test."
    msg("TrainConfig", [("ubatch_size", 1, u32, {}), ("gradient_accumulation", 2, u32, {}), ("compression_rate", 3, f32, {})])
    msg("Measurements", [(n, i + 1, f32, {}) for i, n in enumerate(
        ["grad_send_thpt_mbps", "grad_recv_thpt_mbps", "fwd_delay_ms", "bwd_delay_ms", "bwd_fwd_gap_ms", "intra_fwd_gap_ms"])])
    msg("GlobalTelemetryInit", [("num_nodes", 1, u32, {}), ("num_gpus", 2, u32, {}),
                                ("param_counts", 3, u32, {"label": F.LABEL_REPEATED}), ("grad_fp16", 4, boolean, {}),
                                ("grad_idx_u16", 5, boolean, {})])
    msg("LocalTelemetryInit", [("client_id", 1, u32, {}), ("rank", 2, u32, {}), ("gpu_name", 3, string, {}),
                               ("local_rank", 4, u32, {}), ("local_world_size", 5, u32, {}), ("max_batch_size", 6, u32, {})])
    msg("Telemetry", [("client_id", 1, u32, {}), ("message_id", 2, u32, {}), ("uiter_count", 3, u32, {}),
                      ("config", 4, message, {"type_name": pkg + "TrainConfig"}),
                      ("measurements", 5, message, {"type_name": pkg + "Measurements"})])
    msg("Instruction", [("client_id", 1, u32, {}), ("message_id", 2, u32, {}), ("effective_since_uiter", 3, u32, {}),
                        ("valid", 4, boolean, {}), ("config", 5, message, {"type_name": pkg + "TrainConfig"})])
    msg("Request", [("type", 1, enum, {"type_name": pkg + "Request.Type"}),
                    ("global_telemetry_init", 2, message, {"type_name": pkg + "GlobalTelemetryInit", "oneof": True}),
                    ("local_telemetry_init", 3, message, {"type_name": pkg + "LocalTelemetryInit", "oneof": True}),
                    ("telemetry", 4, message, {"type_name": pkg + "Telemetry", "oneof": True})],
        enums=[("Type", ["INVALID", "INIT", "GLOBAL_TELEMETRY_INIT", "LOCAL_TELEMETRY_INIT", "LOCAL_TELEMETRY", "TERMINATE"])])
    msg("Response", [("type", 1, enum, {"type_name": pkg + "Response.Type"}),
                     ("instruction", 2, message, {"type_name": pkg + "Instruction", "oneof": True})],
        enums=[("Type", ["INVALID", "OK", "INSTRUCTION"])])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return {n: message_factory.GetMessageClass(pool.FindMessageTypeByName("fasterdp_test." + n))
            for n in ("Request", "Response", "TrainConfig")}


def test_codec_agrees_with_the_protobuf_library_on_the_references_schema():
    """Every message the codec writes parses with the protobuf run time into the same fields, and what the run time
    serialises (what a process built from the reference sends) is read back by the codec."""
    cls = _schema_classes()
    Request, Response = cls["Request"], cls["Response"]

    # ours -> library
    t = M.LocalTelemetry(5, 1234, M.TrainConfig(48, 2, 0.95), M.Measurement(100.5, 99.25, 7.0, 14.5, 0.75, 0.125))
    r = Request.FromString(PB.encode_request(PB.REQ_LOCAL_TELEMETRY, t, message_id=9))
    assert r.type == 4 and r.WhichOneof("payload") == "telemetry"
    assert (r.telemetry.client_id, r.telemetry.message_id, r.telemetry.uiter_count) == (5, 9, 1234)
    assert (r.telemetry.config.ubatch_size, r.telemetry.config.gradient_accumulation) == (48, 2)
    assert r.telemetry.config.compression_rate == pytest.approx(0.95, rel=1e-6)
    assert r.telemetry.measurements.bwd_delay_ms == 14.5 and r.telemetry.measurements.intra_fwd_gap_ms == 0.125
    g = M.GlobalInit(2, 8, False, True, [9408, 64, 2359296, 100])
    r = Request.FromString(PB.encode_request(PB.REQ_GLOBAL_TELEMETRY_INIT, g))
    assert r.type == 2 and list(r.global_telemetry_init.param_counts) == g.param_counts
    assert (r.global_telemetry_init.num_nodes, r.global_telemetry_init.num_gpus) == (2, 8)
    assert r.global_telemetry_init.grad_idx_u16 and not r.global_telemetry_init.grad_fp16
    r = Request.FromString(PB.encode_request(PB.REQ_LOCAL_TELEMETRY_INIT, M.LocalInit(3, 1, 2, "NVIDIA B200"),
                                             local_world_size=4, max_batch_size=64))
    li = r.local_telemetry_init
    assert (li.client_id, li.rank, li.gpu_name, li.local_rank, li.local_world_size, li.max_batch_size) == (3, 1, "NVIDIA B200", 2, 4, 64)
    resp = Response.FromString(PB.encode_response(PB.RESP_INSTRUCTION, M.Instruction(77, M.TrainConfig(24, 1, 0.875)), client_id=3))
    assert resp.type == 2 and resp.instruction.valid and resp.instruction.client_id == 3
    assert resp.instruction.effective_since_uiter == 77 and resp.instruction.config.compression_rate == 0.875
    assert Request.FromString(PB.encode_request(PB.REQ_TERMINATE)).type == 5

    # library -> ours; where no default value is involved the bytes are the same, too
    lib = Request(type=4)
    lib.telemetry.client_id, lib.telemetry.message_id, lib.telemetry.uiter_count = 5, 9, 1234
    lib.telemetry.config.ubatch_size, lib.telemetry.config.gradient_accumulation, lib.telemetry.config.compression_rate = 48, 2, 0.95
    for name, v in zip(["grad_send_thpt_mbps", "grad_recv_thpt_mbps", "fwd_delay_ms", "bwd_delay_ms", "bwd_fwd_gap_ms",
                        "intra_fwd_gap_ms"], t.measurement.as_tuple()):
        setattr(lib.telemetry.measurements, name, v)
    assert lib.SerializeToString() == PB.encode_request(PB.REQ_LOCAL_TELEMETRY, t, message_id=9)
    rtype, got = PB.decode_request(lib.SerializeToString())
    assert rtype == PB.REQ_LOCAL_TELEMETRY and got.uiter == 1234 and got.measurement.as_tuple() == t.measurement.as_tuple()
    lib = Request(type=2)
    lib.global_telemetry_init.num_nodes, lib.global_telemetry_init.num_gpus, lib.global_telemetry_init.grad_idx_u16 = 2, 8, True
    lib.global_telemetry_init.param_counts.extend(g.param_counts)
    assert lib.SerializeToString() == PB.encode_request(PB.REQ_GLOBAL_TELEMETRY_INIT, g)
    assert PB.decode_request(lib.SerializeToString()) == (PB.REQ_GLOBAL_TELEMETRY_INIT, g)
    lib = Response(type=2)
    lib.instruction.effective_since_uiter, lib.instruction.valid = 77, True
    lib.instruction.config.ubatch_size, lib.instruction.config.gradient_accumulation, lib.instruction.config.compression_rate = 24, 1, 0.875
    rtype, inst = PB.decode_response(lib.SerializeToString())
    assert rtype == PB.RESP_INSTRUCTION and inst.iter_effective_since == 77 and inst.config.ubatch_size == 24
    lib.instruction.valid = False
    assert PB.decode_response(lib.SerializeToString()) == (PB.RESP_INSTRUCTION, None)     # not marked valid: counts as none


def test_native_client_and_server_speak_protobuf_over_zeromq(monkeypatch):
    """The C++ telemetry client and server shim on the reference's transport: uri "zmq://..." makes them send protobuf
    requests over a ZeroMQ REQ socket (libzmq opened at run time), answered here by the controller's ROUTER endpoint."""
    pytest.importorskip("zmq")
    from stellatrain_b200 import cpu_tier
    from stellatrain_b200.control.controller import Controller
    from stellatrain_b200.control.zmq_endpoint import ZmqControllerEndpoint

    lib = cpu_tier.bundled_libzmq()
    if not lib:
        pytest.skip("no libzmq inside pyzmq")
    monkeypatch.setenv("STELLATRAIN_LIBZMQ", lib)
    ext = cpu_tier._load()
    ctl = Controller(port=0, host="127.0.0.1", adapt=False).start()
    ep = ZmqControllerEndpoint(ctl, "tcp://127.0.0.1:0").start()
    got = []
    try:
        uri = f"zmq://127.0.0.1:{ep.port}"
        server = ext.TelemetryServer(uri, False, 3000)
        assert server.send_global_telemetry(1, 2, [1000, 2000, 300000], False, True)
        gi = ctl.global_init
        assert (gi.num_nodes, gi.num_gpus, gi.param_counts, gi.grad_fp16, gi.grad_idx_u16) == (1, 2, [1000, 2000, 300000], False, True)
        clients = [ext.TelemetryClient(uri, g, "NVIDIA B200", 0, g, 3000) for g in range(2)]
        assert sorted(ctl.clients) == [0, 1] and ctl.clients[1].gpu_name == "NVIDIA B200" and ctl.clients[1].local_rank == 1
        ctl.clients[0].pending.put(M.Instruction(40, M.TrainConfig(20, 1, 0.875)))
        for it in range(5):
            for g, c in enumerate(clients):
                c.report(it, ext.TrainConfig(16, 1, 0.99), [300.0, 200.0, 5.0, 10.0 + g, 1.0, 0.0],
                         lambda since, ub, ga, cr, g=g: got.append((g, since, ub, ga, cr)))
        deadline = time.time() + 5.0
        while (ctl.latest_iter < 4 or not got or clients[1].sent() < 5) and time.time() < deadline:
            time.sleep(0.02)
        assert ctl.latest_iter >= 4 and clients[0].alive() and clients[0].sent() == 5
        assert float(ctl.scoreboard.loc[1, "bwd_ms"]) == pytest.approx(11.0)
        assert float(ctl.scoreboard.loc[1, "send_mbps"]) == pytest.approx(300.0)
        assert got == [(0, 40, 20, 1, 0.875)]
        assert server.terminate() and ctl.stop.is_set()
        del clients, server
    finally:
        ep.close()
        ctl.close()


def test_cpu_tier_hook_reports_over_zeromq_when_given_a_zmq_uri():
    """`zmq://` as the controller address of the training hooks: the native client finds pyzmq's libzmq by itself."""
    pytest.importorskip("zmq")
    import torch
    import torch.nn as nn
    import torch.nn.functional as F

    from stellatrain_b200 import cpu_tier
    from stellatrain_b200.control.controller import Controller
    from stellatrain_b200.control.zmq_endpoint import ZmqControllerEndpoint

    if not cpu_tier.bundled_libzmq():
        pytest.skip("no libzmq inside pyzmq")
    ctl = Controller(port=0, host="127.0.0.1", adapt=False).start()
    ep = ZmqControllerEndpoint(ctl, "tcp://127.0.0.1:0").start()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 4))
    eng = cpu_tier.CpuOffloadEngine(model, method="topk", ratio=0.9, optimizer="sgd", optimizer_options={"lr": 0.05},
                                    staleness=1, data_bytes=4 << 20, workers=2)
    try:
        hook = cpu_tier.CpuTierTelemetry(eng, f"zmq://127.0.0.1:{ep.port}", batch_size=8)
        for i in range(6):
            x, y = torch.randn(8, 16), torch.randint(0, 4, (8,))
            with hook.step() as marker:
                loss = F.cross_entropy(model(x), y)
                marker.backward_begins()
                loss.backward()
        deadline = time.time() + 5.0
        while ctl.latest_iter < 5 and time.time() < deadline:
            time.sleep(0.02)
        assert ctl.latest_iter >= 5 and 0 in ctl.clients
        assert float(ctl.scoreboard.loc[0, "bwd_ms"]) > 0.0
        hook.client = None
    finally:
        eng.synchronize()
        eng.close()
        ep.close()
        ctl.close()
