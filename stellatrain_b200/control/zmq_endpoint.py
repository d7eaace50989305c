"""ZeroMQ + protobuf front ends of the control plane: the reference's own transport and wire format.

The reference's clients are ZeroMQ REQ sockets that send protobuf ``Request`` messages to a ROUTER socket on
``tcp://*:5556`` and read a ``Response`` back, which is either ``OK`` or an ``INSTRUCTION`` that was waiting for that
client (backend/src/engine/telemetry_client.cpp:5-110, backend/src/engine/telemetry_server.cpp:10-96,
backend/src/engine/batch_rate_alloc.py:283-321).  Two classes speak that protocol:

* ``ZmqControllerEndpoint`` puts a ROUTER socket in front of this package's ``Controller``, next to its framed-TCP
  port, so that a telemetry client or server built from the reference can drive it;
* ``ZmqTelemetryClient`` is the client side (LOCAL_TELEMETRY_INIT, then one LOCAL_TELEMETRY per report, instructions
  through a callback) and ``send_global_init`` / ``send_terminate`` the server side's one-shot messages, so that this
  package's hooks can report to the reference's controller.

ZeroMQ comes from ``pyzmq`` (its bundled libzmq); the messages are coded by ``protobuf_wire``.  Both are optional:
the package's own transport (``messages.py`` frames over TCP, native client in ``csrc/telemetry``) needs neither.
"""
from __future__ import annotations

import queue
import threading
from typing import Callable, Optional

from . import messages as M
from . import protobuf_wire as PB


def _zmq():
    try:
        import zmq
    except ImportError as e:  # pragma: no cover - pyzmq is an optional dependency
        raise RuntimeError("the ZeroMQ endpoints need pyzmq") from e
    return zmq


class ZmqControllerEndpoint:
    """ROUTER socket that feeds a running ``Controller`` with the reference's protobuf requests."""

    def __init__(self, controller, uri: str = "tcp://127.0.0.1:5556") -> None:
        zmq = _zmq()
        self.controller = controller
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.ROUTER)
        self.sock.setsockopt(zmq.LINGER, 0)
        if uri.endswith(":0") or uri.endswith(":*"):
            base = uri.rsplit(":", 1)[0]
            self.port = self.sock.bind_to_random_port(base)
            self.uri = f"{base}:{self.port}"
        else:
            self.sock.bind(uri)
            self.uri = uri
            self.port = int(uri.rsplit(":", 1)[1])
        self.stop = threading.Event()
        self.thread = threading.Thread(target=self._main, daemon=True, name="controller-zmq")
        self.requests = 0

    def start(self) -> "ZmqControllerEndpoint":
        self.thread.start()
        return self

    def close(self) -> None:
        self.stop.set()
        self.thread.join(timeout=2.0)
        self.sock.close(0)

    def _main(self) -> None:
        zmq = _zmq()
        poller = zmq.Poller()
        poller.register(self.sock, zmq.POLLIN)
        while not self.stop.is_set() and not self.controller.stop.is_set():
            if not dict(poller.poll(100)):
                continue
            frames = self.sock.recv_multipart()
            # REQ -> ROUTER: [identity, empty delimiter, body]; a DEALER peer may leave the delimiter out
            ident, body = frames[0], frames[-1]
            envelope = frames[:-1]
            try:
                reply = self._handle(ident, body)
            except ValueError:
                reply = PB.encode_response(PB.RESP_INVALID)
            self.requests += 1
            self.sock.send_multipart(envelope + [reply])

    def _handle(self, ident: bytes, body: bytes) -> bytes:
        from .controller import Client
        from .optimizer import max_batch_for

        c = self.controller
        rtype, payload = PB.decode_request(body)
        if rtype == PB.REQ_LOCAL_TELEMETRY_INIT and payload is not None:
            li: M.LocalInit = payload
            with c.lock:
                c.clients[li.gpu_id] = Client(li.gpu_id, li.rank, li.local_rank, li.gpu_name)
                c.scoreboard.loc[li.gpu_id, ["location", "gpu"]] = [f"{li.rank}:{li.local_rank}", li.gpu_name]
                if c.optimizer is not None and li.gpu_id < c.optimizer.num_gpus:
                    c.optimizer.set_max_batch(li.gpu_id, getattr(c, "max_batch", None) or max_batch_for(li.gpu_name))
                c._choose_profile()
        elif rtype == PB.REQ_LOCAL_TELEMETRY and payload is not None:
            t: M.LocalTelemetry = payload
            c.rx.put(t)
            client = c.clients.get(t.gpu_id)
            if client is not None:
                try:
                    inst = client.pending.get_nowait()
                    return PB.encode_response(PB.RESP_INSTRUCTION, inst, client_id=t.gpu_id)
                except queue.Empty:
                    pass
        elif rtype == PB.REQ_GLOBAL_TELEMETRY_INIT and payload is not None:
            c._on_global_init(payload)
        elif rtype == PB.REQ_TERMINATE:
            c.stop.set()
        return PB.encode_response(PB.RESP_OK)


class ZmqTelemetryClient:
    """The reference's per-GPU client: REQ socket, init message in the constructor, reports from a worker thread,
    ``callback(effective_since, TrainConfig)`` for every valid instruction in a reply."""

    def __init__(self, uri: str, gpu_id: int, gpu_name: str, rank: int, local_rank: int, timeout_ms: int = 5000) -> None:
        zmq = _zmq()
        self.gpu_id = gpu_id
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.REQ)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.sock.setsockopt(zmq.RCVTIMEO, timeout_ms)
        self.sock.setsockopt(zmq.SNDTIMEO, timeout_ms)
        self.sock.connect(uri)
        self._alive = True
        self._messages = 0
        self._q: "queue.Queue" = queue.Queue()
        self._roundtrip(PB.encode_request(PB.REQ_LOCAL_TELEMETRY_INIT, M.LocalInit(gpu_id, rank, local_rank, gpu_name)))
        self.thread = threading.Thread(target=self._main, daemon=True, name="telemetry-zmq")
        self.thread.start()

    def alive(self) -> bool:
        return self._alive

    def _roundtrip(self, body: bytes) -> Optional[bytes]:
        zmq = _zmq()
        try:
            self.sock.send(body)
            return self.sock.recv()
        except zmq.ZMQError:
            self._alive = False      # controller gone: training goes on without it
            return None

    def report(self, uiter: int, config: M.TrainConfig, measurement: M.Measurement,
               callback: Optional[Callable[[int, M.TrainConfig], None]] = None) -> None:
        body = PB.encode_request(PB.REQ_LOCAL_TELEMETRY, M.LocalTelemetry(self.gpu_id, uiter, config, measurement),
                                 message_id=self._messages)
        self._messages += 1
        self._q.put((body, callback))

    def _main(self) -> None:
        while self._alive:
            item = self._q.get()
            if item is None:
                return
            body, callback = item
            reply = self._roundtrip(body)
            if reply is None:
                return
            rtype, inst = PB.decode_response(reply)
            if rtype == PB.RESP_INSTRUCTION and inst is not None and callback is not None:
                callback(inst.iter_effective_since, inst.config)

    def close(self) -> None:
        self._alive = False
        self._q.put(None)
        self.thread.join(timeout=2.0)
        self.sock.close(0)


def _one_shot(uri: str, body: bytes, timeout_ms: int = 5000) -> Optional[bytes]:
    zmq = _zmq()
    sock = zmq.Context.instance().socket(zmq.REQ)
    sock.setsockopt(zmq.LINGER, 0)
    sock.setsockopt(zmq.RCVTIMEO, timeout_ms)
    sock.setsockopt(zmq.SNDTIMEO, timeout_ms)
    try:
        sock.connect(uri)
        sock.send(body)
        return sock.recv()
    except zmq.ZMQError:
        return None
    finally:
        sock.close(0)


def send_global_init(uri: str, g: M.GlobalInit, timeout_ms: int = 5000) -> bool:
    """What the reference's ``TelemetryServer::send_global_telemetry`` sends (telemetry_server.cpp:75-96)."""
    return _one_shot(uri, PB.encode_request(PB.REQ_GLOBAL_TELEMETRY_INIT, g), timeout_ms) is not None


def send_terminate(uri: str, timeout_ms: int = 2000) -> bool:
    return _one_shot(uri, PB.encode_request(PB.REQ_TERMINATE), timeout_ms) is not None
