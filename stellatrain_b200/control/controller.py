"""Centralised controller: receives per-GPU telemetry, answers with instructions.

Role of the reference's ``BatchSizeRateAlloc`` server (backend/src/engine/batch_rate_alloc.py:16-335):
one connection per GPU, every report is answered with either ``OK`` or a queued ``INSTRUCTION``; a
scoreboard keeps the latest smoothed measurements per client; a worker fits the per-GPU compute model and
runs the optimiser; ``DISABLE_RATE_ADAPT`` turns instructions off; ``MODEL_PROFILE`` names the
convergence profile.  Transport is framed TCP (``messages.py``) instead of ZeroMQ ROUTER/REQ, threads
talk through queues, and a pid file guards against two controllers on one port.

    python -m stellatrain_b200.control.controller --port 5556
"""
from __future__ import annotations

import argparse
import os
import queue
import socket
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import pandas as pd

from . import messages as M
from .gp_profile import AnalyticProfile, load_profile
from .optimizer import BatchRateOptimizer, TrafficModel, max_batch_for

LOG_PATH = "/tmp/stellatrain-b200-controller.log"
# one line per issued instruction set (the reference appends to instruction_history_log.txt,
# backend/src/engine/batch_rate_alloc_optim.py:474-477)
INSTRUCTION_LOG_PATH = "/tmp/stellatrain-b200-instructions.log"
SMOOTH = 0.9     # scoreboard EWMA
VERBOSE = os.environ.get("STELLATRAIN_CONTROLLER_VERBOSE", "0") not in ("", "0")   # registrations and replies on stderr


@dataclass
class Client:
    gpu_id: int
    rank: int
    local_rank: int
    gpu_name: str
    pending: "queue.Queue[M.Instruction]" = field(default_factory=queue.Queue)


class Controller:
    def __init__(self, port: int = 5556, host: str = "0.0.0.0", adapt: Optional[bool] = None,
                 profile_path: Optional[str] = None, transport: str = "nvlink", state_path: Optional[str] = None,
                 wire_blocks: Optional[bool] = None, max_batch: Optional[int] = None) -> None:
        self.adapt = (os.environ.get("DISABLE_RATE_ADAPT", "0") in ("", "0")) if adapt is None else adapt
        # Without a named profile (argument or MODEL_PROFILE, batch_rate_alloc_optim.py:139-141) the one that ships for the
        # clients' kind of GPU is taken once their names are known, and the analytic surrogate when none ships.
        self.profile_path = profile_path or os.environ.get("MODEL_PROFILE")
        self.profile = load_profile(self.profile_path)
        self.transport = transport
        self.max_batch = max_batch        # per-GPU batch ceiling of this job; None: by device name (MAX_BATCH_SIZE_MAP)
        # the CPU tier's TCP messages carry whole blocks of 16 entries behind one block id by default: the byte model
        # that turns a compression ratio into required goodput has to know
        self.wire_blocks = (transport == "tcp") if wire_blocks is None else wire_blocks
        self.state_path = state_path      # optimiser state is written here after every instruction and read back at start
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.sock.bind((host, port))
        self.sock.listen(64)
        self.port = self.sock.getsockname()[1]
        self.clients: Dict[int, Client] = {}
        self.scoreboard = pd.DataFrame(columns=["location", "gpu", "batch_size", "grad_acc", "comp_ratio", "fwd_ms", "bwd_ms",
                                                "bwd_fwd_gap_ms", "intra_fwd_gap_ms", "send_mbps", "recv_mbps", "uiter"])
        self.global_init: Optional[M.GlobalInit] = None
        self.optimizer: Optional[BatchRateOptimizer] = None
        self.rx: "queue.Queue[M.LocalTelemetry]" = queue.Queue()
        self.lock = threading.Lock()
        self.stop = threading.Event()
        self.latest_iter = 0
        self.issued: List[M.Instruction] = []
        self.threads: List[threading.Thread] = []

    # ---------------------------------------------------------------- threads
    def start(self) -> "Controller":
        for fn in (self._accept_main, self._logic_main):
            t = threading.Thread(target=fn, daemon=True, name=fn.__name__)
            t.start()
            self.threads.append(t)
        return self

    def close(self) -> None:
        self.stop.set()
        try:
            self.sock.close()
        except OSError:
            pass

    def _accept_main(self) -> None:
        self.sock.settimeout(0.2)
        while not self.stop.is_set():
            try:
                conn, _ = self.sock.accept()
            except (socket.timeout, OSError):
                continue
            conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            t = threading.Thread(target=self._io_main, args=(conn,), daemon=True, name="controller-io")
            t.start()

    def _io_main(self, conn: socket.socket) -> None:
        client: Optional[Client] = None
        try:
            while not self.stop.is_set():
                frame = M.recv_frame(conn)
                if frame is None:
                    return
                mtype, payload = frame
                reply = M.pack_frame(M.OK)
                if mtype == M.LOCAL_INIT:
                    li = M.parse(mtype, payload)
                    client = Client(li.gpu_id, li.rank, li.local_rank, li.gpu_name)
                    if VERBOSE:
                        print(f"[controller] {time.time():.3f} registration of gpu {li.gpu_id} ({li.gpu_name}) arrived",
                              file=sys.stderr, flush=True)
                    with self.lock:
                        self.clients[li.gpu_id] = client
                        self.scoreboard.loc[li.gpu_id, ["location", "gpu"]] = [f"{li.rank}:{li.local_rank}", li.gpu_name]
                        if self.optimizer is not None and li.gpu_id < self.optimizer.num_gpus:
                            self.optimizer.set_max_batch(li.gpu_id, self.max_batch or max_batch_for(li.gpu_name))
                        self._choose_profile()
                    if VERBOSE:
                        print(f"[controller] {time.time():.3f} registration of gpu {li.gpu_id} answered, profile "
                              f"{type(self.profile).__name__}", file=sys.stderr, flush=True)
                elif mtype == M.LOCAL:
                    t = M.parse(mtype, payload)
                    self.rx.put(t)
                    if client is not None:
                        try:
                            reply = M.pack_instruction(client.pending.get_nowait())
                        except queue.Empty:
                            pass
                elif mtype == M.GLOBAL_INIT:
                    self._on_global_init(M.parse(mtype, payload))
                elif mtype == M.TERMINATE:
                    conn.sendall(reply)
                    self.stop.set()
                    return
                conn.sendall(reply)
        except (OSError, ValueError):
            return
        finally:
            conn.close()

    def _choose_profile(self) -> None:
        """Called with the lock held, whenever a client or the job description arrives: the shipped profile for the
        clients' kind of GPU and, once the job description is there, for a model of the job's size."""
        if self.profile_path:
            return
        n_params = float(sum(self.global_init.param_counts)) if self.global_init is not None else None
        for c in self.clients.values():
            want = (c.gpu_name, n_params)
            if getattr(self, "_profile_for", None) == want:
                return
            chosen = load_profile(None, c.gpu_name, n_params)
            if not isinstance(chosen, AnalyticProfile):
                self._profile_for = want
                self.profile = chosen
                if self.optimizer is not None:
                    self.optimizer.profile = chosen
                return

    def _on_global_init(self, gi: M.GlobalInit) -> None:
        with self.lock:
            self.global_init = gi
            traffic = TrafficModel(gi.param_counts, self.transport, gi.grad_fp16, gi.grad_idx_u16, grad_block16=self.wire_blocks)
            self._choose_profile()
            self.optimizer = BatchRateOptimizer(gi.num_gpus, gi.num_nodes, traffic, self.profile,
                                                latest_iter=lambda: self.latest_iter)
            for gid, c in self.clients.items():
                if gid < gi.num_gpus:
                    self.optimizer.set_max_batch(gid, self.max_batch or max_batch_for(c.gpu_name))
            self._restore_state()

    # ---------------------------------------------------------------- persistence
    def save_state(self) -> None:
        """Atomic write of the optimiser's state (fitted curves, phase, instruction history); the reference keeps
        all of it in memory only (backend/src/engine/batch_rate_alloc_optim.py:117-162)."""
        if not self.state_path or self.optimizer is None:
            return
        import pickle

        tmp = self.state_path + ".tmp"
        try:
            with open(tmp, "wb") as f:
                pickle.dump({"optimizer": self.optimizer.state_dict(), "latest_iter": self.latest_iter}, f)
            os.replace(tmp, self.state_path)
        except OSError:
            pass

    def _restore_state(self) -> None:
        if not self.state_path or not os.path.exists(self.state_path) or self.optimizer is None:
            return
        import pickle

        try:
            with open(self.state_path, "rb") as f:
                sd = pickle.load(f)
            self.optimizer.load_state_dict(sd["optimizer"])
            self.latest_iter = max(self.latest_iter, int(sd.get("latest_iter", 0)))
        except (OSError, ValueError, KeyError, pickle.UnpicklingError):
            pass      # a state file of another job (different number of GPUs) or a damaged one: start afresh

    def _update_scoreboard(self, t: M.LocalTelemetry) -> dict:
        m, c = t.measurement, t.config
        new = {"batch_size": c.ubatch_size, "grad_acc": c.gradient_accumulation, "comp_ratio": c.compression_rate,
               "fwd_ms": m.fwd_delay_ms, "bwd_ms": m.bwd_delay_ms, "bwd_fwd_gap_ms": m.bwd_fwd_gap_ms,
               "intra_fwd_gap_ms": m.intra_fwd_gap_ms, "send_mbps": m.grad_send_thpt_mbps, "recv_mbps": m.grad_recv_thpt_mbps}
        with self.lock:
            for k, v in new.items():
                old = self.scoreboard.at[t.gpu_id, k] if (t.gpu_id in self.scoreboard.index and k in self.scoreboard.columns) else None
                smooth = k in ("fwd_ms", "bwd_ms", "bwd_fwd_gap_ms", "intra_fwd_gap_ms", "send_mbps", "recv_mbps")
                if smooth and old is not None and not pd.isna(old) and self.scoreboard.at[t.gpu_id, "batch_size"] == c.ubatch_size:
                    v = SMOOTH * float(old) + (1.0 - SMOOTH) * float(v)
                self.scoreboard.at[t.gpu_id, k] = v
            self.scoreboard.at[t.gpu_id, "uiter"] = t.uiter
            self.latest_iter = max(self.latest_iter, int(t.uiter) // max(1, c.gradient_accumulation))
            row = {k: self.scoreboard.at[t.gpu_id, k] for k in new}
        row["gpu"] = t.gpu_id
        return row

    def _logic_main(self) -> None:
        last_dump = 0.0
        while not self.stop.is_set():
            try:
                t = self.rx.get(timeout=0.2)
            except queue.Empty:
                continue
            batch = [t]
            while True:
                try:
                    batch.append(self.rx.get_nowait())
                except queue.Empty:
                    break
            rows = [self._update_scoreboard(x) for x in batch]
            opt = self.optimizer
            if opt is None or not self.adapt:
                continue
            rows = [r for r in rows if r["gpu"] < opt.num_gpus]
            opt.update(rows)
            with self.lock:
                recv = pd.to_numeric(self.scoreboard["recv_mbps"], errors="coerce").dropna()
            measured = float(recv.max()) if len(recv) else 0.0
            inst = opt.step(self.latest_iter, measured)
            if inst is not None:
                for gid, c in list(self.clients.items()):
                    if gid < len(inst.batch):
                        msg = M.Instruction(inst.iter, M.TrainConfig(int(inst.batch[gid]), 1, float(inst.comp_ratio)))
                        c.pending.put(msg)
                        self.issued.append(msg)
                try:
                    with open(INSTRUCTION_LOG_PATH, "a") as f:
                        f.write(f"{time.time():.3f} observed_iter={self.latest_iter} effective_iter={inst.iter} "
                                f"ratio={float(inst.comp_ratio):.6f} batch={[int(b) for b in inst.batch]} "
                                f"measured_mbps={measured:.1f}\n")
                except OSError:
                    pass
                self.save_state()
            if time.time() - last_dump > 2.0:
                last_dump = time.time()
                try:
                    with self.lock, open(LOG_PATH, "w") as f:
                        f.write(self.scoreboard.to_string())
                except OSError:
                    pass


def _single_instance(port: int) -> None:
    pid_file = f"/tmp/stellatrain-b200-controller-{port}.pid"
    try:
        old = int(open(pid_file).read())
        # the pid recorded by the previous controller on this port, and only while it still is a controller: a stale
        # file may name a process id that the system has handed to somebody else since
        with open(f"/proc/{old}/cmdline", "rb") as f:
            still_a_controller = b"stellatrain_b200.control.controller" in f.read()
        if old != os.getpid() and still_a_controller:
            os.kill(old, 15)
            time.sleep(0.2)
    except (OSError, ValueError):
        pass
    with open(pid_file, "w") as f:
        f.write(str(os.getpid()))


def spawn_controller(port: int, host: str = "127.0.0.1", max_batch: Optional[int] = None, profile: Optional[str] = None,
                     transport: str = "nvlink", state_file: Optional[str] = None, wait_s: float = 30.0):
    """Starts the controller in a process of its own (``python -m stellatrain_b200.control.controller``), the way the
    reference's telemetry server starts its ``batch_rate_alloc.py`` (backend/src/engine/telemetry_server.cpp:57-73), and
    returns the ``subprocess.Popen`` once the port accepts connections.  A controller inside a training process shares
    that process's interpreter lock: its fits and optimisations slow the training loop down, and a training thread
    that waits for the device with the lock held keeps it from answering anybody."""
    import subprocess

    cmd = [sys.executable, "-m", "stellatrain_b200.control.controller", "--port", str(port), "--host", host,
           "--transport", transport]
    if max_batch:
        cmd += ["--max-batch", str(int(max_batch))]
    if profile:
        cmd += ["--profile", profile]
    if state_file:
        cmd += ["--state-file", state_file]
    def _die_with_parent() -> None:      # in the child, before exec: SIGTERM when the process that started it goes away
        import ctypes
        import signal

        try:
            ctypes.CDLL("libc.so.6", use_errno=True).prctl(1, signal.SIGTERM)     # PR_SET_PDEATHSIG
        except OSError:
            pass

    proc = subprocess.Popen(cmd, preexec_fn=_die_with_parent)
    deadline = time.time() + wait_s
    while time.time() < deadline:
        if proc.poll() is not None:
            raise RuntimeError(f"the controller process ended with status {proc.returncode} before it listened")
        try:
            with socket.create_connection((host, port), timeout=0.5):
                return proc
        except OSError:
            time.sleep(0.1)
    proc.terminate()
    raise RuntimeError(f"the controller process did not listen on {host}:{port} within {wait_s:.0f} s")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, default=5556)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--profile", default=None)
    ap.add_argument("--transport", default="nvlink", choices=["nvlink", "tcp"])
    ap.add_argument("--state-file", default=None, help="optimiser state is kept here across restarts of the controller")
    ap.add_argument("--max-batch", type=int, default=None, help="per-GPU batch ceiling (default: by device name)")
    args = ap.parse_args()
    _single_instance(args.port)
    c = Controller(args.port, host=args.host, profile_path=args.profile, transport=args.transport, state_path=args.state_file,
                   max_batch=args.max_batch).start()
    try:
        while not c.stop.is_set():
            time.sleep(0.2)
    finally:
        c.close()


if __name__ == "__main__":
    main()
