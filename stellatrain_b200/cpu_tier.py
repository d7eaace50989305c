"""Python face of the CPU-offload tier (native module ``_Ccpu``).

The reference *is* this tier: gradients leave the GPU, are reduced, sparsified, exchanged and applied on
the CPU, and parameters come back (backend/src/engine/modules/*.cpp).  Here it is an option next to the
GPU-resident engine: the stand-in baseline for the reference pipeline, the home of the flat-gradient CPU
benchmark, and a way to train when optimiser state should not live in HBM.

``CpuOffloadEngine`` drives the native ``CpuEngine`` for an ``nn.Module``:

* host parameters: the engine reads gradients from and writes parameters to the tensors directly;
* CUDA parameters: the native engine copies gradients into the pinned shared slots on copy streams (event on the
  backward stream, stream wait, asynchronous copy, host callback that starts the task) and copies updated parameters
  back behind its CopyOut stage (the reference's D2H_Copy / H2D_Copy stages, d2h_copy.cpp:20-66, h2d_copy.cpp:31-56).
  ``native_copies=False`` keeps the older route: torch copies issued by this class and two helper threads.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch
import torch.nn as nn

_ext = None


def _load():
    global _ext
    if _ext is None:
        from . import _build

        _ext = _build.load_extension("_Ccpu")
    return _ext


def available() -> bool:
    try:
        _load()
        return True
    except Exception:  # noqa: BLE001
        return False


_compressors: dict = {}


def get_compressor(method: str):
    c = _compressors.get(method)
    if c is None:
        c = _load().Compressor(method)
        _compressors[method] = c
    return c


def compress(name: str, flat: torch.Tensor, k: int, method: str):
    """One tensor, no residual: (idx:int32, val:float32) with at most k entries."""
    flat = flat.detach().contiguous().float().reshape(-1)
    idx = torch.empty(k, dtype=torch.int32)
    val = torch.empty(k, dtype=torch.float32)
    n = get_compressor(method).compress(name, flat.data_ptr(), flat.numel(), k, idx.data_ptr(), val.data_ptr())
    return idx[:n], val[:n]


def compress_with_feedback(name: str, grad: torch.Tensor, resid: torch.Tensor, k: int, method: str):
    """Error-feedback compression in place on ``resid``; returns (idx:int64 view of uint32, val)."""
    assert grad.dtype == torch.float32 and resid.dtype == torch.float32 and grad.is_contiguous() and resid.is_contiguous()
    idx = torch.empty(k, dtype=torch.int32)
    val = torch.empty(k, dtype=torch.float32)
    n = get_compressor(method).compress_with_feedback(name, grad.data_ptr(), resid.data_ptr(), grad.numel(), k,
                                                      idx.data_ptr(), val.data_ptr())
    return idx[:n], val[:n]


def make_optimizer(kind: str):
    ext = _load()
    return {"sgd": ext.SGD, "adam": ext.Adam, "sgd_naive": ext.SGDNaive}[kind]()


def _from_ptr(ptr: int, numel: int) -> torch.Tensor:
    """A float32 tensor over foreign host memory (the shared-memory pool); no ownership."""
    buf = (ctypes.c_float * numel).from_address(ptr)
    return torch.frombuffer(buf, dtype=torch.float32, count=numel)


def bundled_libzmq() -> str:
    """Path of the libzmq that ships inside pyzmq ('' when that package is not installed)."""
    import glob
    import importlib.util

    spec = importlib.util.find_spec("zmq")
    if spec is None or not spec.submodule_search_locations:
        return ""
    root = os.path.dirname(list(spec.submodule_search_locations)[0])
    found = sorted(glob.glob(os.path.join(root, "pyzmq.libs", "libzmq*.so*")))
    return found[0] if found else ""


def prepare_telemetry_uri(uri: str) -> str:
    """For a ``zmq://`` controller address (the reference's transport) tell the native client where pyzmq keeps its
    libzmq, unless the environment already names one.  Returns the uri unchanged."""
    if uri and uri.startswith("zmq") and not os.environ.get("STELLATRAIN_LIBZMQ"):
        found = bundled_libzmq()
        if found:
            os.environ["STELLATRAIN_LIBZMQ"] = found
    return uri


class CpuOffloadEngine:
    def __init__(self, module: nn.Module, *, master_addr: str = "127.0.0.1", master_port: int = 5555, world_size: int = 1,
                 rank: int = 0, session: Optional[int] = None, local_world_size: int = 1, local_rank: int = 0,
                 method: str = "thresholdv16", gradient_accumulation: int = 1, staleness: int = 1, ratio: float = 0.99,
                 optimizer: str = "sgd", optimizer_options: Optional[dict] = None, data_bytes: int = 0,
                 timeout_ms: int = 30000, workers: int = 0, debug_accuracy: bool = False, debug_barrier: bool = False,
                 wire_blocks: bool = True, wire_values: str = "fp32", native_copies: Optional[bool] = None,
                 data_transport: str = "tcp", bundle_elems: int = 1 << 16):
        """``bundle_elems``: tensors with fewer elements than this are registered in bundles (consecutive small
        tensors, laid end to end, closed once a bundle holds that many elements) that pass through the pipeline as one
        task per iteration; selection still treats every tensor by itself.  0 gives one task per tensor, which is what
        the reference does (backend/src/engine/core.cpp:1025-1095) and costs it a fixed price per tensor per iteration."""
        ext = _load()
        if data_transport == "zmq":
            # the ring between nodes over ZeroMQ PUSH/PULL sockets, the reference's transport; the native comm manager
            # opens the library at run time and is told where pyzmq keeps its copy
            os.environ["STELLATRAIN_DATA_TRANSPORT"] = "zmq"
            if not os.environ.get("STELLATRAIN_LIBZMQ"):
                found = bundled_libzmq()
                if found:
                    os.environ["STELLATRAIN_LIBZMQ"] = found
        elif data_transport != "tcp":
            raise ValueError("data_transport must be 'tcp' or 'zmq'")
        self.module = module
        self.engine = ext.CpuEngine()
        params = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        self.cuda = params[0][1].is_cuda
        if data_bytes == 0:
            # parameter + residual + 2 * local_world gradient slots per element, with head-room
            need = sum(p.numel() for _, p in params) * 4 * (2 + 2 * local_world_size)
            data_bytes = max(64 << 20, int(need * 1.25) + (8 << 20))
        self.engine.configure(master_addr, master_port, world_size, rank, os.getpid() if session is None else session,
                              local_world_size, local_rank, method, gradient_accumulation, staleness, ratio,
                              data_bytes, timeout_ms, workers, self.cuda, debug_accuracy, debug_barrier)
        # messages between nodes: block ids for whole aligned runs of 16 indices, optionally 16-bit values whose
        # rounding error stays in the sender's residual
        self.engine.configure_wire(wire_blocks, {"fp32": 0, "fp16": 1, "bf16": 2}[wire_values])
        self._meta = {"method": method, "ratio": ratio, "staleness": staleness, "gradient_accumulation": gradient_accumulation,
                      "optimizer": optimizer, "optimizer_options": dict(optimizer_options or {}), "world_size": world_size,
                      "local_world_size": local_world_size}
        self._local_rank = local_rank
        self.engine.set_optimizer(optimizer)
        for k, v in (optimizer_options or {}).items():
            self.engine.configure_optimizer(k, v)
        self.grad_accumulation = gradient_accumulation
        self.params = [p for _, p in params]
        self._meta["bundle_elems"] = int(bundle_elems)
        for name, p in params:
            if not p.is_contiguous():
                raise ValueError(f"parameter {name} must be contiguous")
        # units: what the native engine sees as one parameter.  (first layer index, key, [(name, tensor, offset)], numel)
        self._units = []
        open_unit = None
        layer_of = {name: li for li, (name, _) in enumerate(params)}
        for li, (name, p) in enumerate(params):
            if p.numel() >= bundle_elems:
                self._units.append([li, name[-40:], [(name, p, 0)], p.numel()])
                continue
            if open_unit is None:
                open_unit = [li, "", [], 0]
                self._units.append(open_unit)
            open_unit[2].append((name, p, open_unit[3]))
            open_unit[3] += (p.numel() + 15) // 16 * 16        # aligned blocks of a member stay aligned in the bundle
            if open_unit[3] >= bundle_elems:
                open_unit = None
        self._where = {}               # id(tensor) -> (engine index, member number or -1)
        self._stash = {}               # engine index -> gradients of a bundle's members waiting for the last one
        for unit in self._units:
            li, key, members, total = unit
            if len(members) == 1:
                name, p, _ = members[0]
                unit[1] = key = name[-40:]
                unit[3] = total = p.numel()
                if self.cuda:
                    # the engine never writes device memory through `user_param`; it starts the master copy from a
                    # host copy of the initial values
                    init = p.detach().reshape(-1).to("cpu", torch.float32).contiguous()
                    idx = self.engine.pre_train_init(li, key, total, 0, init.data_ptr())
                else:
                    idx = self.engine.pre_train_init(li, key, total, p.data.data_ptr())
                self._where[id(p)] = (idx, -1)
            else:
                unit[1] = key = f"{members[0][0][-28:]}+{len(members) - 1}"
                init = torch.zeros(total, dtype=torch.float32)
                for name, p, off in members:
                    init[off:off + p.numel()] = p.detach().reshape(-1).to("cpu", torch.float32)
                idx = self.engine.pre_train_init(li, key, total, 0, init.data_ptr())
                self.engine.set_param_members(idx, [f"{layer_of[name]}@{name[-40:]}" for name, _, _ in members],
                                              [off for _, _, off in members], [p.numel() for _, p, _ in members],
                                              [] if self.cuda else [p.data.data_ptr() for _, p, _ in members])
                for m, (_, p, _) in enumerate(members):
                    self._where[id(p)] = (idx, m)
            unit.append(idx)
            if self.cuda:
                master = _from_ptr(self.engine.master_param(idx), total)
                for _, p, off in members:
                    p.data.copy_(master[off:off + p.numel()].view_as(p), non_blocking=False)
        # CUDA parameters, two ways to move data: copies issued by this class with torch streams and two helper threads,
        # or by the native engine itself (event, stream wait, asynchronous copy and a host callback per task, its
        # D2H_Copy / H2D_Copy stages); the second needs no Python thread on the path of a task
        if native_copies is None:
            native_copies = self.cuda and self.engine.device_copies_available()
        self.native_copies = bool(native_copies and self.cuda)
        if self.native_copies:
            if not self.engine.device_copies_available():
                raise RuntimeError("native_copies=True needs the CUDA runtime in this process")
            self._native_streams = [torch.cuda.Stream() for _ in range(4)]
            for _, _, members, _, idx in self._units:
                if len(members) == 1:
                    self.engine.attach_device_param(idx, members[0][1].data.data_ptr())
                else:
                    self.engine.attach_device_members(idx, [p.data.data_ptr() for _, p, _ in members])
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in self.params]
        self._hooks.append(module.register_forward_pre_hook(self._pre_forward))
        self._stop = False
        self._copy_stream = torch.cuda.Stream() if self.cuda else None
        self._h2d_thread = None
        self._pending_events: list = []
        if self.cuda and not self.native_copies:
            self._h2d_thread = threading.Thread(target=self._h2d_main, name="H2DCopy", daemon=True)
            self._h2d_thread.start()
            self._d2h_thread = threading.Thread(target=self._d2h_main, name="D2HCopy", daemon=True)
            self._d2h_cv = threading.Condition()
            self._d2h_thread.start()

    # ------------------------------------------------------------------ hooks
    def _pre_forward(self, _mod, _inp) -> None:
        if self._micro != 0:
            return   # later micro-iterations do not wait (model_wrapper.py:88-92)
        for i in range(len(self._units)):
            self.engine.pre_forward_process(i)

    def _on_grad(self, p: torch.Tensor) -> None:
        idx, member = self._where[id(p)]
        g = p.grad
        if not self.cuda:
            if member < 0:
                self.engine.post_backward_process(idx, g.contiguous().data_ptr())
            else:
                self.engine.post_backward_member(idx, member, g.contiguous().data_ptr())
            p.grad = None
            return
        # device accumulation across micro-iterations, one D2H at the end (core.cpp:781-788)
        if self._micro != self.grad_accumulation - 1:
            return
        g = g if (g.is_contiguous() and g.dtype == torch.float32) else g.contiguous().float()
        p.grad = None
        members = self._units[idx][2]
        if member < 0:
            grads = [g]
        else:
            # a bundle leaves the device when its last member's gradient is there
            stash = self._stash.setdefault(idx, {})
            stash[member] = g
            if len(stash) < len(members):
                return
            grads = [stash[m] for m in range(len(members))]
            del self._stash[idx]
        if self.native_copies:
            stream = self._native_streams[idx % len(self._native_streams)]
            cur = torch.cuda.current_stream().cuda_stream
            if member < 0:
                self.engine.post_backward_device(idx, g.data_ptr(), cur, stream.cuda_stream)
            else:
                self.engine.post_backward_device_members(idx, [t.data_ptr() for t in grads], cur, stream.cuda_stream)
            for t in grads:
                t.record_stream(stream)          # the allocator must not reuse the gradient before the copy has read it
        else:
            slot = _from_ptr(self.engine.claim_grad_slot(idx), self._units[idx][3])   # one per iteration, in turn
            ev = torch.cuda.Event()
            cur = torch.cuda.current_stream()
            self._copy_stream.wait_stream(cur)
            with torch.cuda.stream(self._copy_stream):
                for t, (_, q, off) in zip(grads, members):
                    slot[off:off + q.numel()].copy_(t.reshape(-1), non_blocking=True)
                    t.record_stream(self._copy_stream)
                ev.record(self._copy_stream)
            with self._d2h_cv:
                self._pending_events.append((ev, idx))
                self._d2h_cv.notify()

    @property
    def _micro(self) -> int:
        """Micro-iteration index published by StellaTrainDataLoader (0 outside a loader loop)."""
        from .utils.loader import current_micro_step

        return max(0, current_micro_step())

    def _d2h_main(self) -> None:
        while not self._stop:
            with self._d2h_cv:
                if not self._pending_events:
                    self._d2h_cv.wait(timeout=0.05)
                    continue
                ev, idx = self._pending_events.pop(0)
            ev.synchronize()
            for _ in range(self.grad_accumulation):
                self.engine.post_backward_in_slot(idx)

    def _h2d_main(self) -> None:
        stream = torch.cuda.Stream()
        while not self._stop:
            for idx, it in self.engine.pop_ready_updates(50):
                master = _from_ptr(self.engine.master_param(idx), self._units[idx][3])
                with torch.cuda.stream(stream):
                    for _, p, off in self._units[idx][2]:
                        p.data.copy_(master[off:off + p.numel()].view_as(p), non_blocking=True)
                stream.synchronize()
                self.engine.copy_out_done(idx, it)

    # ------------------------------------------------------------------ control
    def synchronize(self) -> None:
        if self.cuda and self.native_copies:
            torch.cuda.synchronize()
        elif self.cuda:
            torch.cuda.synchronize()
            import time
            while True:
                with self._d2h_cv:
                    if not self._pending_events:
                        break
                time.sleep(0.001)
        self.engine.synchronize()
        if self.cuda:
            torch.cuda.synchronize()

    def barrier(self) -> None:
        self.engine.barrier()

    # the calls the ``fasterdp``-named frontend makes on whichever engine is attached
    def set_compression_ratio(self, ratio: float) -> None:
        self.engine.configure_compression_ratio(float(ratio))
        self._meta["ratio"] = float(ratio)

    def configure_optimizer(self, **options) -> None:
        for k, v in options.items():
            self.engine.configure_optimizer(k, v)
            self._meta["optimizer_options"][k] = v

    def replica_drift(self) -> float:
        """Largest difference between this node's master copy and node 0's (0.0 on one node)."""
        self.synchronize()
        return max((self.engine.force_model_sync(i, True) for i in range(len(self._units))), default=0.0)

    def broadcast_parameters(self) -> None:
        self.synchronize()
        for i in range(len(self._units)):
            self.engine.force_model_sync(i, False)

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        """Everything a later run needs to continue bit for bit, in torch's plain-container form (``torch.save``-able):
        the module's ``state_dict``, the sparse optimiser's per-tensor state (moments and step counters, or momentum
        buffers), the error-feedback residuals, the thresholds of the compressor and the engine's settings.  Flushes
        the pipeline first.  Optimiser state and thresholds live in the node master (local rank 0): save its dictionary.
        The reference keeps all of this only in memory (backend/src/optim/adam.h:15-18, sgd.h:15-18,
        compress/thresholdv16.h:13-14, engine/core.h:63)."""
        self.synchronize()
        resid = {}
        for _, _, members, total, idx in self._units:
            whole = _from_ptr(self.engine.grad_residual(idx), total)
            for n, p, off in members:
                resid[n] = whole[off:off + p.numel()].clone()
        opt = {}
        for tensor, (arrays, counters) in self.engine.optimizer_state().items():
            opt[tensor] = {"arrays": {k: torch.frombuffer(bytearray(v), dtype=torch.float32).clone() if len(v) else
                                      torch.zeros(0) for k, v in arrays.items()},
                           "counters": dict(counters)}
        return {"model": {k: v.detach().to("cpu").clone() for k, v in self.module.state_dict().items()},
                "optimizer": {"kind": self.engine.optimizer_kind(), "options": dict(self._meta["optimizer_options"]), "state": opt},
                "sparsifier": {"residual": resid,
                               "threshold": {k: tuple(v) for k, v in self.engine.compressor_state().items()}},
                "engine": dict(self._meta)}

    def load_state_dict(self, sd: dict) -> None:
        """Inverse of :meth:`state_dict` on an engine built with the same settings around the same architecture.
        Every local process calls it (each loads its module); the node master also restores the shared master copy,
        the residuals, the optimiser state and the thresholds."""
        if sd["optimizer"]["kind"] != self.engine.optimizer_kind():
            raise ValueError(f"checkpoint was written by the {sd['optimizer']['kind']} optimiser")
        self.synchronize()
        self.module.load_state_dict(sd["model"])
        if sd["engine"].get("bundle_elems", 0) != self._meta["bundle_elems"]:
            raise ValueError("checkpoint was written with bundle_elems=%d: the optimiser state is laid out by bundle, build "
                             "the engine with the same value" % sd["engine"].get("bundle_elems", 0))
        if self._local_rank == 0:
            for _, _, members, total, idx in self._units:
                master = _from_ptr(self.engine.master_param(idx), total)
                whole = _from_ptr(self.engine.grad_residual(idx), total)
                for n, p, off in members:
                    master[off:off + p.numel()].copy_(p.detach().reshape(-1).to("cpu", torch.float32))
                    whole[off:off + p.numel()].copy_(sd["sparsifier"]["residual"][n])
            self.engine.set_optimizer_state({t: ({k: v.contiguous().numpy().tobytes() for k, v in st["arrays"].items()},
                                                 {k: int(c) for k, c in st["counters"].items()})
                                             for t, st in sd["optimizer"]["state"].items()})
            self.engine.set_compressor_state({k: (float(v[0]), float(v[1]), bool(v[2]))
                                              for k, v in sd["sparsifier"]["threshold"].items()})
        if self._meta["local_world_size"] > 1 or self._meta["world_size"] > 1:
            self.engine.barrier()

    def stats_json(self, clear: bool = False) -> str:
        return self.engine.stats_json(clear)

    def close(self) -> None:
        self._stop = True
        for h in self._hooks:
            h.remove()
        if self._h2d_thread is not None:
            self._h2d_thread.join(timeout=2)
            self._d2h_thread.join(timeout=2)
        self.engine = None


class CpuTierTelemetry:
    """Closes the control loop for the CPU tier: times every step on the host, reports to the controller through the
    native telemetry client and applies the instructions that come back.

    The reference ships the client, the server and the controller but never connects them to its engine
    (backend/src/engine/telemetry_client.cpp:39-110, batch_rate_alloc.py:194-215).  Usage::

        hook = CpuTierTelemetry(engine, "127.0.0.1:5556", batch_size=32, rank=node_rank, local_rank=local_rank)
        for x, y in loader:
            x, y = hook.resize_batch(x, y)              # per-GPU batch size the controller asked for
            with hook.step() as marker:
                loss = criterion(model(x), y); marker.backward_begins(); loss.backward()

    A new compression ratio is handed to the engine together with the iteration from which it counts
    (``configure_compression_ratio_from``), so every node switches at the same task even though the instruction
    reaches the nodes at different moments.  Throughput fields are the bytes the node's comm manager sent and
    received during the step.
    """

    def __init__(self, engine: "CpuOffloadEngine", uri: Optional[str], batch_size: int, gpu_id: int = 0, rank: int = 0,
                 local_rank: int = 0, gpu_name: Optional[str] = None, apply_batch: bool = True, apply_ratio: bool = True,
                 timeout_ms: int = 5000) -> None:
        import time

        self._now = time.perf_counter
        self.engine = engine
        self.batch_size = int(batch_size)
        self.apply_batch, self.apply_ratio = apply_batch, apply_ratio
        self.iteration = 0
        self.ratio = float(engine._meta["ratio"])
        self.pending: list = []         # (effective_since, ubatch, ratio), written by the client's thread
        self.applied: list = []
        self.last: dict = {}
        self._lock = threading.Lock()
        self._prev_end: Optional[float] = None
        self._prev_bytes = engine.engine.comm_bytes()
        from .parallel.telemetry import _WeakInstruction

        self._callback = _WeakInstruction(self)
        self.client = None
        if uri:
            ext = _load()
            name = gpu_name or (torch.cuda.get_device_name(0) if engine.cuda else "cpu")
            self._TrainConfig = ext.TrainConfig
            self.client = ext.TelemetryClient(prepare_telemetry_uri(uri), gpu_id, name, rank, local_rank, timeout_ms)

    def _on_instruction(self, since: int, ubatch: int, grad_acc: int, ratio: float) -> None:
        with self._lock:
            self.pending.append((int(since), int(ubatch), float(ratio)))

    def _take_instructions(self) -> None:
        with self._lock:
            new, self.pending = self.pending, []
        for since, ubatch, ratio in new:
            # a switch that would lie in the past on this node counts from the next iteration
            since = max(since, self.iteration)
            if self.apply_ratio and 0.0 < ratio <= 1.0:
                self.engine.engine.configure_compression_ratio_from(since, ratio)
            self.applied.append((since, ubatch, ratio))
        for since, ubatch, ratio in self.applied:
            if since == self.iteration:
                if self.apply_batch and ubatch > 0:
                    self.batch_size = ubatch
                if self.apply_ratio and 0.0 < ratio <= 1.0:
                    self.ratio = ratio

    def resize_batch(self, *tensors: torch.Tensor):
        """Cut or tile a batch along dim 0 to the size the controller asked for."""
        self._take_instructions()      # a size that counts from this iteration applies to this batch already
        out = []
        for t in tensors:
            n = t.shape[0]
            if n >= self.batch_size:
                out.append(t[: self.batch_size])
            else:
                reps = (self.batch_size + n - 1) // n
                out.append(t.repeat(reps, *([1] * (t.dim() - 1)))[: self.batch_size])
        return tuple(out)

    def step(self):
        import contextlib

        @contextlib.contextmanager
        def _ctx():
            self._take_instructions()
            t0 = self._now()
            marker = _HostBackwardStart(self._now)
            try:
                yield marker
            finally:
                if self.engine.cuda:
                    torch.cuda.current_stream().synchronize()      # the step's kernels, not only their launches
                t1 = self._now()
                fwd = (marker.at - t0) * 1e3 if marker.at is not None else 0.0
                bwd = (t1 - marker.at) * 1e3 if marker.at is not None else (t1 - t0) * 1e3
                gap = (t0 - self._prev_end) * 1e3 if self._prev_end is not None else 0.0
                self._prev_end = t1
                tx, rx = self.engine.engine.comm_bytes()
                step_ms = max(fwd + bwd + gap, 1e-3)
                send = (tx - self._prev_bytes[0]) * 8.0 / (step_ms * 1000.0)
                recv = (rx - self._prev_bytes[1]) * 8.0 / (step_ms * 1000.0)
                self._prev_bytes = (tx, rx)
                self.last = {"fwd_delay_ms": fwd, "bwd_delay_ms": bwd, "bwd_fwd_gap_ms": gap, "intra_fwd_gap_ms": 0.0,
                             "grad_send_thpt_mbps": send, "grad_recv_thpt_mbps": recv}
                if self.client is not None and self.client.alive():
                    cfg = self._TrainConfig(self.batch_size, self.engine.grad_accumulation, self.ratio)
                    self.client.report(self.iteration, cfg, [send, recv, fwd, bwd, gap, 0.0], self._callback)
                self.iteration += 1

        return _ctx()


class _HostBackwardStart:
    """``marker.backward_begins()`` between forward and backward splits the two host times."""

    def __init__(self, now) -> None:
        self._now, self.at = now, None

    def backward_begins(self) -> None:
        self.at = self._now()
