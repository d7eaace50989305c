"""Connects a training loop to the controller: measures every step, reports, applies instructions.

The reference defines the client (backend/src/engine/telemetry_client.cpp:39-110) and the instruction
protocol (effective a few iterations after issue, backend/src/engine/batch_rate_alloc_optim.py:454-479)
but never instantiates them in its engine.  Here the loop is closed:

    hook = TelemetryHook(engine, "tcp://127.0.0.1:5556", batch_size=32)
    for x, y in loader:
        x, y = hook.resize_batch(x, y)          # per-GPU batch size the controller asked for
        with hook.step():                       # times forward/backward, reports, applies instructions
            loss = criterion(model(x), y); loss.backward()

Measurements are device times from CUDA events: forward, backward, the gap between the end of backward
and the start of the next forward, and the time a forward spent blocked on outstanding updates (exposed
communication).  Throughput fields come from the bytes the engine pushed during the step.
"""
from __future__ import annotations

import contextlib
import threading
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


class TelemetryHook:
    def __init__(self, engine, uri: Optional[str], batch_size: int, gpu_name: Optional[str] = None,
                 apply_batch: bool = True, apply_ratio: bool = True, link_bytes_per_entry: int = 8) -> None:
        self.engine = engine
        self.batch_size = int(batch_size)
        self.apply_batch, self.apply_ratio = apply_batch, apply_ratio
        self.bytes_per_entry = link_bytes_per_entry
        self.iteration = 0
        self.pending: List[Tuple[int, int, float]] = []      # (effective_since, ubatch, ratio)
        self.applied: List[Tuple[int, int, float]] = []
        self.lock = threading.Lock()
        self.client = None
        self._callback = _WeakInstruction(self)
        self._ev = {k: torch.cuda.Event(enable_timing=True) for k in ("f0", "f1", "b1", "prev_b1")}
        self._have_prev = False
        self.last: Dict[str, float] = {}
        self._agree_event = None
        self._agree_dev = torch.zeros(1, dtype=torch.float64, device=engine.device)
        self._agree_host = torch.zeros(1, dtype=torch.float64).pin_memory()
        if uri:
            from .. import cpu_tier

            ext = cpu_tier._load()
            name = gpu_name or (torch.cuda.get_device_name(engine.device) if engine.device.type == "cuda" else "cpu")
            self._TrainConfig = ext.TrainConfig
            self.client = ext.TelemetryClient(uri, engine.rank, name, 0, engine.rank, 5000)

    # ------------------------------------------------------------------ instructions
    def _on_instruction(self, since: int, ubatch: int, grad_acc: int, ratio: float) -> None:
        with self.lock:
            self.pending.append((int(since), int(ubatch), float(ratio)))

    _INF = float(2 ** 40)

    def _agreed_since(self) -> float:
        """Ranks receive an instruction at slightly different times, but must switch at the same
        iteration.  Every step each rank contributes the effective iteration of its earliest pending
        instruction (or "none yet"); the maximum over ranks, read one step later, is an iteration by
        which every rank holds the instruction."""
        eng = self.engine
        if eng.world == 1:
            with self.lock:
                return min((p[0] for p in self.pending), default=self._INF)
        agreed = self._INF
        if self._agree_event is not None:
            self._agree_event.synchronize()
            agreed = float(self._agree_host[0])
        with self.lock:
            mine = min((p[0] for p in self.pending), default=self._INF)
        self._agree_dev.fill_(mine)
        dist.all_reduce(self._agree_dev, op=dist.ReduceOp.MAX, group=eng.group)
        self._agree_host.copy_(self._agree_dev, non_blocking=True)
        self._agree_event = torch.cuda.Event()
        self._agree_event.record()
        return agreed

    def _apply_due(self) -> None:
        agreed = self._agreed_since()
        limit = min(agreed, float(self.iteration)) if agreed < self._INF else -1.0
        with self.lock:
            due = [p for p in self.pending if p[0] <= limit and agreed <= self.iteration]
            self.pending = [p for p in self.pending if p not in due]
        for since, ubatch, ratio in due:
            if self.apply_batch and ubatch > 0:
                self.batch_size = ubatch
            if self.apply_ratio and 0.0 < ratio <= 1.0:
                # every rank receives the same ratio for the same effective iteration
                lo = self.engine.buckets[0].bucket.min_ratio
                self.engine.set_compression_ratio(max(ratio, lo))
            self.applied.append((since, ubatch, ratio))
        if due and self.apply_batch and self.engine.world > 1:
            # unequal batches: weight each rank's gradient by its share of the global batch
            t = torch.tensor([float(self.batch_size)], device=self.engine.device)
            all_b = [torch.zeros_like(t) for _ in range(self.engine.world)]
            dist.all_gather(all_b, t, group=self.engine.group)
            b = torch.cat(all_b)
            self.engine.set_rank_weights((b / b.sum()).tolist())

    def resize_batch(self, *tensors: torch.Tensor):
        """Cut or tile a batch along dim 0 to the size the controller asked for."""
        out = []
        for t in tensors:
            n = t.shape[0]
            if n == self.batch_size:
                out.append(t)
            elif n > self.batch_size:
                out.append(t[: self.batch_size])
            else:
                reps = (self.batch_size + n - 1) // n
                out.append(t.repeat(reps, *([1] * (t.dim() - 1)))[: self.batch_size])
        return tuple(out)

    # ------------------------------------------------------------------ per step
    @contextlib.contextmanager
    def step(self):
        self._apply_due()
        e = self._ev
        e["f0"].record()
        marker = _BackwardStart(e["f1"])
        try:
            yield marker
        finally:
            e["b1"].record()
            e["b1"].synchronize()
            fwd = e["f0"].elapsed_time(e["f1"]) if marker.recorded else 0.0
            bwd = e["f1"].elapsed_time(e["b1"]) if marker.recorded else e["f0"].elapsed_time(e["b1"])
            gap = e["prev_b1"].elapsed_time(e["f0"]) if self._have_prev else 0.0
            e["prev_b1"], e["b1"] = e["b1"], e["prev_b1"]
            self._have_prev = True
            # bytes this rank stored into one peer (4-byte entries for tensors on the narrow wire format)
            nbytes = sum(rt.bucket.layout.wire_bytes() for rt in self.engine.buckets) * self.bytes_per_entry / 8.0
            step_ms = max(fwd + bwd + gap, 1e-3)
            mbps = nbytes * 8.0 * max(self.engine.world - 1, 0) / (step_ms * 1000.0)
            self.last = {"fwd_delay_ms": fwd, "bwd_delay_ms": bwd, "bwd_fwd_gap_ms": gap, "intra_fwd_gap_ms": 0.0,
                         "grad_send_thpt_mbps": mbps, "grad_recv_thpt_mbps": mbps}
            if self.client is not None and self.client.alive():
                cfg = self._TrainConfig(self.batch_size, self.engine.cfg.grad_accumulation, self.engine.cfg.ratio)
                self.client.report(self.iteration, cfg, [mbps, mbps, fwd, bwd, gap, 0.0], self._callback)
            self.iteration += 1


class _WeakInstruction:
    """Callback handed to the native client: holds the hook weakly, so that reports still queued in the client's
    thread never keep the hook (and through it the client itself) alive."""

    def __init__(self, hook) -> None:
        import weakref

        self._ref = weakref.ref(hook)

    def __call__(self, since: int, ubatch: int, grad_acc: int, ratio: float) -> None:
        hook = self._ref()
        if hook is not None:
            hook._on_instruction(since, ubatch, grad_acc, ratio)


class _BackwardStart:
    """``marker.backward_begins()`` between forward and backward splits the two device times."""

    def __init__(self, ev: torch.cuda.Event) -> None:
        self.ev, self.recorded = ev, False

    def backward_begins(self) -> None:
        self.ev.record()
        self.recorded = True
