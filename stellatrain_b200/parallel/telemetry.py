"""Connects a training loop to the controller: measures every step, reports, applies instructions.

The reference defines the client (backend/src/engine/telemetry_client.cpp:39-110) and the instruction
protocol (effective a few iterations after issue, backend/src/engine/batch_rate_alloc_optim.py:454-479)
but never instantiates them in its engine.  Here the loop is closed:

    hook = TelemetryHook(engine, "tcp://127.0.0.1:5556", batch_size=32)
    for x, y in loader:
        x, y = hook.resize_batch(x, y)          # per-GPU batch size the controller asked for
        with hook.step():                       # times forward/backward, reports, applies instructions
            loss = criterion(model(x), y); loss.backward()

    # or, with the wrapper's whole-iteration call (eager or replayed from a CUDA graph):
    loss = hook.run(model, x, y)

Measurements are device times: three one-thread kernels write the GPU's clock when the compute stream reaches
the start of the forward pass (behind the wait for the updates this forward must see), the start of backward and
its end, so the numbers are the same whether the iteration is launched kernel by kernel or replayed from a graph.
They give forward, backward and the exposed communication: the time the stream was blocked on outstanding updates or on
the shaped link (the wait in front of an eagerly launched forward, or the join behind a captured iteration).
The stamps of iteration i are read while iteration i + 1 runs, so nothing here makes the host wait for the GPU.
Throughput fields come from the bytes the engine pushed during the step.
"""
from __future__ import annotations

import contextlib
import threading
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


class TelemetryHook:
    def __init__(self, engine, uri: Optional[str], batch_size: int, gpu_name: Optional[str] = None,
                 apply_batch: bool = True, apply_ratio: bool = True, link_bytes_per_entry: int = 8,
                 ratio_tolerance: float = 0.15, ratio_min_interval: int = 0) -> None:
        self.engine = engine
        self.batch_size = int(batch_size)
        self.apply_batch, self.apply_ratio = apply_batch, apply_ratio
        self.bytes_per_entry = link_bytes_per_entry
        # A new ratio drains the pipeline and makes a captured step stale, so one that moves the kept fraction by
        # less than this (relative) is not worth applying; the controller re-issues its current view every few
        # iterations anyway (backend/src/engine/batch_rate_alloc_optim.py:454-472).
        self.ratio_tolerance = float(ratio_tolerance)
        # Iterations that must lie between two applied ratio changes.  With captured iterations every change costs an
        # eager iteration and a new capture (about as much as fifty replays of a 20 ms step), so a controller that
        # walks the ratio a little every few iterations is followed in larger steps.
        self.ratio_min_interval = int(ratio_min_interval)
        self._last_ratio_change = -(1 << 30)
        self.iteration = 0
        self.pending: List[Tuple[int, int, float]] = []      # (effective_since, ubatch, ratio)
        self.applied: List[Tuple[int, int, float]] = []
        self.lock = threading.Lock()
        self.client = None
        self._callback = _WeakInstruction(self)
        self._ring = [torch.zeros(5, dtype=torch.int64).pin_memory() for _ in range(4)]   # stamps of the last iterations
        self._ring_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._prev_b1 = 0             # device clock at the end of the previous measured backward
        engine.cfg.step_clock = True  # the engine stamps the start of every forward behind its gate
        self.last: Dict[str, float] = {}
        self._agree_event = None
        self._agree_dev = torch.zeros(1, dtype=torch.float64, device=engine.device)
        self._agree_host = torch.zeros(1, dtype=torch.float64).pin_memory()
        if uri:
            from .. import cpu_tier

            ext = cpu_tier._load()
            name = gpu_name or (torch.cuda.get_device_name(engine.device) if engine.device.type == "cuda" else "cpu")
            self._TrainConfig = ext.TrainConfig
            # the controller may be busy when a job starts (it fits and optimises under the interpreter lock of its
            # own process): a registration that is not answered in time is tried again before giving up
            last = None
            for _ in range(3):
                try:
                    self.client = ext.TelemetryClient(cpu_tier.prepare_telemetry_uri(uri), engine.rank, name, 0, engine.rank, 10000)
                    break
                except RuntimeError as e:
                    last = e
            if self.client is None:
                raise last

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
                target, now = max(ratio, lo), self.engine.cfg.ratio
                kept_now, kept_new = max(1.0 - now, 1e-9), max(1.0 - target, 1e-9)
                if (abs(kept_new - kept_now) > self.ratio_tolerance * kept_now and
                        self.iteration - self._last_ratio_change >= self.ratio_min_interval):
                    self.engine.set_compression_ratio(target)
                    self._last_ratio_change = self.iteration
            self.applied.append((since, ubatch, ratio))
        if due and self.apply_batch and self.engine.world > 1:
            # unequal batches: weight each rank's gradient by its share of the global batch
            t = torch.tensor([float(self.batch_size)], device=self.engine.device)
            all_b = [torch.zeros_like(t) for _ in range(self.engine.world)]
            dist.all_gather(all_b, t, group=self.engine.group)
            b = torch.cat(all_b)
            # from the coming iteration on, which is the same one on every rank; nothing is drained
            self.engine.set_rank_weights((b / b.sum()).tolist(), from_iteration=self.engine.iterations_started())

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
    def begin(self) -> None:
        """Start of an iteration: instructions whose effective iteration has come are applied."""
        self._apply_due()

    def end(self) -> None:
        """End of an iteration (everything enqueued): its stamps travel to pinned memory behind it, and the
        iteration before it, whose stamps have landed, is measured and reported."""
        eng = self.engine
        slot = self.iteration % len(self._ring)
        if hasattr(eng, "step_stamps"):
            self._ring[slot].copy_(eng.step_stamps[:5], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._ring_events[slot] = ev
        if self.iteration > 0:
            self._measure(self.iteration - 1)
        self.iteration += 1

    def flush(self) -> None:
        """Measure and report the latest iteration too (end of training)."""
        if self.iteration > 0:
            self._measure(self.iteration - 1)

    def _measure(self, it: int) -> None:
        slot = it % len(self._ring)
        ev = self._ring_events[slot]
        if ev is None:
            return
        ev.synchronize()
        self._ring_events[slot] = None
        f0, f1, b1, pre, joined = (int(v) for v in self._ring[slot])
        if not (f0 and b1):
            return
        split = f0 <= f1 <= b1                 # the start of backward was stamped in this iteration
        fwd = (f1 - f0) / 1e6 if split else 0.0
        bwd = (b1 - f1) / 1e6 if split else (b1 - f0) / 1e6
        # Exposed communication, on the device's clock: a captured iteration ends with a join of its bucket chains
        # (stamp 4 behind it), an eagerly launched one waits at the start of the next forward (stamp 3 in front).
        # Host-side pauses (a new capture, a slow launch loop) are in neither, unlike in the distance between the end
        # of one backward and the start of the next forward.
        if joined >= b1:
            gap = (joined - b1) / 1e6
        elif 0 < pre <= f0:
            gap = (f0 - pre) / 1e6
        else:
            gap = 0.0
        self._prev_b1 = b1
        # bytes this rank stored into one peer (4-byte entries for tensors on the narrow wire format)
        nbytes = sum(rt.bucket.layout.wire_bytes() for rt in self.engine.buckets) * self.bytes_per_entry / 8.0
        step_ms = max(fwd + bwd + gap, 1e-3)
        mbps = nbytes * 8.0 * max(self.engine.world - 1, 0) / (step_ms * 1000.0)
        if self.engine.shaper is not None:
            # a shaped cross-group link: what the controller has to fit is the traffic that crosses it
            mbps = self.engine.shaped_bytes_per_step() * 8.0 / (step_ms * 1000.0)
        self.last = {"fwd_delay_ms": fwd, "bwd_delay_ms": bwd, "bwd_fwd_gap_ms": gap, "intra_fwd_gap_ms": 0.0,
                     "grad_send_thpt_mbps": mbps, "grad_recv_thpt_mbps": mbps}
        if self.client is not None and self.client.alive():
            cfg = self._TrainConfig(self.batch_size, self.engine.cfg.grad_accumulation, self.engine.cfg.ratio)
            self.client.report(it, cfg, [mbps, mbps, fwd, bwd, gap, 0.0], self._callback)

    @contextlib.contextmanager
    def step(self):
        """Around a hand-written iteration: ``marker.backward_begins()`` between forward and backward."""
        self.begin()
        marker = _BackwardStart(self.engine)
        try:
            yield marker
        finally:
            self.engine.stamp(2)
            self.end()

    def run(self, net, *inputs: torch.Tensor) -> torch.Tensor:
        """One whole iteration through the wrapper (``net.train_step``), eager or replayed from a CUDA graph."""
        self.begin()
        try:
            return net.train_step(*inputs)
        finally:
            self.end()


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

    def __init__(self, engine) -> None:
        self.engine, self.recorded = engine, False

    def backward_begins(self) -> None:
        self.engine.stamp(1)
        self.recorded = True
