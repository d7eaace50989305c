"""Tracing and timing (the reference's NVTX ranges and per-task stage timers,
backend/src/engine/core_internal.h:11-16, backend/src/engine/core.cpp:1151-1207).

* ``nvtx_range``: context manager around ``torch.cuda.nvtx`` (no-op without CUDA).
* ``StepTimer``: CUDA-event timers per named stage with a bounded history and the reference's JSON export
  ``{key: {event: ms}}`` to ``/tmp/time_log_<timestamp>_<pid>.json``.
* ``StepMeasurements``: the six telemetry fields of the reference's schema
  (backend/src/proto/message.proto:11-18) measured on the device: forward and backward time, the gap
  between backward end and the next forward start, and the time the forward was blocked on updates.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import OrderedDict, deque
from typing import Deque, Dict, Optional, Tuple

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class StepTimer:
    def __init__(self, capacity: int = 4096, enabled: bool = True) -> None:
        self.enabled = enabled and torch.cuda.is_available()
        self.pending: Deque[Tuple[str, str, torch.cuda.Event, torch.cuda.Event]] = deque()
        self.history: "OrderedDict[str, Dict[str, float]]" = OrderedDict()
        self.capacity = capacity

    @contextlib.contextmanager
    def stage(self, key: str, event: str, stream: Optional[torch.cuda.Stream] = None):
        if not self.enabled:
            yield
            return
        s = stream or torch.cuda.current_stream()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(s)
        with nvtx_range(f"{event}-{key}"):
            yield
        b.record(s)
        self.pending.append((key, event, a, b))

    def collect(self) -> None:
        """Move finished measurements into the history without blocking."""
        while self.pending and self.pending[0][3].query():
            key, event, a, b = self.pending.popleft()
            self.history.setdefault(key, {})[event] = a.elapsed_time(b)
            while len(self.history) > self.capacity:
                self.history.popitem(last=False)

    def export_json(self, path: Optional[str] = None) -> str:
        self.collect()
        path = path or f"/tmp/time_log_{time.strftime('%Y%m%d%H%M%S')}_{os.getpid()}.json"
        with open(path, "w") as f:
            json.dump(self.history, f)
        return path


class StepMeasurements:
    """Forward/backward times and gaps of the last completed step, measured with CUDA events."""

    def __init__(self) -> None:
        self.ev = {k: torch.cuda.Event(enable_timing=True) for k in ("fwd0", "fwd1", "bwd1", "next_fwd0")}
        self.last: Dict[str, float] = {"fwd_delay_ms": 0.0, "bwd_delay_ms": 0.0, "bwd_fwd_gap_ms": 0.0,
                                       "intra_fwd_gap_ms": 0.0}
        self._have = False

    def mark(self, name: str) -> None:
        self.ev[name].record()

    def finish_step(self) -> Dict[str, float]:
        """Call right after marking ``next_fwd0`` (the start of the following forward)."""
        self.ev["next_fwd0"].synchronize()
        self.last["fwd_delay_ms"] = self.ev["fwd0"].elapsed_time(self.ev["fwd1"])
        self.last["bwd_delay_ms"] = self.ev["fwd1"].elapsed_time(self.ev["bwd1"])
        self.last["bwd_fwd_gap_ms"] = self.ev["bwd1"].elapsed_time(self.ev["next_fwd0"])
        return dict(self.last)
