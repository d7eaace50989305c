"""Link shaping for grouped topologies: a seeded, time-varying bandwidth schedule and a token bucket.

An NVSwitch box has no slow link, so a constrained cross-group link (10-40 Gbps, changing over time) is
emulated: the schedule says how many bytes per second the link offers at time t, and a token bucket
decides how long a payload has to wait.  ``TokenBucket`` keeps the bucket on the host (CPU tier, tests);
``DeviceTokenBucket`` keeps it in GPU memory, where a one-thread kernel in front of a bucket's push takes
the payload's bytes and holds the sparse stream while the bucket is in debt
(``SparseDPEngine.set_link_shaper``).  State and clock are the GPU's own, so the shaper runs unchanged inside
a captured step.  The measured rate that results is what the telemetry reports, so the controller sees the
shaped link, not NVLink.
"""
from __future__ import annotations

import math
import random
import time
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class BandwidthSchedule:
    """Piecewise-constant Gbps levels, drawn once from ``seed``, each lasting ``period_s`` seconds."""

    seed: int = 0
    lo_gbps: float = 10.0
    hi_gbps: float = 40.0
    period_s: float = 2.0
    levels: int = 64
    _table: List[float] = field(default_factory=list)

    def __post_init__(self) -> None:
        rng = random.Random(self.seed)
        self._table = [rng.uniform(self.lo_gbps, self.hi_gbps) for _ in range(self.levels)]

    def gbps_at(self, t_s: float) -> float:
        return self._table[int(max(t_s, 0.0) / self.period_s) % self.levels]

    def bytes_per_s_at(self, t_s: float) -> float:
        return self.gbps_at(t_s) * 1e9 / 8.0


class TokenBucket:
    """Classic token bucket whose fill rate follows a schedule; ``burst_bytes`` bounds what may be sent
    without waiting."""

    def __init__(self, schedule: BandwidthSchedule, burst_bytes: int = 1 << 20, clock=time.monotonic) -> None:
        self.schedule = schedule
        self.burst = float(burst_bytes)
        self.clock = clock
        self.t0 = clock()
        self.last = self.t0
        self.tokens = self.burst
        self.sent_bytes = 0
        self.waited_s = 0.0

    def _refill(self, now: float) -> None:
        dt = max(0.0, now - self.last)
        self.tokens = min(self.burst, self.tokens + dt * self.schedule.bytes_per_s_at(self.last - self.t0))
        self.last = now

    def delay_for(self, nbytes: int) -> float:
        """Seconds the caller has to wait before ``nbytes`` may go out (tokens are taken now)."""
        now = self.clock()
        self._refill(now)
        self.tokens -= nbytes
        self.sent_bytes += nbytes
        if self.tokens >= 0:
            return 0.0
        rate = self.schedule.bytes_per_s_at(now - self.t0)
        wait = -self.tokens / max(rate, 1.0)
        self.waited_s += wait
        return wait

    def throttle(self, nbytes: int, sleep=time.sleep) -> float:
        w = self.delay_for(nbytes)
        if w > 0:
            sleep(w)
        return w

    def achieved_gbps(self) -> float:
        dt = max(self.clock() - self.t0, 1e-9)
        return self.sent_bytes * 8.0 / dt / 1e9


class DeviceTokenBucket:
    """The same token bucket, resident on a GPU (``csrc/cuda/aux_kernels.cu``: ``k_shape``).

    ``share`` divides the schedule's rate: the ranks of one group share the group's link, so each of them
    shapes its own sends to 1 / group size of the scheduled rate.  The schedule starts at the first send."""

    MAX_HOLD_NS = 2_000_000_000      # no single wait holds a stream longer than this

    def __init__(self, schedule: BandwidthSchedule, device, burst_bytes: int = 1 << 20, share: float = 1.0) -> None:
        import numpy as np
        import torch

        from .. import _build

        self._C = _build.load_extension("_C")
        self.schedule, self.share, self.burst = schedule, float(share), float(burst_bytes)
        levels = min(len(schedule._table), self._C.SHAPER_LEVELS)
        raw = np.zeros(self._C.SIZEOF_SHAPER_STATE, dtype=np.uint8)
        head = np.dtype([("tokens", "<f8"), ("last_ns", "<u8"), ("t0_ns", "<u8"), ("sent_bytes", "<u8"), ("waited_ns", "<u8"),
                         ("burst_bytes", "<f4"), ("period_s", "<f4"), ("levels", "<u4"), ("reserved", "<u4")])
        self._head = head
        h = raw[: head.itemsize].view(head)
        h["burst_bytes"], h["period_s"], h["levels"] = self.burst, schedule.period_s, levels
        rates = raw[head.itemsize: head.itemsize + 4 * self._C.SHAPER_LEVELS].view("<f4")
        rates[:levels] = [g * 1e9 / 8.0 * self.share for g in schedule._table[:levels]]
        self.state = torch.from_numpy(raw.copy()).to(device)
        self.device = device

    def take(self, nbytes: int, stream) -> None:
        """Enqueue on ``stream``: take ``nbytes`` from the bucket, hold the stream while it is in debt."""
        if nbytes > 0:
            self._C.shape(self.state.data_ptr(), int(nbytes), self.MAX_HOLD_NS, stream.cuda_stream)

    def stats(self) -> dict:
        """Blocking read of the device state: bytes sent, seconds waited, seconds since the first send."""
        import torch

        h = self.state[: self._head.itemsize].cpu().numpy().view(self._head)[0]
        torch.cuda.synchronize(self.device)
        span_s = max(float(int(h["last_ns"]) - int(h["t0_ns"])) * 1e-9, 1e-9) if int(h["last_ns"]) else 0.0
        return {"sent_bytes": int(h["sent_bytes"]), "waited_s": int(h["waited_ns"]) * 1e-9, "span_s": span_s}

    def achieved_gbps(self) -> float:
        st = self.stats()
        return st["sent_bytes"] * 8.0 / st["span_s"] / 1e9 if st["span_s"] > 0 else 0.0

    def scheduled_mean_gbps(self) -> float:
        """Mean of the schedule over the time the bucket has been in use (this rank's share of it)."""
        st = self.stats()
        if st["span_s"] <= 0:
            return 0.0
        n = max(1, int(st["span_s"] / self.schedule.period_s + 0.999))
        return sum(self.schedule.gbps_at(i * self.schedule.period_s) for i in range(n)) / n * self.share
