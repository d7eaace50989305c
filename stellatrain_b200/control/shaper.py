"""Link shaping for grouped topologies: a seeded, time-varying bandwidth schedule and a token bucket.

An NVSwitch box has no slow link, so a constrained cross-group link (10-40 Gbps, changing over time) is
emulated: the schedule says how many bytes per second the link offers at time t, the token bucket
tells a sender how long a payload has to wait, and the engine delays the cross-group push of a bucket on
the host by that much (``SparseDPEngine.set_link_shaper``).  The measured rate that results is what the
telemetry reports, so the controller sees the shaped link, not NVLink.
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
