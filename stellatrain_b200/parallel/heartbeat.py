"""Host-side failure detection for the GPU-resident engine.

The reference has no failure detection: a dead peer blocks a socket receive or a barrier forever
(backend/src/engine/comm_manager.cpp:833-974 and core_module_api.cpp:113-199 have neither heartbeats nor socket timeouts).  Here three layers cooperate:

1. every device-side wait is bounded and leaves a status word (``SparseStepError``);
2. this module: each rank publishes a heartbeat in the job's key-value store from a small thread, and
   ``HeartbeatMonitor.check()`` called between steps raises ``PeerLostError`` when a peer has been silent for too
   long or has announced that it is leaving, *before* the next kernels that would wait for it are launched;
3. policy: ``abort`` (raise) or ``shrink``: the survivors agree on the new membership through the store, and the
   caller rebuilds its process group and engine from the last checkpoint (``utils.checkpoint.load(...,
   allow_world_change=True)``).

A rank leaves only between steps (``announce_leave``) with none of its kernels in flight.  All of this is host
code and is tested with CPU ranks.
"""
from __future__ import annotations

import threading
import time
from typing import Iterable, List, Optional


class PeerLostError(RuntimeError):
    def __init__(self, lost: List[int], reason: str) -> None:
        super().__init__(f"rank(s) {lost} lost: {reason}")
        self.lost = lost


class HeartbeatMonitor:
    """``store`` is any object with ``set(key, bytes|str)`` and ``get(key)`` that blocks or raises for a
    missing key and supports ``check([keys])`` or ``num_keys`` - a ``torch.distributed.TCPStore`` does."""

    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5, timeout_s: float = 5.0,
                 prefix: str = "hb", startup_timeout_s: Optional[float] = None) -> None:
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        # a peer that has not published anything yet is still starting (processes of one job come up seconds
        # apart): it gets a longer limit than a peer that was heard and then fell silent
        self.startup_timeout_s = max(timeout_s, 30.0) if startup_timeout_s is None else startup_timeout_s
        self._stop = threading.Event()
        self._beat(0)
        self._last_seen = {r: (-1, time.monotonic()) for r in range(world)}
        self._thread = threading.Thread(target=self._main, daemon=True, name="Heartbeat")
        self._thread.start()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def _beat(self, n: int) -> None:
        self.store.set(self._key(self.rank), str(n))

    def _main(self) -> None:
        n = 1
        while not self._stop.wait(self.interval_s):
            try:
                self._beat(n)
            except Exception:  # noqa: BLE001 - the store itself went away: the next check() reports it
                return
            n += 1

    def _read(self, r: int) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            v = self.store.get(self._key(r))
            return v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
        except Exception:  # noqa: BLE001
            return None

    def check(self) -> None:
        """Raises ``PeerLostError`` if a peer left or has not beaten within ``timeout_s``."""
        now = time.monotonic()
        lost, reason = [], ""
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v == "left":
                lost.append(r)
                reason = "announced that it is leaving"
                continue
            count = int(v) if v not in (None, "") and v.lstrip("-").isdigit() else -1
            prev, when = self._last_seen[r]
            if count > prev:
                self._last_seen[r] = (count, now)
            elif now - when > (self.timeout_s if prev >= 0 else self.startup_timeout_s):
                lost.append(r)
                reason = reason or f"no heartbeat for {now - when:.1f} s"
        if lost:
            raise PeerLostError(sorted(lost), reason)

    def announce_leave(self) -> None:
        """Call between steps, after ``engine.synchronize()``: tells the peers not to wait for this rank."""
        self._stop.set()
        self._thread.join(timeout=2 * self.interval_s + 1)
        self.store.set(self._key(self.rank), "left")

    def close(self) -> None:
        self._stop.set()


def agree_on_survivors(store, rank: int, old_world: int, lost: Iterable[int], generation: int, timeout_s: float = 10.0) -> List[int]:
    """Survivors publish the set they believe alive; the membership of generation g is the intersection of what
    every believed-alive rank published.  Returns the sorted list of surviving old ranks (new rank = position)."""
    alive = sorted(set(range(old_world)) - set(lost))
    store.set(f"members/{generation}/{rank}", ",".join(map(str, alive)))
    deadline = time.monotonic() + timeout_s
    views = {}
    while time.monotonic() < deadline and len(views) < len(alive):
        for r in alive:
            if r in views:
                continue
            try:
                if hasattr(store, "check") and not store.check([f"members/{generation}/{r}"]):
                    continue
                v = store.get(f"members/{generation}/{r}")
                v = v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
                views[r] = set(int(x) for x in v.split(",") if x)
            except Exception:  # noqa: BLE001
                continue
        time.sleep(0.02)
    members = set(alive)
    for r, view in views.items():
        members &= view
    members &= set(views)            # a rank that published nothing in time is not part of the new job
    return sorted(members)
