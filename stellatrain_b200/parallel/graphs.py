"""Whole-step CUDA graph: forward, backward and the sparse kernels of every bucket in one launch.

The reference pays one host round trip per parameter tensor per iteration (hook, task creation, stage
scheduling: backend/src/engine/core.cpp:775-797, 1025-1095).  At ResNet-152's 467 tensors and batch 32 a
B200 finishes the kernels faster than the host can issue them, so the step is captured once in steady
state and replayed: the post-accumulate hooks run during capture and put the select/apply kernels of the
sparse stream into the same graph, ordered by the same events as in eager mode.

Epochs, optimiser step counters and thresholds live in device memory and advance inside the kernels, so a
replay is a complete training step; only the host-side counters of the engine are advanced here.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from .engine import SparseDPEngine


class GraphedStep:
    def __init__(self, engine: SparseDPEngine, step_fn: Callable, sample_inputs: Sequence[torch.Tensor],
                 warmup: int = 3, stream: Optional[torch.cuda.Stream] = None) -> None:
        """``step_fn(*inputs)`` must run forward and backward and return the loss tensor.  ``warmup`` eager steps on
        the sample inputs come first (0 when the caller has already run its own steps on ``stream``, which is then
        the stream of the capture: kernels were tuned and the allocator warmed there)."""
        if engine.transport == "nccl":
            raise NotImplementedError("graph capture is provided for the peer and local transports")
        self.engine = engine
        dev = engine.device
        self.static_inputs = [t.clone() for t in sample_inputs]
        side = stream if stream is not None else torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(0, warmup)):
                step_fn(*self.static_inputs)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        if engine.dist_on:
            import torch.distributed as dist
            dist.barrier(engine.group)

        if engine.cfg.staleness == 1 and not all(rt.has_pending_apply for rt in engine.buckets):
            raise RuntimeError("capture needs a steady-state step: run at least one eager step first")
        before = [(rt.select_count, rt.apply_count) for rt in engine.buckets]
        kernels0, shaped0 = engine.kernels_launched(), engine.shaped_bytes
        self.version = engine.capture_version
        self.graph = torch.cuda.CUDAGraph()
        engine.begin_capture()
        try:
            with torch.cuda.graph(self.graph, stream=side):
                self.loss = step_fn(*self.static_inputs)
                torch.cuda.current_stream(dev).wait_stream(engine.sparse_stream)
                if engine.cfg.step_clock:
                    engine.stamp(4)      # behind the join: (4) - (2) is the time the iteration waited for its bucket chains
        finally:
            # A replay reads the captured gradient addresses from pinned rows of its own and reads the gradients
            # themselves at those addresses: both stay alive as long as this object does.
            self._keepalive = engine.end_capture()
        # capture only records: undo the host-side bookkeeping of the captured (not executed) step
        self._per_replay = []
        for rt, (s0, a0) in zip(engine.buckets, before):
            self._per_replay.append((rt.select_count - s0, rt.apply_count - a0))
            rt.select_count, rt.apply_count = s0, a0
            rt.apply_done = None          # events recorded under capture are not waitable outside
            rt.select_done = None
        self._kernels_per_replay = engine.kernels_launched() - kernels0
        engine.stats["kernels"] -= self._kernels_per_replay
        self._shaped_per_replay = engine.shaped_bytes - shaped0
        engine.shaped_bytes = shaped0
        torch.cuda.synchronize(dev)

    @property
    def stale(self) -> bool:
        """True once the engine changed something that is baked into the captured launches (the compression ratio)."""
        return self.version != self.engine.capture_version

    def copy_inputs(self, *host_or_device_tensors: torch.Tensor) -> None:
        for dst, src in zip(self.static_inputs, host_or_device_tensors):
            dst.copy_(src, non_blocking=True)

    def replay(self) -> torch.Tensor:
        eng = self.engine
        if self.stale:
            raise RuntimeError("this captured step is stale (the compression ratio changed): capture a new one")
        if eng._failed is not None:
            raise eng._failed
        eng.before_iteration(torch.cuda.current_stream(eng.device))
        self.graph.replay()
        for rt, (ds, da) in zip(eng.buckets, self._per_replay):
            rt.select_count += ds
            rt.apply_count += da
        eng.stats["kernels"] += self._kernels_per_replay
        eng.stats["graph_replays"] = eng.stats.get("graph_replays", 0) + 1
        eng.shaped_bytes = eng.shaped_bytes + self._shaped_per_replay
        n = eng.stats["graph_replays"]
        if eng.cfg.status_poll_interval and n % eng.cfg.status_poll_interval == 0:
            eng._poll_status()
        return self.loss
