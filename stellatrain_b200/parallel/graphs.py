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

from typing import Callable, Sequence

import torch

from .engine import SparseDPEngine


class GraphedStep:
    def __init__(self, engine: SparseDPEngine, step_fn: Callable, sample_inputs: Sequence[torch.Tensor],
                 warmup: int = 3) -> None:
        """``step_fn(*inputs)`` must run forward and backward and return the loss tensor."""
        if engine.transport == "nccl":
            raise NotImplementedError("graph capture is provided for the peer and local transports")
        self.engine = engine
        dev = engine.device
        self.static_inputs = [t.clone() for t in sample_inputs]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                step_fn(*self.static_inputs)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        if engine.dist_on:
            import torch.distributed as dist
            dist.barrier(engine.group)

        if engine.cfg.staleness == 1 and not all(rt.has_pending_apply for rt in engine.buckets):
            raise RuntimeError("capture needs a steady-state step: run at least one warm-up step first")
        before = [(rt.select_count, rt.apply_count) for rt in engine.buckets]
        kernels0 = engine.stats["kernels"]
        self.graph = torch.cuda.CUDAGraph()
        engine._capturing = True
        try:
            with torch.cuda.graph(self.graph, stream=side):
                self.loss = step_fn(*self.static_inputs)
                torch.cuda.current_stream(dev).wait_stream(engine.sparse_stream)
        finally:
            engine._capturing = False
        # capture only records: undo the host-side bookkeeping of the captured (not executed) step
        self._per_replay = []
        for rt, (s0, a0) in zip(engine.buckets, before):
            self._per_replay.append((rt.select_count - s0, rt.apply_count - a0))
            rt.select_count, rt.apply_count = s0, a0
            rt.apply_done = None          # events recorded under capture are not waitable outside
        self._kernels_per_replay = engine.stats["kernels"] - kernels0
        engine.stats["kernels"] = kernels0
        torch.cuda.synchronize(dev)

    def copy_inputs(self, *host_or_device_tensors: torch.Tensor) -> None:
        for dst, src in zip(self.static_inputs, host_or_device_tensors):
            dst.copy_(src, non_blocking=True)

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        eng = self.engine
        for rt, (ds, da) in zip(eng.buckets, self._per_replay):
            rt.select_count += ds
            rt.apply_count += da
        eng.stats["kernels"] += self._kernels_per_replay
        eng.stats["graph_replays"] = eng.stats.get("graph_replays", 0) + 1
        return self.loss
