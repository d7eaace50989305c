"""Batch-size and compression-ratio optimiser of the controller.

Rebuild of the reference's ``MainOptimizer`` / ``GpuThroughputEstimator``
(backend/src/engine/batch_rate_alloc_optim.py:14-524):

* per-GPU compute model f(x) = min(beta / alpha * x, beta) items/s, fitted by Nelder-Mead least squares
  on (batch, batch * 1000 / bwd_ms) samples that are smoothed per batch size (lines 37-68, 404-427);
* phases INIT_WARMUP (collect 4 samples per GPU) -> INIT_COLLECT_X (ramp every GPU's batch by 1.5x up to
  its maximum) -> RUNNING (lines 105-108, 386-452);
* bandwidth estimate from exposed communication: r = wait / (wait + comp) with
  wait = min_i(bwd_fwd_gap + intra_fwd_gap), comp = mean(1.5 bwd_ms); smoothed 0.9/0.1, then x1.1 when
  r < 0.05 else x max(0.75, 1 - r) (lines 203-233);
* objective g(x) = (1 + 50 h(sum x, T c)) / (sum x / max_k x_k / f_k(x_k)) + lambda2 CoV_k(x_k / f_k(x_k))
  minimised over per-GPU batches with Nelder-Mead, 32 random starts the first time, warm starts later,
  re-solved every 100 controller steps (lines 178-201, 297-322);
* compression ratio: smallest ratio whose required goodput fits the estimate (20-step bisection on
  [0, 0.999]), then spread over the other nodes (lines 264-295, 332-335);
* at most one instruction per 4 (5 when running) observed iterations, effective 3 iterations after the
  latest observed one (lines 14-18, 454-479).

What differs: the byte model knows this package's wire formats (8-byte entries pushed over NVLink, or the
TCP frames of the CPU tier) next to the reference's ZeroMQ/TCP estimate; the profile h comes from
``gp_profile`` (no pickles); the fit bounds are parameters because a B200 is not a 2080 Ti.
"""
from __future__ import annotations

import math
import random
from collections import OrderedDict
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
from scipy.optimize import minimize

from .gp_profile import AnalyticProfile

GPU_INIT_WARMUP_THRESH = 4
GPU_POINT_RELIABLE_THRESH = 4
EFFECTIVE_AFTER_ITER = 3
WAIT_EFFECT_ITER = 4
WAIT_EFFECT_ITER_MAIN = 5

# Per-GPU batch ceilings by device name (reference batch_rate_alloc.py:16-22), extended for this target.
MAX_BATCH_SIZE_MAP = {
    "NVIDIA GeForce RTX 4090": 90, "NVIDIA GeForce RTX 3090": 90, "NVIDIA GeForce RTX 2080 Ti": 36,
    "NVIDIA A100-SXM4-40GB": 120, "Tesla V100-SXM2-32GB": 112,
    "NVIDIA B200": 1024, "NVIDIA H100 80GB HBM3": 512, "cpu": 64,
}


def max_batch_for(gpu_name: str, default: int = 256) -> int:
    return MAX_BATCH_SIZE_MAP.get(gpu_name, default)


class Phase(Enum):
    INIT_WARMUP = 0
    INIT_COLLECT_X = 1
    RUNNING = 2


@dataclass
class InstructionSet:
    iter: int                       # effective from this iteration on
    batch: np.ndarray               # per GPU
    comp_ratio: float


class SmoothedSamples:
    """One exponentially smoothed throughput value per batch size."""

    def __init__(self, momentum: float = 0.9) -> None:
        self.values: Dict[int, float] = {}
        self.momentum = momentum
        self.count = 0

    def add(self, batch: int, thpt: float) -> None:
        old = self.values.get(batch)
        self.values[batch] = thpt if old is None else old * self.momentum + thpt * (1.0 - self.momentum)
        self.count += 1

    def items(self):
        return list(self.values.items())


def saturating(alpha, beta, x):
    """f(x) = min(beta / alpha * x, beta): linear until the device is full, flat afterwards."""
    x = np.asarray(x, dtype=float)
    return np.minimum(np.asarray(beta, float) / np.asarray(alpha, float) * x, beta)


def fit_alpha_beta(samples: Sequence, guess, alpha_min: float, beta_min: float):
    if len(samples) < 2:
        return guess
    xs, ys = (np.asarray(v, float) for v in zip(*samples))

    def err(p):
        return float(np.sum((saturating(p[0], p[1], xs) - ys) ** 2))

    g = np.maximum(np.asarray(guess, float), [alpha_min, beta_min])
    r = minimize(err, g, method="Nelder-Mead", bounds=((alpha_min, None), (beta_min, None)))
    return float(r.x[0]), float(r.x[1])


@dataclass
class TrafficModel:
    """Bytes a rank puts on the constrained link per iteration at a given compression ratio."""

    param_counts: List[int]
    transport: str = "nvlink"        # "nvlink": 8-byte entries + one flag per bucket; "tcp": framed, with headers
    grad_fp16: bool = False
    grad_idx_u16: bool = False
    buckets: int = 8
    grad_block16: bool = False       # "tcp" only: entries travel as whole blocks of 16 behind one block id

    def tx_bytes(self, ratio: float) -> int:
        ratio = min(max(ratio, 0.0), 0.999999)
        total = 0
        for n in self.param_counts:
            k = int(max(1, math.ceil((1.0 - ratio) * n)))
            idx_b = 2 if (self.grad_idx_u16 and n < 65536) else 4
            val_b = 2 if self.grad_fp16 else 4
            if self.transport == "nvlink":
                total += 8 * k if not (self.grad_fp16 or self.grad_idx_u16) else (idx_b + val_b) * k
            else:
                if self.grad_block16 and k >= 16:
                    blk_b = 2 if n <= (1 << 20) else 4
                    arrays = 4 + (k // 16) * blk_b + (k % 16) * idx_b + val_b * k
                else:
                    arrays = (idx_b + val_b) * k
                payload = 24 + 16 + 4 + arrays                           # frame header, key, count, arrays
                mss = 1538 - 0x42
                total += payload + math.ceil(payload / mss) * 0x42       # Ethernet/IP/TCP per segment
        if self.transport == "nvlink":
            total += 8 * self.buckets
        return total

    def goodput_mbps(self, ratio: float, iter_ms: float) -> float:
        return self.tx_bytes(ratio) * 8.0 / (max(iter_ms, 1e-6) * 1000.0)


class BatchRateOptimizer:
    def __init__(self, num_gpus: int, num_nodes: int, traffic: TrafficModel, profile=None,
                 latest_iter: Optional[Callable[[], int]] = None, alpha_min: float = 1.0, beta_min: float = 1.0,
                 lambda_2: float = 5.0, seed: int = 0, reoptimize_every: int = 100) -> None:
        self.num_gpus, self.num_nodes = num_gpus, num_nodes
        self.traffic = traffic
        self.profile = profile or AnalyticProfile()
        self.latest_iter = latest_iter or (lambda: 0)
        self.alpha_min, self.beta_min, self.lambda_2 = alpha_min, beta_min, lambda_2
        self.reoptimize_every = reoptimize_every
        self.alphas = np.full(num_gpus, max(10.0, alpha_min))
        self.betas = np.full(num_gpus, max(200.0, beta_min))
        self.max_batch = np.full(num_gpus, np.inf)
        # Smallest batch size every GPU has been measured at.  The allocation never goes below it: two parameters are
        # fitted to the samples, and when all samples lie on the flat part of the curve (a fast GPU whose run started
        # at a batch beyond its knee) the knee is not determined by them, so a batch below the sampled range would
        # rest on the initial guess alone.  The reference ramps up from a batch of 4 and always has the low end
        # (backend/src/engine/batch_rate_alloc_optim.py:203-215); a job that starts at its working batch does not.
        self.min_sampled = np.full(num_gpus, np.inf)
        self.samples = [SmoothedSamples() for _ in range(num_gpus)]
        self.seen = [0] * num_gpus
        self.initialized = [False] * num_gpus
        self.init_batch = np.zeros(num_gpus)
        self.init_ratio = 0.0
        self.history: "OrderedDict[int, InstructionSet]" = OrderedDict()
        self.phase = Phase.INIT_WARMUP
        self.bw_estimate: Optional[float] = None      # Mbps on the constrained link
        self.prev_x: Optional[np.ndarray] = None
        self.prev_fun = 0.0
        self.main_iter = 0
        self.rng = random.Random(seed)
        self.last_rows: Dict[int, dict] = {}
        self.log: List[str] = []

    # ---------------------------------------------------------------- persistence
    def state_dict(self) -> dict:
        """What a restarted controller needs to carry on where it was: the fitted per-GPU throughput curves, the
        smoothed samples behind them, the phase, the bandwidth estimate and the instruction history (the state the
        reference keeps only in memory, backend/src/engine/batch_rate_alloc_optim.py:117-162)."""
        return {
            "alphas": self.alphas.copy(), "betas": self.betas.copy(), "max_batch": self.max_batch.copy(),
            "min_sampled": self.min_sampled.copy(),
            "samples": [{"values": dict(s.values), "count": s.count, "momentum": s.momentum} for s in self.samples],
            "seen": list(self.seen), "initialized": list(self.initialized), "init_batch": self.init_batch.copy(),
            "init_ratio": self.init_ratio, "phase": int(self.phase.value), "bw_estimate": self.bw_estimate,
            "prev_x": None if self.prev_x is None else self.prev_x.copy(), "prev_fun": self.prev_fun,
            "main_iter": self.main_iter, "rng": self.rng.getstate(),
            "history": [(i.iter, i.batch.copy(), i.comp_ratio) for i in self.history.values()],
        }

    def load_state_dict(self, sd: dict) -> None:
        if len(sd["alphas"]) != self.num_gpus:
            raise ValueError(f"controller state is for {len(sd['alphas'])} GPUs, this job has {self.num_gpus}")
        self.alphas, self.betas = np.array(sd["alphas"], float), np.array(sd["betas"], float)
        self.max_batch = np.array(sd["max_batch"], float)
        self.min_sampled = np.array(sd.get("min_sampled", np.full(self.num_gpus, np.inf)), float)
        self.samples = []
        for row in sd["samples"]:
            s = SmoothedSamples(row["momentum"])
            s.values, s.count = {int(k): float(v) for k, v in row["values"].items()}, int(row["count"])
            self.samples.append(s)
        self.seen, self.initialized = list(sd["seen"]), list(sd["initialized"])
        self.init_batch, self.init_ratio = np.array(sd["init_batch"], float), float(sd["init_ratio"])
        self.phase = Phase(sd["phase"])
        self.bw_estimate = sd["bw_estimate"]
        self.prev_x = None if sd["prev_x"] is None else np.array(sd["prev_x"], float)
        self.prev_fun, self.main_iter = float(sd["prev_fun"]), int(sd["main_iter"])
        self.rng.setstate(sd["rng"])
        self.history = OrderedDict((it, InstructionSet(it, np.array(b, float), float(r))) for it, b, r in sd["history"])

    # ---------------------------------------------------------------- telemetry in
    def set_max_batch(self, gpu: int, value: int) -> None:
        self.max_batch[gpu] = value

    def update(self, rows: Sequence[dict]) -> None:
        """rows: dicts with gpu, batch_size, bwd_ms, fwd_ms, comp_ratio, bwd_fwd_gap_ms, intra_fwd_gap_ms."""
        for row in rows:
            g = row["gpu"]
            if self.seen[g] >= GPU_INIT_WARMUP_THRESH and row["bwd_ms"] > 0:
                self.samples[g].add(int(row["batch_size"]), row["batch_size"] * 1000.0 / row["bwd_ms"])
                self.min_sampled[g] = min(self.min_sampled[g], float(row["batch_size"]))
            self.seen[g] += 1
            self.last_rows[g] = row
            if self.phase == Phase.INIT_WARMUP:
                self.initialized[g] = True
                self.init_ratio = row["comp_ratio"]
                self.init_batch[g] = row["batch_size"]
        self._fit()
        if self.phase == Phase.INIT_WARMUP:
            if all(self.initialized) and 0 not in self.history:
                self.history[0] = InstructionSet(0, self.init_batch.copy(), self.init_ratio)
            if all(s.count >= GPU_INIT_WARMUP_THRESH for s in self.samples):
                self.phase = Phase.INIT_COLLECT_X

    def _fit(self) -> None:
        for g in range(self.num_gpus):
            if self.samples[g].count < GPU_POINT_RELIABLE_THRESH:
                continue
            self.alphas[g], self.betas[g] = fit_alpha_beta(self.samples[g].items(), (self.alphas[g], self.betas[g]),
                                                          self.alpha_min, self.beta_min)

    # ---------------------------------------------------------------- objective
    def f(self, x: np.ndarray) -> np.ndarray:
        return saturating(self.alphas, self.betas, x)

    def iteration_seconds(self, x: np.ndarray) -> np.ndarray:
        return x / np.maximum(self.f(x), 1e-9)

    def objective(self, x: np.ndarray, bandwidth_mbps: float, conversion: float) -> float:
        x = np.maximum(np.round(np.asarray(x, float)), 1.0)
        t = self.iteration_seconds(x)
        total = float(x.sum())
        penalty = 1.0 + 50.0 * float(self.profile.h(total, bandwidth_mbps * conversion / 1000.0)[0])
        throughput = total / float(t.max())
        cov = float(np.std(t) / max(np.mean(t), 1e-12))
        return penalty / throughput + self.lambda_2 * cov

    def _conversion_factor(self) -> float:
        """Rescales the measured bandwidth to the system the profile was taken on: if these GPUs
        need less bandwidth than the profile's at its operating point, the link is relatively wider."""
        meta = self.profile.meta
        ref_x = np.full(self.num_gpus, meta.batch_size / self.num_gpus) if self.prev_x is None \
            else self.prev_x / self.prev_x.sum() * meta.batch_size
        aggr = float(self.f(ref_x).sum())
        iter_ms = 1500.0 * meta.batch_size / max(aggr, 1e-9)
        need = self.traffic.goodput_mbps(meta.compression, iter_ms)
        return 1000.0 / max(need * meta.bandwidth, 1e-9)

    def _update_bandwidth(self, measured_mbps: float) -> float:
        if self.bw_estimate is None:
            self.bw_estimate = measured_mbps
            return self.bw_estimate
        rows = list(self.last_rows.values())
        wait = min(r["bwd_fwd_gap_ms"] + r["intra_fwd_gap_ms"] for r in rows)
        comp = float(np.mean([1.5 * r["bwd_ms"] for r in rows]))
        frac = wait / max(wait + comp, 1e-9)
        if frac < 0.05:
            frac = 0.0
        smoothed = 0.9 * self.bw_estimate + 0.1 * measured_mbps
        self.bw_estimate = smoothed * 1.1 if frac == 0.0 else smoothed * max(0.75, 1.0 - frac)
        return self.bw_estimate

    def _min_ratio_for(self, x: np.ndarray, bandwidth_mbps: float) -> float:
        iter_ms = 1500.0 * float(np.mean(self.iteration_seconds(np.maximum(x, 1.0))))
        lo, hi = 0.0, 0.999
        for _ in range(20):
            mid = lo + (hi - lo) / 2.0
            if self.traffic.goodput_mbps(mid, iter_ms) <= bandwidth_mbps:
                hi = mid
            else:
                lo = mid
        ratio = hi
        if self.num_nodes > 2:
            ratio = 1.0 - (1.0 - ratio) / (self.num_nodes - 1)
        return float(min(max(ratio, 0.0), 0.999))

    # ---------------------------------------------------------------- phases
    def _step_collect(self, bandwidth_mbps: float) -> Optional[InstructionSet]:
        if not np.all(np.isfinite(self.max_batch)):
            raise RuntimeError("every GPU needs a maximum batch size before the ramp-up phase")
        if not self.history:
            return InstructionSet(0, np.full(self.num_gpus, 4.0), self.init_ratio)
        prev = next(reversed(self.history.values()))
        if np.all(prev.batch >= self.max_batch):
            self.phase = Phase.RUNNING
            for s in self.samples:
                s.momentum = 0.999
            return self._step_running(bandwidth_mbps)
        return InstructionSet(0, np.round(np.minimum(prev.batch * 1.5, self.max_batch)), self.init_ratio)

    def _step_running(self, measured_mbps: float) -> Optional[InstructionSet]:
        bw = self._update_bandwidth(measured_mbps)
        conv = self._conversion_factor()
        low = [float(min(l, m)) if np.isfinite(l) else 1.0 for l, m in zip(self.min_sampled, self.max_batch)]
        bounds = [(lo, float(m)) for lo, m in zip(low, self.max_batch)]
        if self.main_iter % self.reoptimize_every == 0 or self.prev_x is None:
            starts = []
            if self.prev_x is None:
                for _ in range(32):
                    starts.append(np.array([self.rng.randint(int(lo), int(m)) for lo, m in zip(low, self.max_batch)], float))
            else:
                for scale in (1.0, 2.0):
                    starts.append(np.clip(self.prev_x * scale, 1.0, self.max_batch))
            best = None
            for x0 in starts:
                r = minimize(lambda x: self.objective(x, bw, conv), x0, method="Nelder-Mead", bounds=bounds,
                             options={"adaptive": True, "maxiter": 400 * self.num_gpus, "xatol": 0.5, "fatol": 1e-9})
                if best is None or r.fun < best.fun:
                    best = r
            self.prev_x, self.prev_fun = np.clip(np.round(best.x), low, self.max_batch), float(best.fun)
        self.main_iter += 1
        ratio = self._min_ratio_for(self.prev_x, bw)
        return InstructionSet(0, self.prev_x.copy(), ratio)

    def step(self, observed_iter: int, measured_mbps: float) -> Optional[InstructionSet]:
        """Called with the latest observed iteration; returns an instruction set or None."""
        if self.history and observed_iter:
            last_iter = next(reversed(self.history))
            wait = WAIT_EFFECT_ITER_MAIN if self.phase == Phase.RUNNING else WAIT_EFFECT_ITER
            if observed_iter < last_iter + wait:
                return None
        if self.phase == Phase.INIT_COLLECT_X:
            inst = self._step_collect(measured_mbps)
        elif self.phase == Phase.RUNNING:
            inst = self._step_running(measured_mbps)
        else:
            return None
        if inst is None:
            return None
        inst.iter = self.latest_iter() + EFFECTIVE_AFTER_ITER
        self.history[inst.iter] = inst
        self.log.append(f"{inst.iter},{inst.comp_ratio},{','.join(str(int(b)) for b in inst.batch)}")
        return inst
