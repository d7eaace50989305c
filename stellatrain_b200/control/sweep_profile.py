"""Measures a convergence profile h(total batch, bandwidth) for the controller and fits it.

The reference's controller multiplies its throughput estimate by ``1 + 50 h``, an "iterations needed" penalty taken
from offline profiling runs (Gaussian processes over total batch and bandwidth,
backend/src/engine/batch_rate_alloc_optim.py:139-172, 190; the scripts that produced its ``bayesian/profile/*.pkl`` are
not part of its repository).  This tool produces such a profile with this package's own sparse update rule:

    python -m stellatrain_b200.control.sweep_profile --out stellatrain_b200/control/profiles/b200_gpt2_small.json

For every point of a (total batch, bandwidth) grid it trains a small student network on a learnable synthetic task
(labels of a fixed random teacher) the way the engine trains: ``world`` ranks, each with a shard of the batch, error
feedback, top-k selection of the kept budget split over the ranks, mean of the streams, lazy sparse Adam.  The kept
fraction of a point is what the bandwidth can carry for the named deployment (``--params`` parameters at 8 bytes per
entry, ``--step-ms`` per iteration at ``--ref-batch``, iteration time growing with the batch beyond it).  It records how
many samples the run needs to reach the target loss; h is the relative excess over the best point divided by 50, so
that ``1 + 50 h`` is "samples needed, relative to the best configuration".  The fit is ``gp_profile.fit_profile``.

The bandwidth axis of the fitted profile is relative: 1.0 is the bandwidth that carries the kept fraction of the
profile's operating point (``--ref-bandwidth`` Gbps at ``--ref-batch``), which is the unit in which the controller asks
(it rescales the measured rate by what its own job needs at the profile's compression ratio,
``optimizer.BatchRateOptimizer._conversion_factor``).  ``--refit`` fits again from the rows of an existing file without
repeating the sweep.

What the profile carries over to a real job is the shape of the trade-off (less bandwidth, more compression, more
samples; larger batches, fewer but more expensive steps), not absolute numbers: the task is synthetic.
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from .gp_profile import ProfileMeta, fit_profile


def kept_fraction(bandwidth_gbps: float, total_batch: float, ref_batch: float, step_ms: float, params: float) -> float:
    """Fraction of the gradient entries the link can carry per iteration (8-byte entries)."""
    iter_s = step_ms * 1e-3 * max(1.0, total_batch / ref_batch)
    full_bits = params * 8.0 * 8.0
    return float(min(1.0, max(1e-4, bandwidth_gbps * 1e9 * iter_s / full_bits)))


def samples_to_target(total_batch: int, kept: float, world: int = 8, target: float = 1.02, max_iters: int = 3000,
                      lr: float = 3e-3, seed: int = 0, eval_every: int = 10) -> float:
    """Samples processed until the loss on a fixed held-out set falls below ``target`` (inf if it never does)."""
    g = torch.Generator().manual_seed(seed)
    dim, hidden, classes = 32, 128, 8
    teacher = nn.Sequential(nn.Linear(dim, hidden), nn.Tanh(), nn.Linear(hidden, classes))
    student = nn.Sequential(nn.Linear(dim, hidden), nn.Tanh(), nn.Linear(hidden, classes))
    with torch.no_grad():
        for p in teacher.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.6 if p.dim() > 1 else 0.1))
        for p in student.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.2 if p.dim() > 1 else 0.0))
    params = list(student.parameters())
    sizes = [p.numel() for p in params]
    n = sum(sizes)
    k = max(1, int(n * kept / world))
    resid = torch.zeros(world, n)
    m, v = torch.zeros(n), torch.zeros(n)
    tick = 1
    flat = torch.cat([p.detach().reshape(-1) for p in params])
    per_rank = max(1, total_batch // world)
    x_eval = torch.randn(2048, dim, generator=g)
    with torch.no_grad():
        y_eval = teacher(x_eval).argmax(-1)
    for it in range(max_iters):
        merged = torch.zeros(n)
        touched = torch.zeros(n, dtype=torch.bool)
        for r in range(world):
            x = torch.randn(per_rank, dim, generator=g)
            with torch.no_grad():
                y = teacher(x).argmax(-1)
            loss = F.cross_entropy(student(x), y)
            grads = torch.autograd.grad(loss, params)
            a = torch.cat([gr.reshape(-1) for gr in grads]) + resid[r]
            idx = torch.topk(a.abs(), k).indices
            merged[idx] += a[idx] / world
            touched[idx] = True
            a[idx] = 0.0
            resid[r] = a
        # lazy sparse Adam on the union of the touched entries (backend/src/optim/adam.cpp:19-87)
        i = torch.nonzero(touched).flatten()
        gg = merged[i]
        m[i] = 0.9 * m[i] + 0.1 * gg
        v[i] = 0.999 * v[i] + 0.001 * gg * gg
        flat[i] -= lr * (m[i] / (1 - 0.9 ** tick)) / ((v[i] / (1 - 0.999 ** tick)).sqrt() + 1e-8)
        tick += 1
        with torch.no_grad():
            off = 0
            for p, sz in zip(params, sizes):
                p.copy_(flat[off:off + sz].view_as(p))
                off += sz
        if (it + 1) % eval_every == 0:
            with torch.no_grad():
                if float(F.cross_entropy(student(x_eval), y_eval)) < target:
                    return float((it + 1) * per_rank * world)
    return math.inf


def fit_rows(rows, args) -> dict:
    """rows: (total batch, bandwidth in Gbps, kept fraction, samples to target)."""
    finite = [r[3] for r in rows if r[3] is not None and math.isfinite(r[3])]
    best, worst = min(finite), max(finite)
    need = [(r[3] if r[3] is not None and math.isfinite(r[3]) else 2.0 * worst) for r in rows]
    penalty = [(n / best - 1.0) / 50.0 for n in need]
    batches = sorted({r[0] for r in rows})
    kept_ref = kept_fraction(args.ref_bandwidth, args.ref_batch, args.ref_batch, args.step_ms, args.params)
    meta = ProfileMeta(batch_size=args.ref_batch, max_batch_size=float(max(batches)), min_batch_size=float(min(batches)),
                       bandwidth=1.0, compression=1.0 - kept_ref, model=args.model)
    prof = fit_profile([r[0] for r in rows], [r[1] / args.ref_bandwidth for r in rows], penalty, meta,
                       length_scale=(0.35, 1.5), noise=1e-3)
    return {"x_train": prof.x_train.tolist(), "alpha": prof.alpha.tolist(), "length_scale": prof.length_scale.tolist(),
            "constant": prof.constant, "nu": prof.nu, "y_mean": prof.y_mean, "y_std": prof.y_std, "metadata": meta.__dict__,
            "sweep": {"columns": ["total_batch", "bandwidth_gbps", "kept_fraction", "samples_to_target", "h"],
                      "rows": [[r[0], r[1], r[2], (r[3] if r[3] is not None and math.isfinite(r[3]) else None), p]
                               for r, p in zip(rows, penalty)],
                      "world": args.world, "params": args.params, "step_ms": args.step_ms, "ref_batch": args.ref_batch,
                      "ref_bandwidth_gbps": args.ref_bandwidth, "best_samples": best, "worst_samples": worst,
                      "bandwidth_axis": "multiples of ref_bandwidth_gbps",
                      "task": "labels of a fixed random teacher MLP (32-128-8), student of the same shape, error feedback + "
                              "top-k split over the ranks + lazy sparse Adam, target loss 1.02 on 2048 held-out samples"}}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--model", default="gpt2-small on B200, synthetic teacher-student convergence task")
    ap.add_argument("--params", type=float, default=124.4e6, help="parameters of the deployed model")
    ap.add_argument("--step-ms", type=float, default=29.0, help="iteration time of the deployed model at --ref-batch")
    ap.add_argument("--ref-batch", type=float, default=64.0, help="total batch at which --step-ms was measured")
    ap.add_argument("--batches", default="16,32,64,128,256,512")
    ap.add_argument("--bandwidths", default="2.5,5,10,20,40,80", help="Gbps")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--seeds", type=int, default=2)
    ap.add_argument("--ref-bandwidth", type=float, default=10.0, help="Gbps of the profile's operating point")
    ap.add_argument("--refit", default=None, help="fit from the sweep rows of this file instead of training")
    args = ap.parse_args()
    if args.refit:
        rows = [tuple(r[:4]) for r in json.loads(Path(args.refit).read_text())["sweep"]["rows"]]
        Path(args.out).write_text(json.dumps(fit_rows(rows, args), indent=1))
        print(f"wrote {args.out}: fitted again from {len(rows)} rows of {args.refit}")
        return
    torch.set_num_threads(max(1, torch.get_num_threads()))
    batches = [int(b) for b in args.batches.split(",")]
    bws = [float(b) for b in args.bandwidths.split(",")]
    rows = []
    for b in batches:
        for bw in bws:
            kept = kept_fraction(bw, b, args.ref_batch, args.step_ms, args.params)
            need = float(np.median([samples_to_target(b, kept, args.world, seed=s) for s in range(args.seeds)]))
            rows.append((b, bw, kept, need))
            print(f"batch {b:4d}  {bw:5.1f} Gbps  kept {kept:7.4f}  samples to target {need:10.0f}", flush=True)
    out = fit_rows(rows, args)
    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    Path(args.out).write_text(json.dumps(out, indent=1))
    print(f"wrote {args.out}: {len(rows)} points, best {out['sweep']['best_samples']:.0f} samples, "
          f"worst {out['sweep']['worst_samples']:.0f}")


if __name__ == "__main__":
    main()
