"""Flat-gradient CPU benchmark: compression with error feedback plus sparse Adam, checked against a
dense-update reference.

    python -m stellatrain_b200.bench_cpu_flat            # 11,689,512 elements (ResNet-18 size), 20 steps, 16 threads
    STELLATRAIN_CPU_THREADS=16 python -m stellatrain_b200.bench_cpu_flat --method thresholdv

World size 1, k = 1 % of the elements, gradients N(0, 1e-2) from seed 0, Adam lr 1e-3, betas 0.9/0.999,
eps 1e-8.  Reported: milliseconds per step of the native compress + optimise path (median), the same
for the plain-PyTorch restatement of the algorithm (the timed CPU baseline), and how the compressed
run relates to the dense run: with error feedback nothing is lost, it is only delayed, so
``sum(sent) + residual == sum(all gradients)`` exactly in exact arithmetic, and the parameter
displacement points in the direction of the dense displacement.
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from . import cpu_tier
from .ops import oracle as O


def run(numel: int = 11_689_512, steps: int = 20, method: str = "topk", seed: int = 0, kept: float = 0.01,
        time_oracle: bool = False) -> dict:
    gen = torch.Generator().manual_seed(seed)
    k = max(1, int(numel * kept))
    param = torch.zeros(numel)
    dense_param = torch.zeros(numel)
    resid = torch.zeros(numel)
    opt = cpu_tier.make_optimizer("adam")
    for key, v in (("lr", 1e-3), ("b1", 0.9), ("b2", 0.999), ("eps", 1e-8)):
        opt.configure(key, v)
    dense = O.DenseReference(dense_param, O.AdamConfig(lr=1e-3))
    comp_name = f"flat-{method}-{numel}-{seed}"
    native_ms, oracle_ms, sent_total = [], [], 0
    grad_sum = torch.zeros(numel, dtype=torch.float64)
    sent_sum = torch.zeros(numel, dtype=torch.float64)
    o_state, o_resid = O.ThresholdState(), torch.zeros(numel)
    for _ in range(steps):
        grad = torch.randn(numel, generator=gen) * 1e-2
        grad_sum += grad.double()
        t0 = time.perf_counter()
        idx, val = cpu_tier.compress_with_feedback(comp_name, grad, resid, k, method)
        opt.optimize(param.data_ptr(), numel, "flat", val.data_ptr(), idx.data_ptr(), idx.numel())
        native_ms.append((time.perf_counter() - t0) * 1e3)
        sent_total += idx.numel()
        sent_sum.index_add_(0, idx.long(), val.double())
        dense.step(grad)
        if time_oracle:
            t0 = time.perf_counter()
            oi, ov, o_resid = O.compress_step(method, grad, o_resid, k, o_state)
            o_resid = o_resid[:numel]
            oracle_ms.append((time.perf_counter() - t0) * 1e3)
    conserved = torch.allclose(sent_sum + resid.double(), grad_sum, rtol=0, atol=1e-4)
    d_sparse, d_dense = param, dense_param
    cos = float(torch.dot(d_sparse, d_dense) / (d_sparse.norm() * d_dense.norm() + 1e-30))
    rel = float((d_sparse - d_dense).norm() / (d_dense.norm() + 1e-30))
    native_ms.sort()
    out = {
        "config": "flat fp32 gradient, world 1, error feedback + sparse Adam",
        "numel": numel, "steps": steps, "method": method, "k": k, "isa": cpu_tier._load().best_isa(),
        "native_ms_per_step_median": native_ms[len(native_ms) // 2],
        "sent_fraction": sent_total / (steps * numel),
        "residual_mass_conserved": bool(conserved),
        "cos_to_dense": cos, "rel_l2_to_dense": rel,
    }
    if oracle_ms:
        oracle_ms.sort()
        out["pytorch_restatement_ms_per_step_median"] = oracle_ms[len(oracle_ms) // 2]
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=11_689_512)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--method", default="all")
    ap.add_argument("--time-oracle", action="store_true")
    args = ap.parse_args()
    methods = ["topk", "thresholdv", "thresholdv16"] if args.method == "all" else [args.method]
    for m in methods:
        print(json.dumps(run(args.numel, args.steps, m, time_oracle=args.time_oracle)))


if __name__ == "__main__":
    main()
