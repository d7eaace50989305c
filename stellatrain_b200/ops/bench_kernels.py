"""Kernel-level timing of the sparse path against its memory roofline.

    python -m stellatrain_b200.ops.bench_kernels --model resnet152 --compressor thresholdv16
    python -m stellatrain_b200.ops.bench_kernels --elems 40000000 --segments 64 --compressor topk

Times, with CUDA events after warm-up, the select chain and the apply chain (scatter, apply) over all buckets
of a parameter-size list, and reports achieved HBM bandwidth against the measured copy bandwidth of the
machine (``MEASURED_PEAKS.json`` next to the repository root when present).  Algorithmic traffic of one select,
per element: the two-pass chain (pass1, plan, pass2, cand) reads g and r and writes r in pass 1 and reads r
again in pass 2 = 16 bytes; the one-pass chain of the threshold compressors (fused, finish) reads g and r and
writes r = 12 bytes; both write 4 more when the consumed gradient is zeroed (``--zero-grad 1``, the engine's
"flat" gradient mode; its default mode hands the kernels autograd's own tensors and zeroes nothing).  The sparse
outputs are below 1 % of that.  Between iterations the gradient buffers are refilled, which also evicts the
previous iteration's lines from L2.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch

from ..parallel import buckets as B
from ..parallel.gpu_bucket import CandidateScratch, GpuBucket


def model_numels(name: str) -> list[int]:
    from ..models.registry import build_model

    with torch.device("meta"):
        m = build_model(name, 100)
    return [p.numel() for p in reversed(list(m.parameters()))]


def measured_peaks() -> dict:
    here = Path(__file__).resolve()
    for parent in here.parents:
        f = parent / "MEASURED_PEAKS.json"
        if f.exists():
            return json.loads(f.read_text())
    return {"hbm_gbs": 6650.0, "fallback": True}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--elems", type=int, default=40_000_000)
    ap.add_argument("--segments", type=int, default=64)
    ap.add_argument("--compressor", default="thresholdv16")
    ap.add_argument("--optimizer", default="adam")
    ap.add_argument("--ratio", type=float, default=0.99)
    ap.add_argument("--bucket-mb", type=float, default=64.0)
    ap.add_argument("--chunk-elems", type=int, default=8192)
    ap.add_argument("--zero-grad", type=int, default=0, help="1: the select also writes zeros over the gradients it consumed")
    ap.add_argument("--fused", type=int, default=1, help="0: keep the threshold compressors on the two-pass chain")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    dev = torch.device("cuda:0")
    numels = model_numels(args.model) if args.model else [args.elems // args.segments] * args.segments
    groups = B.plan_buckets(numels, int(args.bucket_mb * (1 << 20) / 4))
    scratch = CandidateScratch(dev)
    buckets = []
    for bi, grp in enumerate(groups):
        layout = B.BucketLayout([f"t{i}" for i in grp], [numels[i] for i in grp], chunk_elems=args.chunk_elems)
        b = GpuBucket(bi, layout, dev, compressor=args.compressor, ratio=args.ratio, optimizer=args.optimizer,
                      scratch=scratch, fused_select=bool(args.fused))
        b.wire_local()
        b.zero_grad_in_select = bool(args.zero_grad)
        b._bind()
        buckets.append(b)
    n_total = sum(b.layout.n_total for b in buckets)
    gen = torch.Generator(device=dev).manual_seed(0)

    def refill() -> None:
        for b in buckets:
            b.grad.normal_(0.0, 1e-2, generator=gen)

    sel_ms, app_ms = [], []
    for it in range(args.warmup + args.iters):
        refill()
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        for b in buckets:
            b.select()
        e[1].record()
        for b in buckets:
            b.apply()
        e[2].record()
        torch.cuda.synchronize()
        if it >= args.warmup:
            sel_ms.append(e[0].elapsed_time(e[1]))
            app_ms.append(e[1].elapsed_time(e[2]))
    for b in buckets:
        b.check_status()
    peaks = measured_peaks()
    sel = sorted(sel_ms)[len(sel_ms) // 2]
    app = sorted(app_ms)[len(app_ms) // 2]
    one_pass = bool(getattr(buckets[0], "last_select_fused", False))
    sel_bytes = ((12.0 if one_pass else 16.0) + (4.0 if args.zero_grad else 0.0)) * n_total
    entries = sum(b.layout.cap for b in buckets)
    # apply: per entry read 8 B twice; per touched element one 32 B sector of the state record and one of the parameter
    app_bytes = entries * (16.0 + 32.0 * 2)
    out = {
        "compressor": args.compressor, "optimizer": args.optimizer, "elements": n_total, "buckets": len(buckets),
        "segments": len(numels), "entries_per_step": entries,
        "select_chain": "one-pass (fused, finish)" if one_pass else "two-pass (pass1, plan, pass2, cand)",
        "select_bytes_per_element": sel_bytes / n_total,
        "select_ms": sel, "select_GBps": sel_bytes / sel / 1e6,
        "select_frac_of_measured_copy": sel_bytes / sel / 1e6 / peaks["hbm_gbs"],
        "apply_ms": app, "apply_sector_GBps": app_bytes / app / 1e6,
        "hbm_gbs_measured": peaks["hbm_gbs"], "peaks_are_fallback": bool(peaks.get("fallback", False)),
        "kernel_launches_per_step": len(buckets) * (4 if one_pass else 6),
    }
    print(json.dumps(out))


if __name__ == "__main__":
    main()
