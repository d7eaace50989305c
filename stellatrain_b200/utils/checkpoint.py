"""Checkpoints in torch ``state_dict`` form (the reference has none; state that must survive is listed in
backend/src/optim/sgd.h:15-18, backend/src/optim/adam.h:15-18, backend/src/compress/thresholdv16.h:13-14,
backend/src/engine/core.h:63, 111-127).

Layout of one file per rank, written with ``torch.save``::

    {"model": module.state_dict(), "engine": SparseDPEngine.state_dict(), "extra": {...}, "rank": r, "world": W}

With replicated optimiser state (the default, as in the reference) every rank holds the full state for its
replica, so rank 0's file alone restores a job of the same world size; ``save(..., all_ranks=True)`` also keeps
the per-rank residuals, which differ between ranks.  With partitioned state (``state_partition="owner"``) each
file holds the moments of the tensors its rank owns; ``merge_state_shards`` reassembles them when a job resumes
on a different number of ranks.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Optional

import torch
import torch.distributed as dist


def _rank_world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def save(path: str, module: torch.nn.Module, engine, extra: Optional[dict] = None, all_ranks: bool = True,
         gather: bool = False) -> Optional[str]:
    """One file per rank (exact resume), or with ``gather=True`` a single file written by rank 0 that holds the
    whole optimiser state even when it is partitioned over the ranks.  A gathered file keeps rank 0's residual only:
    the other ranks restart theirs from zero, so use per-rank files when the resume must be bit-exact."""
    rank, world = _rank_world()
    engine.synchronize()
    esd = engine.state_dict()
    p = Path(path)
    if gather and world > 1:
        if esd.get("state_partition", "replicated") == "owner":
            keys = ("m", "v", "vmax", "last", "state_range")
            shard = [{k: b[k] for k in keys if k in b} for b in esd["buckets"]]
            shards = [None] * world
            dist.all_gather_object(shards, shard)
            if rank == 0:
                per_rank = [dict(esd, buckets=[dict(b, **sh) for b, sh in zip(esd["buckets"], shards[r])]) for r in range(world)]
                esd = merge_state_shards(per_rank)
        if rank == 0:
            esd["gathered"] = True
            _write(p, {"model": module.state_dict(), "engine": esd, "extra": extra or {}, "rank": 0, "world": world})
        dist.barrier()
        return str(p) if rank == 0 else None
    writes = all_ranks or rank == 0
    if world > 1:
        p = p.with_name(f"{p.stem}.rank{rank}{p.suffix}")
    if writes:
        _write(p, {"model": module.state_dict(), "engine": esd, "extra": extra or {}, "rank": rank, "world": world})
    if world > 1:
        dist.barrier()      # every rank takes part, also the ones that wrote nothing
    return str(p) if writes else None


def _write(p: Path, payload: dict) -> None:
    p.parent.mkdir(parents=True, exist_ok=True)
    tmp = p.with_suffix(p.suffix + ".tmp")
    torch.save(payload, tmp)
    os.replace(tmp, p)     # a crash never leaves a half-written checkpoint under the final name


def merge_state_shards(engine_sds: list[dict]) -> dict:
    """One engine ``state_dict`` with full-size moments from the per-rank dicts of a job that ran with
    partitioned optimiser state.  Every element range is taken from the rank that owned it; parameters,
    thresholds and step counters are replica-independent and come from the first dict."""
    out = dict(engine_sds[0])
    out["buckets"] = []
    for bi, first in enumerate(engine_sds[0]["buckets"]):
        merged = dict(first)
        n = first["param"].numel()
        for k in ("m", "v", "vmax", "last"):
            if k not in first:
                continue
            full = torch.zeros(n, dtype=first[k].dtype)
            for sd in engine_sds:
                b = sd["buckets"][bi]
                lo, hi = b.get("state_range", (0, n))
                full[lo:hi] = b[k][: hi - lo]
            merged[k] = full
        merged["state_range"] = (0, n)
        merged.pop("stamp", None)
        out["buckets"].append(merged)
    out["state_partition"] = "replicated"
    return out


def load(path: str, module: torch.nn.Module, engine, map_location="cpu", allow_world_change: bool = False) -> dict:
    """``allow_world_change``: resume on a different number of ranks (after losing one, or after growing).
    Parameters, optimiser state and thresholds are replica-independent and are restored; residuals, epochs and
    exchange counters depend on the world size and start afresh (the unsent gradient mass of the old job is
    dropped, which costs at most one step's worth of updates)."""
    rank, world = _rank_world()
    p = Path(path)
    if not p.exists():
        mine = p.with_name(f"{p.stem}.rank{rank}{p.suffix}")
        p = mine if mine.exists() else p.with_name(f"{p.stem}.rank0{p.suffix}")
    ck = torch.load(p, map_location=map_location, weights_only=False)
    if ck["world"] != world:
        if not allow_world_change:
            raise ValueError(f"checkpoint was written by {ck['world']} ranks, this job has {world}")
        module.load_state_dict(ck["model"], strict=False)
        esd = ck["engine"]
        if esd.get("state_partition", "replicated") == "owner":
            base = Path(path)
            files = [base.with_name(f"{base.stem}.rank{r}{base.suffix}") for r in range(ck["world"])]
            missing = [str(f) for f in files if not f.exists()]
            if missing:
                raise FileNotFoundError(f"partitioned optimiser state needs every rank's file; missing: {missing}")
            esd = merge_state_shards([torch.load(f, map_location=map_location, weights_only=False)["engine"]
                                      for f in files])
        engine.load_replica_state(esd)
        return ck["extra"]
    # buffers (e.g. BatchNorm statistics) come from the model part, parameters from the engine's buckets
    module.load_state_dict(ck["model"], strict=False)
    engine.load_state_dict(ck["engine"])
    if ck["engine"].get("gathered") and rank != 0:
        for rt in engine.buckets:          # the file carries rank 0's residual only
            rt.bucket.resid.zero_()
    return ck["extra"]
