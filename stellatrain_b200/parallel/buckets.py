"""Bucket layout: how parameter tensors are packed into flat fp32 ranges and cut into work units.

The reference schedules one task per parameter tensor per iteration
(backend/src/python/fasterdp/model_wrapper.py:83-86, backend/src/engine/core.cpp:1052); ResNet-152 has
467 tensors, most of them tiny, so here tensors are packed into buckets and every kernel of the sparse
path works on a whole bucket while keeping the per-tensor rules (k, thresholds) in segment tables.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np

ALIGN = 16  # elements; one 64-byte line, the block size of threshold-v16

SEG_DESC_DTYPE = np.dtype(
    [("off", "<u4"), ("n", "<u4"), ("n_pad", "<u4"), ("k", "<u4"), ("out_off", "<u4"),
     ("chunk_begin", "<u4"), ("chunk_cnt", "<u4"), ("reserved", "<u4")]
)
SEG_STATE_DTYPE = np.dtype([("tau", "<f4"), ("tau_inc", "<f4"), ("inited", "<u4"), ("hist_base", "<u4"),
                            ("hist_shift", "<u4"), ("r0", "<u4"), ("r1", "<u4"), ("r2", "<u4")])
SEG_WORK_WORDS = 12
CHUNK_DTYPE = np.dtype([("seg", "<u4"), ("start", "<u4"), ("len", "<u4"), ("reserved", "<u4")])
OPT_STATE_DTYPE = np.dtype(
    [("lr", "<f4"), ("momentum", "<f4"), ("dampening", "<f4"), ("weight_decay", "<f4"),
     ("beta1", "<f4"), ("beta2", "<f4"), ("eps", "<f4"), ("reserved0", "<f4"),
     ("nesterov", "<u4"), ("maximize", "<u4"), ("amsgrad", "<u4"), ("smart_momentum", "<u4"),
     ("tick", "<u4"), ("first", "<u4"), ("kind", "<u4"), ("reserved1", "<u4")]
)

NARROW_LIMIT = 65536      # reference: u16 indices when the tensor has fewer than 65536 elements (comm_manager.cpp:579-583)

COMPRESSORS = {"topk": 0, "thresholdv": 1, "thresholdv16": 2, "randomk": 3}


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def entries_for(numel: int, ratio: float, world: int) -> int:
    """Entries one rank emits for a tensor.

    ``ratio`` is the fraction dropped; each of ``world`` ranks sends 1/world of the kept budget,
    at least one entry (backend/src/engine/modules/compress.cpp:44-52).
    """
    if numel <= 0:
        return 0
    k_frac = (1.0 - float(ratio)) / max(1, int(world))
    # the small epsilon keeps products such as 5000 * (1 - 0.9) = 499.99999999999994 from losing an entry
    return int(min(numel, max(min(numel, 1), int(numel * k_frac + 1e-6))))


@dataclass
class Segment:
    name: str
    numel: int
    off: int          # offset in the bucket, multiple of ALIGN
    n_pad: int
    k: int = 0
    out_off: int = 0
    chunk_begin: int = 0
    chunk_cnt: int = 0
    skip: bool = False     # grouped mode: another rank of the group owns this tensor
    owner: int = 0         # partitioned optimiser state: the rank that keeps this tensor's state


@dataclass
class BucketLayout:
    """Offsets of the tensors of one bucket plus the chunk table of its streaming kernels."""

    names: Sequence[str]
    numels: Sequence[int]
    chunk_elems: int = 8192
    segments: list[Segment] = field(default_factory=list)
    n_total: int = 0
    cap: int = 0
    narrow_wire: bool = False   # tensors below NARROW_LIMIT padded elements send 4-byte (u16 index, bf16 value) entries

    def __post_init__(self) -> None:
        if self.chunk_elems % 1024:
            raise ValueError("chunk_elems must be a multiple of 1024")
        off = 0
        chunk = 0
        for name, n in zip(self.names, self.numels):
            n = int(n)
            n_pad = round_up(max(n, 1), ALIGN)
            cc = (n_pad + self.chunk_elems - 1) // self.chunk_elems
            self.segments.append(Segment(name, n, off, n_pad, chunk_begin=chunk, chunk_cnt=cc))
            off += n_pad
            chunk += cc
        if off >= 2**32 - 1:
            raise ValueError("a bucket must hold fewer than 2^32-1 elements")
        self.n_total = off
        self.n_chunks = chunk

    def set_ratio(self, ratio: float, world: int) -> None:
        pos = 0
        for s in self.segments:
            s.k = entries_for(s.numel, ratio, world)
            s.out_off = pos
            pos += s.k
        self.cap = pos

    def assign_owners(self, group_size: int, my_local: int) -> list[int]:
        """Grouped mode: spread the tensors of the bucket over the ranks of a group (largest first onto the
        least loaded rank, ties towards the lower rank) and mark the ones this rank does not own."""
        load = [0] * group_size
        owner = [0] * len(self.segments)
        for i in sorted(range(len(self.segments)), key=lambda j: (-self.segments[j].numel, j)):
            r = min(range(group_size), key=lambda q: (load[q], q))
            owner[i] = r
            load[r] += self.segments[i].numel
        for i, s in enumerate(self.segments):
            s.skip = owner[i] != my_local
        return owner

    def assign_state_owners(self, world: int) -> list[int]:
        """Partitioned optimiser state: consecutive tensors go to the same rank so that every rank keeps one
        contiguous element range of the bucket; a tensor belongs to the rank whose 1/world share of the bucket
        contains its midpoint.  Returns the owner of every tensor."""
        for s in self.segments:
            s.owner = min(world - 1, int((s.off + s.n_pad / 2.0) * world / max(1, self.n_total)))
        return [s.owner for s in self.segments]

    def state_range(self, rank: int) -> tuple[int, int]:
        """Element range [lo, hi) of the bucket whose optimiser state ``rank`` keeps (empty: lo == hi)."""
        mine = [s for s in self.segments if s.owner == rank]
        if not mine:
            return (0, 0)
        return (mine[0].off, mine[-1].off + mine[-1].n_pad)

    def owner_bounds(self, world: int) -> list[int]:
        """world + 1 stream positions: owner o consumes the entries [bounds[o], bounds[o + 1])."""
        bounds = [0] * (world + 1)
        for s in self.segments:
            bounds[s.owner + 1] += s.k
        for o in range(world):
            bounds[o + 1] += bounds[o]
        return bounds

    def is_narrow(self, s: Segment) -> bool:
        return self.narrow_wire and s.n_pad < NARROW_LIMIT

    def wire_bytes(self, owned_only: bool = False) -> int:
        """Bytes one rank stores into one destination for this bucket per step."""
        return sum(s.k * (4 if self.is_narrow(s) else 8) for s in self.segments if not (owned_only and s.skip))

    def max_cap(self, min_ratio: float, world: int) -> int:
        return sum(entries_for(s.numel, min_ratio, world) for s in self.segments)

    def seg_table(self) -> np.ndarray:
        t = np.zeros(len(self.segments), dtype=SEG_DESC_DTYPE)
        for i, s in enumerate(self.segments):
            t[i] = (s.off, s.numel, s.n_pad, s.k, s.out_off, s.chunk_begin, s.chunk_cnt,
                    (1 if s.skip else 0) | (2 if self.is_narrow(s) else 0) | ((s.owner & 0xFF) << 8))
        return t

    def chunk_table(self) -> np.ndarray:
        t = np.zeros(self.n_chunks, dtype=CHUNK_DTYPE)
        c = 0
        for i, s in enumerate(self.segments):
            done = 0
            while done < s.n_pad:
                ln = min(self.chunk_elems, s.n_pad - done)
                t[c] = (i, s.off + done, ln, 0)
                done += ln
                c += 1
        assert c == self.n_chunks
        return t


def plan_buckets(numels: Sequence[int], bucket_elems: int) -> list[list[int]]:
    """Greedy grouping of consecutive tensors (already in the order their gradients become ready)
    into buckets of about ``bucket_elems`` elements; a tensor larger than that gets its own bucket."""
    groups: list[list[int]] = []
    cur: list[int] = []
    cur_n = 0
    for i, n in enumerate(numels):
        n_pad = round_up(max(int(n), 1), ALIGN)
        if cur and cur_n + n_pad > bucket_elems:
            groups.append(cur)
            cur, cur_n = [], 0
        cur.append(i)
        cur_n += n_pad
    if cur:
        groups.append(cur)
    return groups
