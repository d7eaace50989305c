"""Device state of one bucket and the thin Python handle that launches its kernels.

Everything the reference keeps per tensor on the CPU lives here per bucket on the GPU: the error-feedback
residual (backend/src/engine/core.h:63), the thresholds of threshold-v / threshold-v16
(backend/src/compress/thresholdv16.h:13-14), the optimiser state (backend/src/optim/sgd.h:15-18,
backend/src/optim/adam.h:15-18) and the master parameters (backend/src/engine/core.cpp:807-830).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import buckets as B

STATUS_NAMES = {
    0: "ok",
    1: "timeout waiting for a peer's acknowledgement",
    2: "timeout waiting for a peer's stream",
    3: "received index outside the bucket",
    4: "candidate scratch exhausted",
    5: "size beyond a compiled-in limit",
    6: "a received stream does not match its source's checksum",
    7: "one-pass select: a chunk never saw the count of the chunk before it",
}


class SparseStepError(RuntimeError):
    """A kernel of the sparse path reported a non-zero status (for example a peer that never pushed)."""

    def __init__(self, bucket: int, code: int):
        super().__init__(f"bucket {bucket}: {STATUS_NAMES.get(code, 'unknown error')} (status {code})")
        self.bucket = bucket
        self.code = code


def _ext():
    from .. import _build

    return _build.load_extension("_C")


def _dev_bytes(arr: np.ndarray, device: torch.device) -> torch.Tensor:
    raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
    return torch.from_numpy(raw.copy()).to(device)


@dataclass
class Wiring:
    """Where a bucket's streams go: addresses of every rank's receive area, flags and acks."""

    world: int
    rank: int
    recv_local: torch.Tensor                 # uint8 view holding [2][world][cap] (idx,val) pairs
    peer_recv: Sequence[int]
    flag_local: Optional[torch.Tensor]       # int64 [2][world]
    peer_flag: Sequence[int]
    ack_local: Optional[torch.Tensor]        # int64 [2][world]
    peer_ack: Sequence[int]
    recv_mc: int = 0
    use_flags: bool = False
    use_acks: bool = False
    # partitioned optimiser state: write-back areas (shape of the receive areas) and "values landed" flags
    wb_local: Optional[torch.Tensor] = None
    peer_wb: Sequence[int] = ()
    wb_mc: int = 0
    pflag_local: Optional[torch.Tensor] = None   # int64 [2][world]
    peer_pflag: Sequence[int] = ()
    # debug checks: per-source stream checksums (int32 [2][world]) and poisoning of consumed entries
    cksum_local: Optional[torch.Tensor] = None
    peer_cksum: Sequence[int] = ()
    poison: bool = False


class GpuBucket:
    GRAD_TAB_RING = 4

    def __init__(
        self,
        index: int,
        layout: B.BucketLayout,
        device: torch.device,
        compressor: str = "thresholdv16",
        ratio: float = 0.99,
        world: int = 1,
        rank: int = 0,
        optimizer: str = "sgd",
        amsgrad: bool = False,
        smart_momentum: bool = False,
        min_ratio: Optional[float] = None,
        scratch: Optional["CandidateScratch"] = None,
        timeout_s: float = 2.0,
        divide_k_by_world: bool = True,
        k_world: Optional[int] = None,
        partition_state: bool = False,
        deterministic_merge: bool = False,
        fused_select: bool = True,
    ) -> None:
        self.index = index
        self.layout = layout
        self.device = device
        self.world, self.rank = world, rank
        self.k_world = k_world if k_world is not None else (world if divide_k_by_world else 1)
        self.compressor = compressor
        self.ratio = ratio
        self.min_ratio = ratio if min_ratio is None else min(min_ratio, ratio)
        self.optimizer = optimizer
        self.timeout_ns = int(timeout_s * 1e9)
        self.deterministic_merge = bool(deterministic_merge)   # scatter one source after the other: bit-equal replicas
        n = layout.n_total
        f32 = dict(dtype=torch.float32, device=device)
        self.grad = torch.zeros(n, **f32)
        self.resid = torch.zeros(n, **f32)
        self.param = torch.zeros(n, **f32)
        # Accumulator, stamps and optimiser state cover the whole bucket, or with partitioned state only the
        # contiguous element range of the tensors this rank owns (1/world of the memory).
        self.partition_state = bool(partition_state) and world > 1
        if self.partition_state:
            layout.assign_state_owners(world)
            self.state_lo, self.state_hi = layout.state_range(rank)
        else:
            self.state_lo, self.state_hi = 0, n
        ns = max(self.state_hi - self.state_lo, B.ALIGN)
        # One 16-byte record per element, {accumulator, stamp, m, v}: an update touches one sector of state.
        # acc / stamp / m / v are strided views of it (v stays unused by SGD).
        self.rec = torch.zeros(ns, 4, **f32)
        self.acc = self.rec[:, 0]
        self.stamp = self.rec[:, 1].view(torch.int32)
        self.m = self.rec[:, 2]
        self.v = self.rec[:, 3] if optimizer == "adam" else None
        self.vmax = torch.zeros(ns, **f32) if (optimizer == "adam" and amsgrad) else None
        self.last = torch.zeros(ns, dtype=torch.int32, device=device) if smart_momentum else None

        layout.set_ratio(ratio, self.k_world)
        self.cap_max = max(layout.max_cap(self.min_ratio, self.k_world), layout.cap, 1)
        n_segs = len(layout.segments)
        self.segs = _dev_bytes(layout.seg_table(), device)
        self.state = torch.zeros(n_segs * B.SEG_STATE_DTYPE.itemsize, dtype=torch.uint8, device=device)
        self.work = torch.zeros(n_segs * B.SEG_WORK_WORDS, dtype=torch.int32, device=device)
        self.chunks = _dev_bytes(layout.chunk_table(), device)
        self.chunk_cnt = torch.zeros(layout.n_chunks, dtype=torch.int32, device=device)
        self.chunk_pos = torch.zeros(layout.n_chunks, dtype=torch.int32, device=device)
        # One-pass select of the threshold compressors: one state word per chunk (epoch | kind | count).  It takes
        # over once every tensor has a threshold: after the first select, or after a checkpoint that carries them.
        self.chunk_state = torch.zeros(layout.n_chunks, dtype=torch.int64, device=device)
        self.fused_select = bool(fused_select)
        self.hist = torch.zeros(n_segs * 2048, dtype=torch.int32, device=device)
        # [select epoch, apply epoch, select CTAs done, apply CTAs done, 4 spare]
        self.counters = torch.tensor([1, 1, 0, 0, 0, 0, 0, 0], dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.stamps = torch.zeros(8, dtype=torch.int64, device=device)    # device clock of the latest chain, see device_times()
        # merge weight of every source, one row per epoch parity (the scatter of epoch e reads row e & 1)
        self.weight = torch.full((2, world), 1.0 / world, **f32)
        opt = np.zeros(1, dtype=B.OPT_STATE_DTYPE)
        opt["lr"] = 1e-3
        opt["beta1"], opt["beta2"], opt["eps"] = 0.9, 0.999, 1e-8
        opt["tick"], opt["first"] = 1, 1
        opt["kind"] = 1 if optimizer == "adam" else 0
        opt["amsgrad"] = 1 if amsgrad else 0
        opt["smart_momentum"] = 1 if smart_momentum else 0
        self._opt_host = opt
        self.opt = _dev_bytes(opt, device)
        self.scratch = scratch if scratch is not None else CandidateScratch(device)
        self.scratch.reserve(n)
        self.handle = _ext().BucketHandle()
        self.wiring: Optional[Wiring] = None
        # library-collective baseline: a second handle whose only destination is a local send buffer
        self.select_handle = None
        self.select_wiring: Optional[Wiring] = None
        self.zero_grad_in_select = True
        # "steal" mode: gradients stay where autograd put them; the kernels read them through a
        # per-segment pointer table that the engine refreshes every iteration
        self.grad_tab_host: Optional[torch.Tensor] = None
        self.grad_tab_dev: Optional[torch.Tensor] = None
        self._bind()

    # ------------------------------------------------------------------ wiring
    def _ptr(self, t: Optional[torch.Tensor]) -> int:
        return 0 if t is None else t.data_ptr()

    def _bind(self) -> None:
        self._bind_one(self.handle, self.wiring)
        if self.select_handle is not None:
            self._bind_one(self.select_handle, self.select_wiring)

    def _bind_one(self, h, wiring: Optional[Wiring]) -> None:
        L = self.layout
        h.set_data(
            grad=self.grad.data_ptr(), grad_tab=self._ptr(self.grad_tab_dev), resid=self.resid.data_ptr(),
            param=self.param.data_ptr(), rec=self.rec.data_ptr(), vmax=self._ptr(self.vmax), last=self._ptr(self.last),
            n_total=L.n_total,
        )
        h.set_tables(
            segs=self.segs.data_ptr(), state=self.state.data_ptr(), work=self.work.data_ptr(),
            chunks=self.chunks.data_ptr(), chunk_cnt=self.chunk_cnt.data_ptr(), chunk_pos=self.chunk_pos.data_ptr(),
            hist=self.hist.data_ptr(), n_segs=len(L.segments), n_chunks=L.n_chunks, cap=L.cap,
            chunk_state=self.chunk_state.data_ptr(), max_chunk=min(L.chunk_elems, max(s.n_pad for s in L.segments)),
        )
        self.scratch.bind(h)
        h.set_control(
            counters=self.counters.data_ptr(), status=self.status.data_ptr(), opt=self.opt.data_ptr(),
            weight=self.weight.data_ptr(), timeout_ns=self.timeout_ns, stamps=self.stamps.data_ptr(),
        )
        h.set_options(B.COMPRESSORS[self.compressor], self.zero_grad_in_select, False,
                      any(self.layout.is_narrow(s) for s in self.layout.segments), self.deterministic_merge)
        h.fused_enabled = self.fused_select
        if wiring is not None:
            self._apply_wiring(h, wiring)

    def rebind_grad(self, storage: torch.Tensor) -> None:
        """Move the flat gradient buffer into caller-provided (peer-visible) memory."""
        assert storage.numel() == self.layout.n_total and storage.dtype == torch.float32
        storage.zero_()
        self.grad = storage
        self._bind()

    def upload_segments(self) -> None:
        self.segs.copy_(_dev_bytes(self.layout.seg_table(), self.device))

    def use_grad_table(self) -> None:
        """Switch the select to per-tensor gradient pointers (no flat gradient copy, no zeroing)."""
        n_segs = len(self.layout.segments)
        # a small ring of pinned tables: the copy of iteration i may still be in flight when the
        # hooks of iteration i+1 write their pointers
        self.grad_tab_host = torch.zeros(self.GRAD_TAB_RING, n_segs, dtype=torch.int64).pin_memory()
        self.grad_tab_dev = torch.zeros(n_segs, dtype=torch.int64, device=self.device)
        for i, seg in enumerate(self.layout.segments):       # default: the flat buffer
            self.grad_tab_host[:, i] = self.grad.data_ptr() + 4 * seg.off
        self.grad_tab_dev.copy_(self.grad_tab_host[0])
        self.zero_grad_in_select = False
        self._bind()

    def recv_bytes(self) -> int:
        """Bytes of receive area one rank needs for this bucket (two slots, all sources)."""
        return 2 * self.world * self.cap_max * 8

    def wire_local(self, debug_checks: bool = False) -> None:
        """Single-process wiring: the stream goes to this GPU's own receive area, stream order is
        the only synchronisation."""
        recv = torch.zeros(self.recv_bytes(), dtype=torch.uint8, device=self.device)
        extra = {}
        if debug_checks:
            ck = torch.zeros(2, dtype=torch.int32, device=self.device)
            extra = dict(cksum_local=ck, peer_cksum=[ck.data_ptr()], poison=True)
        self.wire(Wiring(1, 0, recv, [recv.data_ptr()], None, [0], None, [0], **extra))

    def wire(self, w: Wiring) -> None:
        self.wiring = w
        self._apply_wiring(self.handle, w)

    def wire_select(self, w: Wiring) -> None:
        """Give the select its own destination list (used when a library collective moves the
        stream afterwards); apply keeps using the main wiring."""
        if self.select_handle is None:
            self.select_handle = _ext().BucketHandle()
        self.select_wiring = w
        self._bind_one(self.select_handle, w)

    def _apply_wiring(self, h, w: Wiring) -> None:
        h.set_comm(
            world=w.world, rank=w.rank, recv_local=w.recv_local.data_ptr(), peer_recv=list(w.peer_recv),
            recv_mc=w.recv_mc, flag_local=self._ptr(w.flag_local), peer_flag=list(w.peer_flag),
            ack_local=self._ptr(w.ack_local), peer_ack=list(w.peer_ack), use_flags=w.use_flags,
            use_acks=w.use_acks,
        )
        if w.cksum_local is not None:
            if not hasattr(self, "_cksum_acc"):
                self._cksum_acc = torch.zeros(_ext().MAX_WORLD, dtype=torch.int32, device=self.device)
                self._rsum = torch.zeros(max(w.world, 1), dtype=torch.int32, device=self.device)
            h.set_debug(cksum_acc=self._cksum_acc.data_ptr(), rsum=self._rsum.data_ptr(),
                        cksum_local=w.cksum_local.data_ptr(), peer_cksum=list(w.peer_cksum), poison=w.poison)
        if self.partition_state and w.world > 1:
            if w.wb_local is None or w.pflag_local is None:
                raise ValueError("partitioned optimiser state needs write-back areas and flags in the wiring")
            h.set_owner(
                bounds=self.layout.owner_bounds(w.world), state_base=self.state_lo,
                state_len=self.state_hi - self.state_lo, wb_local=w.wb_local.data_ptr(), peer_wb=list(w.peer_wb),
                wb_mc=w.wb_mc, pflag_local=w.pflag_local.data_ptr(), peer_pflag=list(w.peer_pflag),
            )

    # ------------------------------------------------------------------ configuration
    def set_ratio(self, ratio: float) -> None:
        """Change the compression ratio. The caller guarantees that no select/apply is in flight."""
        if ratio < self.min_ratio - 1e-12:
            raise ValueError(f"ratio {ratio} is below the provisioned minimum {self.min_ratio}")
        self.ratio = ratio
        self.layout.set_ratio(ratio, self.k_world)
        self.segs.copy_(_dev_bytes(self.layout.seg_table(), self.device))
        self._bind()

    def set_optimizer_options(self, **kw) -> None:
        """Update hyper-parameters on the device; counters (tick, first) are left untouched."""
        for k, v in kw.items():
            if k not in self._opt_host.dtype.names or k in ("tick", "first", "kind"):
                raise KeyError(k)
            self._opt_host[k] = v
        raw = np.ascontiguousarray(self._opt_host).view(np.uint8).reshape(-1)[:48].copy()
        self.opt[:48].copy_(torch.from_numpy(raw), non_blocking=False)

    def set_weights(self, weights: Sequence[float]) -> None:
        """Both rows at once; the caller guarantees that no apply is in flight."""
        self.weight.copy_(torch.tensor([list(weights)] * 2, dtype=torch.float32))

    def set_weight_row(self, parity: int, weights: torch.Tensor) -> None:
        """Stream-ordered update of the row that epochs of the given parity read (``weights``: device tensor [world])."""
        self.weight[parity & 1].copy_(weights, non_blocking=True)

    # ------------------------------------------------------------------ execution
    @property
    def _select_h(self):
        return self.select_handle or self.handle

    @property
    def thresholds_ready(self) -> bool:
        """Every tensor has its threshold: the one-pass chain of the threshold compressors may take over."""
        return bool(self._select_h.thresholds_ready)

    @thresholds_ready.setter
    def thresholds_ready(self, v: bool) -> None:
        self._select_h.thresholds_ready = bool(v)

    @property
    def last_select_fused(self) -> bool:
        return bool(self._select_h.last_select_fused)

    def select(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        self._select_h.select(s.cuda_stream)

    def apply(self, stream: Optional[torch.cuda.Stream] = None, phase: int = 0) -> None:
        """phase 0: the whole chain; 1: scatter + optimiser only; 2: copy of the owners' values only."""
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        self.handle.apply(s.cuda_stream, phase)

    @property
    def apply_kernels(self) -> int:
        waits = 1 if (self.wiring is not None and self.wiring.use_flags) else 0     # the one-warp flag wait
        return (3 if self.partition_state else 2) + (self.world - 1 if self.deterministic_merge else 0) + waits

    def device_times(self) -> dict:
        """Device-clock view of the latest select and apply of this bucket, in milliseconds (blocking read):
        how long select + push took, how long the apply ran, and for which epochs the numbers stand."""
        t = self.stamps.cpu().tolist()
        return {"select_ms": max(0, t[1] - t[0]) / 1e6, "apply_ms": max(0, t[3] - t[2]) / 1e6,
                "select_epoch": t[4], "apply_epoch": t[5],
                "select_end_to_apply_start_ms": (t[2] - t[1]) / 1e6 if t[4] == t[5] else None}

    def check_status(self) -> None:
        code = int(self.status.item())
        if code != 0:
            raise SparseStepError(self.index, code)

    # ------------------------------------------------------------------ views and state
    def view(self, buf: torch.Tensor, seg: int) -> torch.Tensor:
        s = self.layout.segments[seg]
        return buf[s.off : s.off + s.numel]

    def stream_of(self, slot: int, src: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(idx, val) of one received stream, for tests and debugging; narrow tensors are decoded."""
        cap = self.layout.cap
        w = self.wiring
        pairs = w.recv_local.view(torch.int32)[: 2 * w.world * cap * 2].view(2, w.world, cap, 2)
        e = pairs[slot, src]
        idx, val = e[:, 0].clone(), e[:, 1].clone().view(torch.float32)
        for s in self.layout.segments:
            if self.layout.is_narrow(s) and s.k:
                # the first s.k 32-bit words of the tensor's region: (relative index : 16 | bf16 value : 16)
                words = e[s.out_off : s.out_off + s.k].reshape(-1)[: s.k].contiguous()
                none = words == -1
                idx[s.out_off : s.out_off + s.k] = torch.where(none, words, (words & 0xFFFF) + s.off)
                val[s.out_off : s.out_off + s.k] = torch.where(none, torch.zeros_like(words), words & -65536).view(torch.float32)
        return idx, val

    def _all_thresholds_set(self) -> bool:
        inited = self.seg_state()["inited"]
        return all(bool(inited[i]) for i, s in enumerate(self.layout.segments) if not s.skip)

    def seg_state(self) -> np.ndarray:
        return self.state.cpu().numpy().view(B.SEG_STATE_DTYPE).copy()

    def state_dict(self) -> dict:
        d = {
            "resid": self.resid, "param": self.param, "m": self.m, "seg_state": self.state,
            "opt": self.opt, "counters": self.counters, "stamp": self.stamp, "ratio": self.ratio,
            "state_range": (self.state_lo, self.state_hi),
        }
        for k in ("v", "vmax", "last"):
            t = getattr(self, k)
            if t is not None:
                d[k] = t
        return {k: (v.detach().cpu().clone() if torch.is_tensor(v) else v) for k, v in d.items()}

    def load_state_dict(self, d: dict) -> None:
        src_range = tuple(d.get("state_range", (0, self.layout.n_total)))
        mine = (self.state_lo, self.state_hi)
        if src_range != mine and src_range != (0, self.layout.n_total):
            raise ValueError("checkpoint was written with a different partition of the optimiser state")
        if abs(d["ratio"] - self.ratio) > 1e-12:
            self.set_ratio(d["ratio"])
        for k in ("resid", "param", "opt"):
            getattr(self, k).copy_(d[k])
        self.counters[:4].copy_(d["counters"][:4])       # epochs and completion counters; the rest is scratch
        # per-element state: the checkpoint holds this rank's range, or the whole bucket (a gathered file)
        off = 0 if src_range == mine else self.state_lo
        n_state = self.state_hi - self.state_lo
        for k in ("m", "v", "vmax", "last", "stamp"):
            t = getattr(self, k)
            if t is None:
                continue
            if k == "stamp" and (k not in d or src_range != mine):
                t.zero_()           # no stamps for this layout in the file; epochs start above zero
                continue
            if k not in d:
                continue
            t[:n_state].copy_(d[k][off : off + n_state])
        self.state.copy_(d["seg_state"])
        self.thresholds_ready = self._all_thresholds_set()
        self._opt_host = self.opt.cpu().numpy().view(B.OPT_STATE_DTYPE).copy()
        self.acc.zero_()
        self.grad.zero_()


class CandidateScratch:
    """Scratch for the undecided items of the threshold bin, shared by all buckets that run their
    selects on one stream (worst case: every item of the largest bucket)."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.cap = 0
        self.buf: Optional[torch.Tensor] = None
        self.cursor = torch.zeros(1, dtype=torch.int32, device=device)
        self._bound: list = []

    def reserve(self, items: int) -> None:
        if items > self.cap:
            self.cap = items
            self.buf = torch.empty(items * 2, dtype=torch.int32, device=self.device)
            for h in self._bound:
                self.bind(h, remember=False)

    def bind(self, handle, remember: bool = True) -> None:
        handle.set_scratch(self.buf.data_ptr(), self.cursor.data_ptr(), self.cap)
        if remember and not any(h is handle for h in self._bound):
            self._bound.append(handle)
