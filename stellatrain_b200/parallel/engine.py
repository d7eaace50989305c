"""GPU-resident sparse data-parallel engine (one process per GPU).

Role of the reference's ``FasterDpEngine`` (backend/src/engine/core.cpp:64-183, 712-758, 761-834,
1025-1140) with the CPU hop removed: gradients land in flat device buckets, a post-accumulate hook marks
a bucket ready, and the bucket's select+push and scatter+apply kernels run on a high-priority side
stream ordered against the compute stream with events only.  The bounded-staleness protocol of the
reference (backend/src/engine/core.cpp:730-739, 898-908; backend/src/engine/core_module_api.cpp:290) is
kept: with staleness 1 the update of iteration i is applied once backward i+1 of the same bucket has run
and forward i+2 waits for it; staleness 0 applies right after the select.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import buckets as B
from . import symm
from .gpu_bucket import CandidateScratch, GpuBucket, SparseStepError, Wiring


@dataclass
class EngineConfig:
    compressor: str = "thresholdv16"      # default of the reference (backend/src/engine/core.cpp:25)
    ratio: float = 0.99                   # fraction dropped (backend/src/engine/core.cpp:23)
    min_ratio: Optional[float] = None     # lowest ratio the controller may ask for (sizes receive areas)
    optimizer: str = "sgd"
    optimizer_options: dict = field(default_factory=dict)
    staleness: int = 1                    # backend/src/engine/core.cpp:80
    grad_accumulation: int = 1
    bucket_mb: float = 64.0               # few, large buckets: every chain of six launches has a fixed cost
    chunk_elems: int = 8192               # work unit of the streaming passes (one CTA); small units balance the tail
    transport: str = "auto"               # auto | peer | nccl | local
    multicast: bool = True                # use the NVLS multicast alias for pushes when available
    timeout_s: float = 10.0               # bound of every device-side wait
    broadcast_init: bool = True
    divide_k_by_world: bool = True        # k per rank = kept budget / world (compress.cpp:44)
    amsgrad: bool = False
    smart_momentum: bool = False
    grad_mode: str = "steal"              # "steal": kernels read autograd's own gradient tensors through a
                                          # pointer table; "flat": param.grad are views of a flat buffer
    group_size: int = 1                   # > 1: ranks form groups of this size; gradients are summed densely inside a
                                          # group (each rank reducing the tensors it owns) and exchanged sparsely
                                          # between all ranks, with k = kept budget / number of groups per tensor
    state_partition: str = "replicated"   # "owner": every tensor's optimiser state lives on one rank, which receives
                                          # all ranks' entries for it, applies the update and stores the new values
                                          # into every replica (1/world of the state memory, bit-equal replicas)
    wire_format: str = "wide"             # "narrow": tensors below 65536 elements send 4-byte entries (u16 index relative
                                          # to the tensor, bf16 value; the rounding error stays in the residual)
    fine_grained_gating: bool = False     # wait per first-using module instead of at the root
    status_poll_interval: int = 16        # forwards between non-blocking looks at the status words
    deterministic_merge: bool = False     # add the sources' contributions in rank order (one scatter launch per source):
                                          # replicas with replicated state stay bit-equal; world - 1 more launches per bucket
    fused_select: bool = True             # threshold compressors: one pass over gradient and residual once every tensor
                                          # has its threshold (12 bytes per element instead of 16 to 20)
    debug_checks: bool = False            # every stream carries a checksum that the receiver verifies (status 6), consumed
                                          # entries are overwritten with the "no entry" marker; slower, for debugging
    native_hooks: bool = True             # C++ hooks on the parameters and C++ bucket scheduling (csrc/cuda/native_engine.cpp);
                                          # False: the same protocol from Python hooks (needed by profile=True and by the
                                          # library-collective baseline transport)
    step_clock: bool = False              # stamp the device clock at the start of every forward (behind the gate that
                                          # waits for outstanding updates); the telemetry hook switches it on
    profile: bool = False                 # NVTX ranges and CUDA-event timers per bucket and stage (utils/stats.py)


class _BucketRuntime:
    """Host-side state of one bucket.  With the native step engine the counters live there and these fields read
    and write through to it."""

    def __init__(self, bucket: GpuBucket, params: list[nn.Parameter], ga: int):
        self.bucket = bucket
        self.index = bucket.index
        self.params = params
        self.full = len(params) * ga
        self._pending = self.full
        self.grad_ready = torch.cuda.Event()
        self.apply_done: Optional[torch.cuda.Event] = None
        self.select_done: Optional[torch.cuda.Event] = None      # Python hooks: the latest select has read its gradients
        self._has_pending_apply = False
        self._select_count = 0
        self._apply_count = 0
        self.first_module = None
        self.held: list = []          # gradient tensors the current select reads ("steal" mode)
        self.seg_of = {id(p): i for i, p in enumerate(params)}
        self.tab_slot = 0             # row of the pinned pointer-table ring the hooks write now
        self.tab_events: list = [None] * GpuBucket.GRAD_TAB_RING
        self.native = None            # the C++ step engine, when it drives this bucket

    def _push(self, selects=None, applies=None, pending_apply=None) -> None:
        n = self.native
        n.set_counts(self.index, n.select_count(self.index) if selects is None else int(selects),
                     n.apply_count(self.index) if applies is None else int(applies),
                     n.pending_apply(self.index) if pending_apply is None else bool(pending_apply))

    @property
    def select_count(self) -> int:
        return self.native.select_count(self.index) if self.native is not None else self._select_count

    @select_count.setter
    def select_count(self, v: int) -> None:
        if self.native is not None:
            self._push(selects=v)
        else:
            self._select_count = int(v)

    @property
    def apply_count(self) -> int:
        return self.native.apply_count(self.index) if self.native is not None else self._apply_count

    @apply_count.setter
    def apply_count(self, v: int) -> None:
        if self.native is not None:
            self._push(applies=v)
        else:
            self._apply_count = int(v)

    @property
    def has_pending_apply(self) -> bool:
        return self.native.pending_apply(self.index) if self.native is not None else self._has_pending_apply

    @has_pending_apply.setter
    def has_pending_apply(self, v: bool) -> None:
        if self.native is not None:
            self._push(pending_apply=v)
        else:
            self._has_pending_apply = bool(v)

    @property
    def pending(self) -> int:
        """Gradient hooks still to come before the bucket is ready (``full`` between iterations)."""
        return self.native.pending_hooks(self.index) if self.native is not None else self._pending

    @pending.setter
    def pending(self, v: int) -> None:
        if self.native is not None:
            if int(v) != self.full:
                raise ValueError("the native engine only resets the hook counter")
            self._push()
        else:
            self._pending = int(v)


class SparseDPEngine:
    """Owns buckets, streams and the step protocol for one ``nn.Module`` replica."""

    def __init__(self, module: nn.Module, config: Optional[EngineConfig] = None, process_group=None,
                 device: Optional[torch.device] = None) -> None:
        self.cfg = cfg = config or EngineConfig()
        self.module = module
        self.group = process_group
        self.dist_on = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(process_group) if self.dist_on else 1
        self.rank = dist.get_rank(process_group) if self.dist_on else 0
        params = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        if not params:
            raise ValueError("module has no trainable parameters")
        odd = [n for n, p in params if p.dtype != torch.float32]
        if odd:
            # residuals, moments and the master copy are fp32, as in the reference (backend/src/engine/core.cpp:807-830);
            # reduced-precision compute belongs in autocast, which leaves the parameters alone
            raise TypeError(f"the engine keeps fp32 master parameters; {odd[0]} is {dict(params)[odd[0]].dtype} "
                            f"({len(odd)} such tensors): use torch.autocast for bf16/fp16 compute")
        self.device = device or params[0][1].device
        if self.device.type != "cuda":
            raise RuntimeError("the GPU-resident engine needs CUDA parameters; use the CPU tier otherwise")
        torch.cuda.set_device(self.device)
        if cfg.staleness not in (0, 1):
            raise ValueError("staleness must be 0 or 1")
        transport = cfg.transport
        if transport == "auto":
            transport = "local" if self.world == 1 else "peer"
        self.transport = transport
        L = max(1, int(cfg.group_size))
        if self.world % L:
            raise ValueError("world size must be a multiple of group_size")
        self.group_size, self.groups = L, self.world // L
        self.my_group, self.my_local = self.rank // L, self.rank % L
        if L > 1:
            if transport != "peer":
                raise ValueError("grouped mode needs the peer transport")
            cfg.grad_mode = "flat"          # group-mates read each other's gradients: they must sit in the pool
        if cfg.wire_format not in ("wide", "narrow"):
            raise ValueError("wire_format must be 'wide' or 'narrow'")
        if cfg.state_partition not in ("replicated", "owner"):
            raise ValueError("state_partition must be 'replicated' or 'owner'")
        self.partitioned = cfg.state_partition == "owner" and self.world > 1
        if self.partitioned and (transport != "peer" or L > 1):
            raise ValueError("partitioned optimiser state needs the peer transport and group_size 1")
        self.shaper = None
        self._shaped_bytes = 0
        low, high = torch.cuda.Stream.priority_range()
        self.sparse_stream = torch.cuda.Stream(device=self.device, priority=high)
        self.iteration = 0            # completed optimiser iterations (selects issued per bucket)
        self.micro_step = 0
        self._failed: Optional[SparseStepError] = None
        self._capturing = False       # set while a CUDA graph of the step is being captured
        self._pending_weights: list = []   # [from_iteration, device weights, rows written]
        self.capture_version = 0      # bumped by everything that makes a captured step stale (ratio, hyper-parameters are not)
        self._capture_keepalive: list = []
        self._capture_rows: dict = {}     # bucket index -> pinned row of gradient addresses of the running capture
        self._build_buckets(params)
        self._wire()
        self._install_hooks()
        if cfg.optimizer_options:
            self.configure_optimizer(**cfg.optimizer_options)
        if cfg.broadcast_init and self.world > 1:
            self.broadcast_parameters()
        self._status_host = torch.zeros(len(self.buckets), dtype=torch.int32).pin_memory()
        self._status_dev = torch.zeros(len(self.buckets), dtype=torch.int32, device=self.device)
        self._status_event: Optional[torch.cuda.Event] = None
        self.stats = {"select_launches": 0, "apply_launches": 0, "kernels": 0}
        from ..utils.stats import StepTimer
        self.timer = StepTimer(enabled=cfg.profile)

    # ------------------------------------------------------------------ construction
    def _build_buckets(self, params: list[tuple[str, nn.Parameter]]) -> None:
        cfg = self.cfg
        # gradients become ready roughly in reverse registration order
        order = list(reversed(range(len(params))))
        numels = [params[i][1].numel() for i in order]
        groups = B.plan_buckets(numels, int(cfg.bucket_mb * (1 << 20) / 4))
        self.scratch = CandidateScratch(self.device)
        self.buckets: list[_BucketRuntime] = []
        self.param_names: list[list[str]] = []
        self._param_to_bucket: dict[int, int] = {}
        for bi, grp in enumerate(groups):
            idxs = [order[j] for j in grp]
            names = [params[i][0] for i in idxs]
            plist = [params[i][1] for i in idxs]
            layout = B.BucketLayout(names, [p.numel() for p in plist], chunk_elems=cfg.chunk_elems,
                                    narrow_wire=(cfg.wire_format == "narrow"))
            bucket = GpuBucket(
                bi, layout, self.device, compressor=cfg.compressor, ratio=cfg.ratio, world=self.world,
                rank=self.rank, optimizer=cfg.optimizer, amsgrad=cfg.amsgrad,
                smart_momentum=cfg.smart_momentum, min_ratio=cfg.min_ratio, scratch=self.scratch,
                timeout_s=cfg.timeout_s, divide_k_by_world=cfg.divide_k_by_world,
                k_world=(self.groups if (self.group_size > 1 and cfg.divide_k_by_world) else None),
                partition_state=self.partitioned, deterministic_merge=cfg.deterministic_merge,
                fused_select=cfg.fused_select,
            )
            if self.group_size > 1:
                layout.assign_owners(self.group_size, self.my_local)
                bucket.upload_segments()
                bucket.set_weights([1.0 / self.groups] * self.world)   # disjoint tensors inside a group, mean over groups
            with torch.no_grad():
                for seg, p in zip(layout.segments, plist):
                    dense = _dense_like(p)
                    flat_p = bucket.param[seg.off : seg.off + seg.numel]
                    flat_g = bucket.grad[seg.off : seg.off + seg.numel]
                    flat_p.copy_(_flatten_storage_order(dense))
                    p.data = flat_p.as_strided(dense.shape, dense.stride())
                    p.grad = flat_g.as_strided(dense.shape, dense.stride()) if cfg.grad_mode == "flat" else None
            if cfg.grad_mode != "flat":
                bucket.use_grad_table()
            rt = _BucketRuntime(bucket, plist, cfg.grad_accumulation)
            self.buckets.append(rt)
            self.param_names.append(names)
            for p in plist:
                self._param_to_bucket[id(p)] = bi

    def _wire(self) -> None:
        if self.transport == "local":
            if self.world != 1:
                raise ValueError("transport 'local' needs world size 1")
            for rt in self.buckets:
                rt.bucket.wire_local(debug_checks=self.cfg.debug_checks)
            self.pool = None
            return
        W = self.world
        max_n = max(rt.bucket.layout.n_total for rt in self.buckets)
        need = sum(rt.bucket.recv_bytes() + 4 * W * 8 + 1024 for rt in self.buckets) + max_n * 4 + 65536
        if self.group_size > 1:
            need += sum(rt.bucket.layout.n_total * 4 + 4 * self.group_size * 8 + 1024 for rt in self.buckets)
        if self.partitioned:
            need += sum(rt.bucket.recv_bytes() + 2 * W * 8 + 1024 for rt in self.buckets)
        if self.cfg.debug_checks:
            need += len(self.buckets) * (2 * W * 4 + 1024)
        if self.transport == "nccl":
            # library baseline: streams are staged locally and moved by ncclAllGather
            self.pool = symm._alloc_local(need, self.device, 1, 0)
        else:
            self.pool = symm.allocate(need, self.device, self.group, multicast=self.cfg.multicast)
        pool = self.pool
        self._staging_off = pool.take(max_n * 4)
        self._staging_elems = max_n
        for rt in self.buckets:
            b = rt.bucket
            if self.transport == "nccl":
                send = torch.zeros(2 * b.cap_max * 8, dtype=torch.uint8, device=self.device)
                gathered = torch.zeros(b.recv_bytes(), dtype=torch.uint8, device=self.device)
                b._nccl_send, b._nccl_recv = send, gathered
                # select side: a world of one writing into the send buffer; apply side: all sources
                b.wire(Wiring(W, self.rank, gathered, [0] * W, None, [0] * W, None, [0] * W))
                b.wire_select(Wiring(1, 0, send, [send.data_ptr()], None, [0], None, [0]))
                continue
            r_off = pool.take(b.recv_bytes())
            f_off = pool.take(2 * W * 8)
            a_off = pool.take(2 * W * 8)
            extra = {}
            if self.partitioned:
                w_off = pool.take(b.recv_bytes())
                p_off = pool.take(2 * W * 8)
                extra = dict(
                    wb_local=pool.local_view(w_off, b.recv_bytes()), peer_wb=[pool.peer_addr(r, w_off) for r in range(W)],
                    wb_mc=pool.mc_addr(w_off), pflag_local=pool.local_view(p_off, 2 * W * 8).view(torch.int64),
                    peer_pflag=[pool.peer_addr(r, p_off) for r in range(W)],
                )
            if self.cfg.debug_checks:
                c_off = pool.take(2 * W * 4)
                extra.update(cksum_local=pool.local_view(c_off, 2 * W * 4).view(torch.int32),
                             peer_cksum=[pool.peer_addr(r, c_off) for r in range(W)], poison=True)
            b.wire(Wiring(
                world=W, rank=self.rank,
                recv_local=pool.local_view(r_off, b.recv_bytes()),
                peer_recv=[pool.peer_addr(r, r_off) for r in range(W)],
                flag_local=pool.local_view(f_off, 2 * W * 8).view(torch.int64),
                peer_flag=[pool.peer_addr(r, f_off) for r in range(W)],
                ack_local=pool.local_view(a_off, 2 * W * 8).view(torch.int64),
                peer_ack=[pool.peer_addr(r, a_off) for r in range(W)],
                recv_mc=pool.mc_addr(r_off), use_flags=True, use_acks=True, **extra,
            ))
            if self.group_size > 1:
                self._wire_group(rt, r_off)
        if self.dist_on:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)

    def _wire_group(self, rt: "_BucketRuntime", recv_off: int) -> None:
        """Grouped mode: gradients into the pool, ready/done flags, receive areas pre-filled with the
        'no entry' marker because a source never writes the stream regions of tensors it does not own."""
        b, pool, L = rt.bucket, self.pool, self.group_size
        pool.local_view(recv_off, b.recv_bytes()).fill_(0xFF)
        n = b.layout.n_total
        g_off = pool.take(n * 4)
        rdy_off = pool.take(L * 8)
        done_off = pool.take(L * 8)
        b.rebind_grad(pool.local_view(g_off, n * 4).view(torch.float32))
        with torch.no_grad():
            for seg, p in zip(b.layout.segments, rt.params):
                p.grad = b.grad[seg.off : seg.off + seg.numel].as_strided(p.shape, p.stride())
        base = self.my_group * L
        mates = [l for l in range(L) if l != self.my_local]
        b._group_ctr = torch.zeros(1, dtype=torch.int32, device=self.device)
        b.handle.set_group(
            grad_local=b.grad.data_ptr(), mate_grad=[pool.peer_addr(base + l, g_off) for l in mates], mate_local=mates,
            my_local=self.my_local, ready_local=pool.peer_addr(self.rank, rdy_off),
            mate_ready=[pool.peer_addr(base + l, rdy_off) for l in mates], done_local=pool.peer_addr(self.rank, done_off),
            mate_done=[pool.peer_addr(base + l, done_off) for l in mates], group_done_ctr=b._group_ctr.data_ptr(),
        )

    def set_link_shaper(self, shaper, destinations: Optional[int] = None) -> None:
        """Emulate a constrained cross-group link: before a bucket's streams are pushed, a one-thread kernel takes
        the bytes that leave the group from a token bucket in device memory and holds the sparse stream while the
        bucket is in debt (``control.shaper.DeviceTokenBucket``; a host ``TokenBucket`` or a ``BandwidthSchedule`` is
        turned into one, the ranks of a group sharing the scheduled rate).  Works in eager and in captured steps.
        ``destinations`` overrides the number of ranks outside the own group that every stream is charged for (a job
        without a second group can rehearse a shaped link that way)."""
        from ..control.shaper import BandwidthSchedule, DeviceTokenBucket, TokenBucket

        if isinstance(shaper, TokenBucket):
            shaper = DeviceTokenBucket(shaper.schedule, self.device, burst_bytes=int(shaper.burst), share=1.0 / self.group_size)
        elif isinstance(shaper, BandwidthSchedule):
            shaper = DeviceTokenBucket(shaper, self.device, share=1.0 / self.group_size)
        self.shaper = shaper
        self._shaped_bytes = 0
        self._shaped_destinations = destinations
        self._push_shaper()

    def _push_shaper(self) -> None:
        if self.native is None or self.shaper is None:
            return
        self.native.set_shaper(self.shaper.state.data_ptr(), self.shaper.MAX_HOLD_NS)
        for bi, rt in enumerate(self.buckets):
            self.native.set_shaped_bytes(bi, rt.bucket.layout.wire_bytes(owned_only=True) * self._remote_ranks())

    @property
    def shaped_bytes(self) -> int:
        """Bytes charged to the link shaper so far."""
        return self._shaped_bytes + (self.native.shaped_bytes() if self.native is not None else 0)

    @shaped_bytes.setter
    def shaped_bytes(self, v: int) -> None:
        self._shaped_bytes = int(v) - (self.native.shaped_bytes() if self.native is not None else 0)

    def kernels_launched(self) -> int:
        """Kernels of this package launched so far (or, for a captured step, replayed)."""
        return self.stats["kernels"] + (self.native.kernels_launched() if self.native is not None else 0)

    def begin_capture(self) -> None:
        """A CUDA graph of the iteration is about to be captured: gradients of the captured step stay referenced,
        their addresses go to pinned rows of the capture's own."""
        self._capturing = True
        self._capture_keepalive, self._capture_rows = [], {}
        if self.native is not None:
            self.native.begin_capture()

    def end_capture(self) -> list:
        """Returns what the captured step reads on every replay and must therefore outlive it."""
        self._capturing = False
        keep, self._capture_keepalive, self._capture_rows = self._capture_keepalive, [], {}
        if self.native is not None:
            keep = keep + list(self.native.end_capture())
        return keep

    def shaped_bytes_per_step(self) -> int:
        """Bytes this rank stores into other groups per iteration (what the shaper charges)."""
        return sum(rt.bucket.layout.wire_bytes(owned_only=True) for rt in self.buckets) * self._remote_ranks()

    def _remote_ranks(self) -> int:
        d = getattr(self, "_shaped_destinations", None)
        return (self.world - self.group_size) if d is None else int(d)

    # ------------------------------------------------------------------ step clock
    def stamp(self, slot: int) -> None:
        """Write the device clock into slot 0..7 of ``step_stamps`` when the current stream gets here (capturable):
        0 forward begins (behind the wait for outstanding updates), 1 backward begins, 2 backward ended, 3 in front of
        that wait (eager launches), 4 behind the join of a captured iteration with its bucket chains.  Step timing
        that survives CUDA-graph replay."""
        from .. import _build

        if not hasattr(self, "step_stamps"):
            self.step_stamps = torch.zeros(8, dtype=torch.int64, device=self.device)
        _build.load_extension("_C").stamp(self.step_stamps.data_ptr() + 8 * int(slot),
                                          torch.cuda.current_stream(self.device).cuda_stream)

    def _use_native(self) -> bool:
        return bool(self.cfg.native_hooks) and self.transport != "nccl" and not self.cfg.profile

    def _install_native(self) -> None:
        """C++ hooks and C++ bucket scheduling (role of backend/src/engine/core.cpp:775-797 and 1025-1095): from the
        moment autograd has a gradient to the moment the bucket's kernels are in the sparse stream the interpreter is
        not involved.  Buffers, tables and wiring stay where the Python side created them."""
        from .. import _build

        C = _build.load_extension("_C")
        steal = self.cfg.grad_mode != "flat"
        self.native = C.NativeEngine(self.device.index if self.device.index is not None else torch.cuda.current_device(),
                                     self.sparse_stream.cuda_stream, self.cfg.staleness, self.cfg.grad_accumulation)
        for bi, rt in enumerate(self.buckets):
            b = rt.bucket
            segs = b.layout.segments
            got = self.native.add_bucket(
                b.handle, b.select_handle, len(rt.params), steal,
                b.grad_tab_host.data_ptr() if steal else 0, GpuBucket.GRAD_TAB_RING if steal else 0,
                b.grad_tab_dev.data_ptr() if steal else 0, b.grad, [s.off for s in segs], [s.numel for s in segs], 0)
            assert got == bi
            for si, p in enumerate(rt.params):
                self.native.add_param(bi, si, p)
            rt.native = self.native

    def _install_hooks(self) -> None:
        self._hooks = []
        self.native = None
        if self._use_native():
            self._install_native()
        else:
            for bi, rt in enumerate(self.buckets):
                for p in rt.params:
                    self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(bi)))
        # forward gating: wait for the updates this forward must see
        first_owner: dict[int, nn.Module] = {}
        if self.cfg.fine_grained_gating:
            for mod in self.module.modules():
                for p in mod.parameters(recurse=False):
                    bi = self._param_to_bucket.get(id(p))
                    if bi is not None and bi not in first_owner:
                        first_owner[bi] = mod
        gate: dict[int, list[int]] = {}
        for bi, mod in first_owner.items():
            gate.setdefault(id(mod), []).append(bi)
            self.buckets[bi].first_module = mod
        self._gated = set(first_owner.keys())
        for mod in self.module.modules():
            bis = gate.get(id(mod))
            if bis:
                self._hooks.append(mod.register_forward_pre_hook(self._make_gate(bis)))
        self._hooks.append(self.module.register_forward_pre_hook(self._root_pre_forward))

    # ------------------------------------------------------------------ hooks
    def _make_hook(self, bi: int) -> Callable:
        rt = self.buckets[bi]

        steal = self.cfg.grad_mode != "flat"

        def hook(param) -> None:
            rt.pending -= 1
            if steal and rt.pending < len(rt.params):      # last micro-iteration: the gradient is final
                self._note_gradient(rt, param)
            if rt.pending == 0:
                rt.pending = rt.full
                self._bucket_ready(bi)

        return hook

    def _note_gradient(self, rt: _BucketRuntime, p: torch.Tensor) -> None:
        """Record where autograd left this parameter's gradient.  The tensor must have the parameter's
        memory layout and a 16-byte aligned start; otherwise it is copied into the flat buffer."""
        si = rt.seg_of[id(p)]
        seg = rt.bucket.layout.segments[si]
        g = p.grad
        if g.dtype != torch.float32 or g.stride() != p.stride() or (g.data_ptr() & 15):
            flat = rt.bucket.grad[seg.off : seg.off + seg.numel].as_strided(p.shape, p.stride())
            if not self._capturing and rt.select_done is not None:
                torch.cuda.current_stream(self.device).wait_event(rt.select_done)   # a late select may still read this
            flat.copy_(g)
            g = flat
        self._table_row(rt)[si] = g.data_ptr()
        rt.held.append(g)

    def _table_row(self, rt: _BucketRuntime) -> torch.Tensor:
        """Pinned row of gradient addresses the hooks of the running step write: a row of the bucket's ring in eager
        mode; under capture a row of the capture's own, which no eager step ever writes (the captured copy reads it
        on every replay, long after eager steps have moved on through the ring)."""
        if not self._capturing:
            return rt.bucket.grad_tab_host[rt.tab_slot]
        row = self._capture_rows.get(rt.bucket.index)
        if row is None:
            row = rt.bucket.grad_tab_host[0].clone().pin_memory()
            self._capture_rows[rt.bucket.index] = row
            self._capture_keepalive.append(row)
        return row

    def _make_gate(self, bis: list[int]) -> Callable:
        def pre(_mod, _inp) -> None:
            if self._capturing:
                return
            cur = torch.cuda.current_stream(self.device)
            for bi in bis:
                if self.native is not None:
                    self.native.wait_applies(cur.cuda_stream, bi)
                    continue
                ev = self.buckets[bi].apply_done
                if ev is not None:
                    cur.wait_event(ev)
                ev = self.buckets[bi].select_done
                if self.cfg.grad_mode == "flat" and ev is not None:
                    cur.wait_event(ev)

        return pre

    def _root_pre_forward(self, _mod, _inp) -> None:
        if self._failed is not None:
            raise self._failed
        if self._capturing:
            # replays of a captured step serialise on their stream, which already orders this
            # forward after every update of the previous replay
            if self.cfg.step_clock:
                self.stamp(0)
            return
        if torch.is_grad_enabled() and not getattr(self, "_warned_unused", False):
            for bi, rt in enumerate(self.buckets):
                if rt.pending % len(rt.params):
                    # a finished backward leaves every bucket a whole number of micro-iterations short
                    import warnings

                    self._warned_unused = True
                    warnings.warn(f"bucket {bi}: {rt.pending % len(rt.params)} of {len(rt.params)} parameters received no "
                                  f"gradient in the last backward pass; their bucket is exchanged only when all of them "
                                  f"have one (every parameter must take part in every iteration, as in the reference, "
                                  f"whose forward gate would wait for such a tensor forever)", RuntimeWarning, stacklevel=3)
                    break
        if all(rt.pending == rt.full for rt in self.buckets):     # first micro-step of an iteration
            self.before_iteration()
        cur = torch.cuda.current_stream(self.device)
        if self.cfg.step_clock:
            self.stamp(3)             # in front of the waits: (0) - (3) is the time this forward was held back by updates
        if self.native is not None:
            if self._gated:
                for bi in range(len(self.buckets)):
                    if bi not in self._gated:
                        self.native.wait_applies(cur.cuda_stream, bi)
            else:
                self.native.wait_applies(cur.cuda_stream, -1)
            err = self.native.last_error()
            if err:
                raise RuntimeError(f"a CUDA call of the native step engine failed with error {err}")
        else:
            for bi, rt in enumerate(self.buckets):
                if bi in self._gated:
                    continue
                if rt.apply_done is not None:
                    cur.wait_event(rt.apply_done)
                # flat gradient buffer: the coming backward pass accumulates into what the latest select reads and clears
                if self.cfg.grad_mode == "flat" and rt.select_done is not None:
                    cur.wait_event(rt.select_done)
        if self.cfg.step_clock:
            self.stamp(0)             # behind the waits: time spent blocked on updates counts as gap, not as forward
        self._forward_count = getattr(self, "_forward_count", 0) + 1
        if self.cfg.status_poll_interval and self._forward_count % self.cfg.status_poll_interval == 0:
            self._poll_status()

    def _bucket_ready(self, bi: int) -> None:
        rt = self.buckets[bi]
        cur = torch.cuda.current_stream(self.device)
        s = self.sparse_stream
        if self.cfg.grad_mode != "flat":
            b = rt.bucket
            # one table of gradient addresses per bucket on the device: the previous iteration's select, which may still
            # be waiting in the sparse stream (a slow peer, the link shaper), has to have read it before it is rewritten
            if not self._capturing and rt.select_done is not None:
                cur.wait_event(rt.select_done)
            b.grad_tab_dev.copy_(self._table_row(rt), non_blocking=True)   # compute stream, before the event
            if not self._capturing:
                ev = torch.cuda.Event()
                ev.record(cur)
                rt.tab_events[rt.tab_slot] = ev
                rt.tab_slot = (rt.tab_slot + 1) % len(rt.tab_events)
                nxt = rt.tab_events[rt.tab_slot]
                if nxt is not None:
                    nxt.synchronize()       # the copy that last used the next row must be done before it is rewritten
            held, rt.held = rt.held, []
            if not self._capturing:
                for g in held:
                    g.record_stream(s)          # the allocator must not reuse them before the select has read them
            else:
                self._capture_keepalive.extend(held)   # a captured step reads these addresses on every replay
            for p in rt.params:
                p.grad = None
        rt.grad_ready.record(cur)
        s.wait_event(rt.grad_ready)
        if self.cfg.staleness == 1 and rt.has_pending_apply:
            self._apply(rt)
        self._select(rt)
        if self.cfg.staleness == 0:
            self._apply(rt)
        else:
            rt.has_pending_apply = True

    def _select(self, rt: _BucketRuntime) -> None:
        if self.cfg.profile and not self._capturing:
            with self.timer.stage(f"{rt.select_count}@bucket{rt.bucket.index}", "Select", self.sparse_stream):
                self._select_impl(rt)
            self.timer.collect()
        else:
            self._select_impl(rt)

    def _apply(self, rt: _BucketRuntime) -> None:
        if self.cfg.profile and not self._capturing:
            with self.timer.stage(f"{rt.apply_count}@bucket{rt.bucket.index}", "Apply", self.sparse_stream):
                self._apply_impl(rt)
        else:
            self._apply_impl(rt)

    def _select_impl(self, rt: _BucketRuntime) -> None:
        b = rt.bucket
        s = self.sparse_stream
        if self.transport == "nccl":
            b.select(s)
            slot = (rt.select_count + 1) & 1
            cap = b.layout.cap
            send = b._nccl_send.view(torch.int64)[slot * cap : (slot + 1) * cap]
            recv = b._nccl_recv.view(torch.int64)[slot * self.world * cap : (slot + 1) * self.world * cap]
            with torch.cuda.stream(s):
                dist.all_gather_into_tensor(recv, send, group=self.group)
        else:
            if self.group_size > 1:
                b.handle.group_reduce(s.cuda_stream)
                self.stats["kernels"] += 3
            if self.shaper is not None:
                nbytes = b.layout.wire_bytes(owned_only=True) * self._remote_ranks()   # stored into other groups
                self._shaped_bytes += nbytes
                self.shaper.take(nbytes, s)
                self.stats["kernels"] += 1
            b.select(s)
        if self._capturing:
            rt.select_done = None
        else:
            rt.select_done = torch.cuda.Event()
            rt.select_done.record(s)
        rt.select_count += 1
        self.stats["select_launches"] += 1
        self.stats["kernels"] += (b.select_handle or b.handle).select_kernels

    def _apply_impl(self, rt: _BucketRuntime) -> None:
        s = self.sparse_stream
        rt.bucket.handle.apply(s.cuda_stream)
        ev = torch.cuda.Event()
        ev.record(s)
        rt.apply_done = ev
        rt.has_pending_apply = False
        rt.apply_count += 1
        self.stats["apply_launches"] += 1
        self.stats["kernels"] += rt.bucket.apply_kernels

    # ------------------------------------------------------------------ public control
    def synchronize(self) -> None:
        """Flush every pending update and wait for the sparse stream
        (role of backend/src/engine/core.cpp:1097-1140)."""
        cur = torch.cuda.current_stream(self.device)
        if self.native is not None:
            self.native.flush(cur.cuda_stream)
            err = self.native.last_error()
            if err:
                raise RuntimeError(f"a CUDA call of the native step engine failed with error {err}")
        else:
            self.sparse_stream.wait_stream(cur)
            for rt in self.buckets:
                if rt.has_pending_apply:
                    self._apply(rt)
            cur.wait_stream(self.sparse_stream)
        self.sparse_stream.synchronize()
        self.check_status()

    def device_timeline(self) -> list:
        """Per bucket: device-clock durations of the latest select + push and apply (``GpuBucket.device_times``)."""
        self.sparse_stream.synchronize()
        return [rt.bucket.device_times() for rt in self.buckets]

    def export_stats(self, path: Optional[str] = None) -> str:
        """Per-bucket stage times as JSON ``{"<iteration>@bucket<i>": {"Select": ms, "Apply": ms}}``
        (the reference writes /tmp/time_log_<timestamp>_<pid>.json, backend/src/engine/core.cpp:1176-1207)."""
        torch.cuda.synchronize(self.device)
        return self.timer.export_json(path)

    def barrier(self) -> None:
        torch.cuda.synchronize(self.device)
        if self.dist_on:
            dist.barrier(self.group)

    def _poll_status(self) -> None:
        """Non-blocking: looks at the status words copied to pinned memory after an earlier step."""
        if self._status_event is not None and self._status_event.query():
            bad = torch.nonzero(self._status_host).flatten()
            if len(bad):
                bi = int(bad[0])
                self._failed = SparseStepError(bi, int(self._status_host[bi]))
                raise self._failed
            self._status_event = None
        if self._status_event is None:
            s = self.sparse_stream
            with torch.cuda.stream(s):
                torch.stack([rt.bucket.status[0] for rt in self.buckets], out=self._status_dev)
                self._status_host.copy_(self._status_dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(s)
            self._status_event = ev

    def check_status(self) -> None:
        for rt in self.buckets:
            try:
                rt.bucket.check_status()
            except SparseStepError as e:
                self._failed = e
                raise

    def configure_optimizer(self, **options) -> None:
        """Hyper-parameters by the reference's option names (backend/src/optim/sgd.cpp:266-297,
        backend/src/optim/adam.cpp:91-122): lr, momentum, weight_decay, dampening, nestrov/nesterov,
        maximize, smart_momentum; lr, b1, b2, weight_decay, eps, amsgrad, maximize."""
        alias = {"nestrov": "nesterov", "b1": "beta1", "b2": "beta2"}
        opts = {}
        for k, v in options.items():
            k = alias.get(k, k)
            if k == "smart_momentum" and bool(v) and not self.cfg.smart_momentum:
                raise RuntimeError("smart_momentum must be enabled in EngineConfig (it allocates state)")
            if k == "amsgrad" and bool(v) and not self.cfg.amsgrad:
                raise RuntimeError("amsgrad must be enabled in EngineConfig (it allocates state)")
            opts[k] = int(v) if isinstance(v, bool) else v
        for rt in self.buckets:
            rt.bucket.set_optimizer_options(**opts)

    def set_compression_ratio(self, ratio: float) -> None:
        """Takes effect at an iteration boundary: the pipeline is drained first."""
        if not (0.0 < ratio <= 1.0):
            raise ValueError("compression ratio must be in (0, 1]")
        self.synchronize()
        for rt in self.buckets:
            rt.bucket.set_ratio(ratio)
        self.cfg.ratio = ratio
        self._push_shaper()
        self.capture_version += 1     # stream sizes are launch arguments: a captured step is stale now

    def set_rank_weights(self, weights: Iterable[float], from_iteration: Optional[int] = None) -> None:
        """Weight of each rank's gradient in the merge, e.g. batch_r / sum(batch) for unequal per-GPU batch sizes
        (the reference averages with 1/W, cpu_optimize.cpp:55).  Without ``from_iteration`` the pipeline is drained
        and the weights count at once.  With it they count from that iteration on (0-based count of backward passes;
        every rank must name the same one, not earlier than the coming iteration) and nothing is drained: the
        scatter of epoch e reads row e & 1 of a two-row table, and each row is rewritten in stream order between the
        last apply that wants the old weights and the first that wants the new ones."""
        w = [float(x) for x in weights]
        if len(w) != self.world:
            raise ValueError("one weight per rank")
        if from_iteration is None:
            self.synchronize()
            for rt in self.buckets:
                rt.bucket.set_weights(w)
            return
        now = self.iterations_started()
        if from_iteration < now:
            raise ValueError(f"iteration {from_iteration} has begun already (the coming one is {now})")
        dev_w = torch.tensor(w, dtype=torch.float32, device=self.device)
        self._pending_weights.append([int(from_iteration), dev_w, 0])

    def iterations_started(self) -> int:
        """Backward passes begun so far = index of the coming iteration."""
        return self.buckets[-1].select_count if self.buckets else 0

    def before_iteration(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Host work at the start of an iteration (first forward of its micro-steps, or a graph replay): rows of
        the merge-weight table that become due.  Iteration i selects with epoch i + 1; its streams are applied one
        iteration later (staleness 1) or in the same one (staleness 0).  The row of parity (i + 1) & 1 is free once
        the apply of epoch i - 1 has been enqueued, which is the case when iteration i begins."""
        if not self._pending_weights:
            return
        it = self.iterations_started()
        # eager: the sparse stream carries the applies; a replayed graph carries them on the stream it is launched on
        stream = stream if stream is not None else self.sparse_stream
        keep = []
        for entry in self._pending_weights:
            since, w, done = entry
            for step in (0, 1):
                if it == since + step and done == step:
                    with torch.cuda.stream(stream):
                        for rt in self.buckets:
                            rt.bucket.set_weight_row((since + step + 1) & 1, w)
                    entry[2] = done = step + 1
            if done < 2:
                keep.append(entry)
        self._pending_weights = keep

    # ------------------------------------------------------------------ replicas
    def broadcast_parameters(self, src: int = 0) -> None:
        """Make every replica equal to rank ``src`` (backend/src/engine/core.cpp:841-885)."""
        if self.world == 1:
            return
        torch.cuda.synchronize(self.device)
        if self.transport == "peer":
            from .. import _build
            C = _build.load_extension("_C")
            pool = self.pool
            stage = pool.local_view(self._staging_off, self._staging_elems * 4).view(torch.float32)
            s = torch.cuda.current_stream(self.device)
            for rt in self.buckets:
                n = rt.bucket.layout.n_total
                if self.rank == src:
                    stage[:n].copy_(rt.bucket.param)
                torch.cuda.synchronize(self.device)
                dist.barrier(self.group)
                if self.rank != src:
                    C.peer_copy(rt.bucket.param.data_ptr(), pool.peer_addr(src, self._staging_off), n, s.cuda_stream)
                torch.cuda.synchronize(self.device)
                dist.barrier(self.group)
        else:
            for rt in self.buckets:
                dist.broadcast(rt.bucket.param, src=src, group=self.group)
        for mod in self.module.buffers():
            dist.broadcast(mod, src=src, group=self.group)

    def replica_drift(self) -> float:
        """max |param - neighbour's param| over all buckets; 0.0 when replicas agree bit for bit
        (the reference's dry-run model sync, backend/src/engine/core.cpp:843-847, 874-878)."""
        if self.world == 1:
            return 0.0
        self.synchronize()
        out = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self.transport == "peer":
            from .. import _build
            C = _build.load_extension("_C")
            pool = self.pool
            stage = pool.local_view(self._staging_off, self._staging_elems * 4).view(torch.float32)
            s = torch.cuda.current_stream(self.device)
            nb = (self.rank + 1) % self.world
            for rt in self.buckets:
                n = rt.bucket.layout.n_total
                stage[:n].copy_(rt.bucket.param)
                torch.cuda.synchronize(self.device)
                dist.barrier(self.group)
                C.max_abs_diff(rt.bucket.param.data_ptr(), pool.peer_addr(nb, self._staging_off), n,
                               out.data_ptr(), s.cuda_stream)
                torch.cuda.synchronize(self.device)
                dist.barrier(self.group)
            drift = out.view(torch.float32).clone()
        else:
            drift = torch.zeros(1, device=self.device)
            for rt in self.buckets:
                ref = rt.bucket.param.clone()
                dist.broadcast(ref, src=0, group=self.group)
                drift = torch.maximum(drift, (ref - rt.bucket.param).abs().max().reshape(1))
        dist.all_reduce(drift, op=dist.ReduceOp.MAX, group=self.group)
        return float(drift.item())

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        self.synchronize()
        return {
            "format": 1,
            "iteration": [rt.select_count for rt in self.buckets],
            "config": {k: getattr(self.cfg, k) for k in ("compressor", "ratio", "optimizer", "staleness",
                                                         "grad_accumulation", "bucket_mb", "chunk_elems")},
            "param_names": self.param_names,
            "buckets": [rt.bucket.state_dict() for rt in self.buckets],
            "world": self.world,
            "state_partition": "owner" if self.partitioned else "replicated",
        }

    def load_state_dict(self, sd: dict) -> None:
        self.synchronize()
        if sd["param_names"] != self.param_names:
            raise ValueError("checkpoint was written for a different model or bucket plan")
        if sd["world"] != self.world:
            raise ValueError(f"checkpoint world size {sd['world']} != {self.world}: receive slots and "
                             f"per-rank k depend on it")
        for rt, bsd, it in zip(self.buckets, sd["buckets"], sd["iteration"]):
            rt.bucket.load_state_dict(bsd)
            rt.select_count = rt.apply_count = it
            rt.has_pending_apply = False
            rt.pending = rt.full
        if self.transport == "peer":
            # flags and acks restart from the restored epochs
            for rt in self.buckets:
                w = rt.bucket.wiring
                e = int(sd["iteration"][rt.bucket.index])
                w.flag_local.fill_(e)
                w.ack_local.fill_(e)
                if w.pflag_local is not None:
                    w.pflag_local.fill_(e)
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)

    def load_replica_state(self, sd: dict) -> None:
        """Restore only what does not depend on the world size: parameters, optimiser moments and step
        counters, thresholds.  Used when a job resumes with a different number of ranks."""
        self.synchronize()
        if sd["param_names"] != self.param_names:
            raise ValueError("checkpoint was written for a different model or bucket plan")
        for rt, bsd in zip(self.buckets, sd["buckets"]):
            b = rt.bucket
            lo, hi = tuple(bsd.get("state_range", (0, b.layout.n_total)))
            if (lo, hi) != (0, b.layout.n_total):
                raise ValueError("optimiser state in the checkpoint is a shard: merge the ranks' files first "
                                 "(utils.checkpoint.load does)")
            b.param.copy_(bsd["param"])
            for k in ("m", "v", "vmax", "last"):
                t = getattr(b, k)
                if t is not None and k in bsd:
                    t[: b.state_hi - b.state_lo].copy_(bsd[k][b.state_lo : b.state_hi])
            b.opt.copy_(bsd["opt"])
            b._opt_host = b.opt.cpu().numpy().view(B.OPT_STATE_DTYPE).copy()
            b.state.copy_(bsd["seg_state"])
            b.thresholds_ready = b._all_thresholds_set()
            b.resid.zero_(); b.acc.zero_(); b.grad.zero_(); b.stamp.zero_()
        torch.cuda.synchronize(self.device)
        if self.dist_on:
            dist.barrier(self.group)

    def close(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if self.native is not None:
            self.native.remove_hooks()


def _is_dense(t: torch.Tensor) -> bool:
    """True when the elements occupy numel() consecutive slots in some permutation of the dims."""
    expect = 1
    for size, stride in sorted(((sz, st) for sz, st in zip(t.shape, t.stride()) if sz != 1), key=lambda x: x[1]):
        if stride != expect:
            return False
        expect *= size
    return True


def _dense_like(p: torch.Tensor) -> torch.Tensor:
    """The parameter itself when its memory is dense and non-overlapping (any permutation of
    strides, e.g. channels_last), else a contiguous copy."""
    d = p.detach()
    return d if _is_dense(d) else d.contiguous()


def _flatten_storage_order(t: torch.Tensor) -> torch.Tensor:
    """Elements of a dense tensor in the order they sit in memory."""
    if t.is_contiguous():
        return t.reshape(-1)
    order = sorted(range(t.dim()), key=lambda d: (-t.stride(d), d))
    return t.permute(order).contiguous().reshape(-1)
