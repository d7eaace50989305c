"""Symmetric device memory: one allocation per rank that every peer maps into its address space.

This is the GPU-side counterpart of the reference's per-node pinned shared-memory pool, which all local
processes map and address through offsets (backend/src/engine/shm_manager.cpp:17-99, 113-187, 288-299).
Here the pool lives in HBM and the "processes" are the GPUs of the NVSwitch domain: a rank stores into a
peer's copy with ordinary st.global (or one multimem store through the switch when a multicast mapping
exists) and signals with epoch flags in the same pool.

Allocation and handle exchange use ``torch.distributed._symmetric_memory`` when it is usable, else CUDA
IPC handles exchanged over the process group; the data movement is always this package's own kernels.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class SymmetricPool:
    """A byte pool with the same layout on every rank; ``peer_ptrs[r]`` is rank r's base address as
    seen from this rank, ``mc_ptr`` the multicast alias (0 when NVLS is unavailable or disabled)."""

    local: torch.Tensor
    peer_ptrs: list[int]
    mc_ptr: int
    world: int
    rank: int
    backend: str
    _keep: list = field(default_factory=list)
    _cursor: int = 0

    def take(self, nbytes: int, align: int = 256) -> int:
        """Reserve ``nbytes`` and return the offset (identical on every rank)."""
        off = (self._cursor + align - 1) // align * align
        if off + nbytes > self.local.numel():
            raise MemoryError(f"symmetric pool exhausted: need {off + nbytes}, have {self.local.numel()}")
        self._cursor = off + nbytes
        return off

    def local_view(self, off: int, nbytes: int) -> torch.Tensor:
        return self.local[off : off + nbytes]

    def peer_addr(self, r: int, off: int) -> int:
        return self.peer_ptrs[r] + off

    def mc_addr(self, off: int) -> int:
        return self.mc_ptr + off if self.mc_ptr else 0


def _alloc_local(nbytes: int, device: torch.device, world: int = 1, rank: int = 0) -> SymmetricPool:
    t = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    return SymmetricPool(t, [t.data_ptr()] * world, 0, world, rank, "local")


def _alloc_torch_symm(nbytes: int, device: torch.device, group) -> SymmetricPool:
    import torch.distributed._symmetric_memory as symm_mem

    t = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    t.zero_()
    hdl = symm_mem.rendezvous(t, group)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    mc = 0
    try:
        mc = int(hdl.multicast_ptr or 0)
    except Exception:
        mc = 0
    # multicast_ptr aliases the start of the underlying block; account for the tensor's offset
    try:
        off = int(hdl.offset)
    except Exception:
        off = 0
    ptrs = [p + off for p in ptrs] if off and ptrs[hdl.rank] != t.data_ptr() else ptrs
    if ptrs[hdl.rank] != t.data_ptr():
        raise RuntimeError("symmetric memory: local pointer mismatch")
    if mc and off:
        mc += off
    return SymmetricPool(t, ptrs, mc, hdl.world_size, hdl.rank, "torch_symm", _keep=[hdl])


def _alloc_ipc(nbytes: int, device: torch.device, group) -> SymmetricPool:
    from .. import _build

    C = _build.load_extension("_C")
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    # cudaMalloc-backed memory is required for IPC export: bypass the expandable-segments allocator
    t = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    handle = C.ipc_get_handle(t.untyped_storage().data_ptr())
    base_off = t.data_ptr() - t.untyped_storage().data_ptr()
    gathered: list = [None] * world
    dist.all_gather_object(gathered, (handle, base_off, os.getpid()), group=group)
    ptrs, opened = [], []
    for r, (h, off, _pid) in enumerate(gathered):
        if r == rank:
            ptrs.append(t.data_ptr())
        else:
            p = C.ipc_open_handle(h)
            opened.append(p)
            ptrs.append(p + off)
    return SymmetricPool(t, ptrs, 0, world, rank, "cuda_ipc", _keep=[opened])


def allocate(nbytes: int, device: torch.device, group=None, prefer: Optional[str] = None,
             multicast: bool = True) -> SymmetricPool:
    """Collective. ``prefer`` in {None, 'torch_symm', 'cuda_ipc', 'local'}; env
    ``STELLATRAIN_SYMM_BACKEND`` overrides. ``multicast=False`` (or env ``STELLATRAIN_NVLS=0``) drops the
    multicast alias so that all pushes use plain peer stores."""
    nbytes = (nbytes + 4095) // 4096 * 4096
    if group is None and not (dist.is_available() and dist.is_initialized()):
        return _alloc_local(nbytes, device)
    world = dist.get_world_size(group)
    if world == 1:
        return _alloc_local(nbytes, device)
    prefer = os.environ.get("STELLATRAIN_SYMM_BACKEND", prefer or "torch_symm")
    if os.environ.get("STELLATRAIN_NVLS", "1") == "0":
        multicast = False
    pool = None
    if prefer == "torch_symm":
        try:
            pool = _alloc_torch_symm(nbytes, device, group if group is not None else dist.group.WORLD)
        except Exception as e:  # noqa: BLE001 - fall back to IPC on any failure of the private API
            if os.environ.get("STELLATRAIN_SYMM_STRICT"):
                raise
            print(f"[stellatrain_b200] torch symmetric memory unavailable ({e!r}); using CUDA IPC", flush=True)
    if pool is None:
        pool = _alloc_ipc(nbytes, device, group if group is not None else dist.group.WORLD)
    if not multicast:
        pool.mc_ptr = 0
    return pool
