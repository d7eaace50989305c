"""Module-level API with the names of the reference's ``fasterdp`` binding
(backend/src/python/pybind.cpp:18-103, stubs in backend/src/python/fasterdp/__init__.pyi:1-33).

The reference keeps one engine singleton per process and lets Python register parameters one by one;
here the singleton holds the configuration and the per-model engine is created when the wrapped model
sees its first batch.  Rank layout follows the reference: ``world_size`` counts groups ("nodes"),
``local_world_size`` the GPUs of a group, and the global rank is ``rank * local_world_size + local_rank``
(backend/src/engine/core.h:216-217).
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Optional, Union

import torch
import torch.distributed as dist

from .parallel.engine import EngineConfig, SparseDPEngine

__version__ = "0.1.0"

_COMPRESSORS = ("thresholdv16", "thresholdv", "topk", "randomk")


@dataclass
class _GlobalState:
    configured: bool = False
    master_addr: str = "127.0.0.1"
    master_port: int = 5555
    world_size: int = 1          # groups ("nodes" of the reference)
    rank: int = 0                # group rank
    local_world_size: int = 1
    local_rank: int = 0
    session_id: int = 0
    engine_cfg: EngineConfig = field(default_factory=EngineConfig)
    engine: Optional[SparseDPEngine] = None
    pending_params: list = field(default_factory=list)   # (layer_idx, name, param) before the engine exists
    debug_accuracy: bool = bool(int(os.environ.get("STELLATRAIN_DEBUG_ACCURACY", "0")))
    tier: str = "gpu"            # "gpu" (device-resident) or "cpu" (offload tier)


_S = _GlobalState()


def state() -> _GlobalState:
    return _S


def global_rank() -> int:
    return _S.rank * _S.local_world_size + _S.local_rank


def global_world() -> int:
    return _S.world_size * _S.local_world_size


def configure(master_addr: str, master_port: int, world_size: int, rank: int, local_session_id: int,
              local_world_size: int = 1, local_rank: int = 0, method: str = "thresholdv16",
              gradient_accumulation: int = 1, *, backend: Optional[str] = None, staleness: Optional[int] = None,
              transport: Optional[str] = None, timeout_s: float = 600.0, tier: Optional[str] = None) -> None:
    """Bind the process to its GPU and join the job (backend/src/engine/core.cpp:64-183).

    ``tier="cpu"`` selects the CPU-offload tier: the same calls then drive the native host pipeline (pinned shared
    memory, gather, compress, TCP ring between nodes, sparse optimiser) with the reference's meaning of the arguments:
    ``world_size`` nodes of ``local_world_size`` processes each.  That tier brings its own transport, so no
    ``torch.distributed`` group is created."""
    if tier is not None:
        if tier not in ("gpu", "cpu"):
            raise ValueError("tier must be 'gpu' or 'cpu'")
        _S.tier = tier
    if method and method not in _COMPRESSORS:
        raise ValueError(f"unknown compression method {method!r}")
    _S.master_addr, _S.master_port = master_addr, int(master_port)
    _S.world_size, _S.rank = int(world_size), int(rank)
    _S.local_world_size, _S.local_rank = max(1, int(local_world_size)), int(local_rank)
    _S.session_id = int(local_session_id)
    if method:
        _S.engine_cfg.compressor = method
    _S.engine_cfg.grad_accumulation = int(gradient_accumulation)
    if staleness is not None:
        _S.engine_cfg.staleness = int(staleness)
    if transport is not None:
        _S.engine_cfg.transport = transport
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(_S.local_rank % torch.cuda.device_count())
    if _S.tier == "gpu" and global_world() > 1 and not dist.is_initialized():
        be = backend or ("nccl" if use_cuda else "gloo")
        kwargs = {}
        if be == "nccl":
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(
            be, init_method=f"tcp://{master_addr}:{int(master_port)}", world_size=global_world(),
            rank=global_rank(), timeout=datetime.timedelta(seconds=timeout_s), **kwargs,
        )
    _S.configured = True


def configure_compression(method: str) -> None:
    """backend/src/engine/core.cpp:185-195 (which rejects "topk"; here every compressor is accepted)."""
    if method not in _COMPRESSORS:
        raise ValueError(f"unknown compression method {method!r}")
    if _S.engine is not None and method != _S.engine_cfg.compressor:
        raise RuntimeError("the compressor cannot change after the first batch")
    _S.engine_cfg.compressor = method


def configure_compression_ratio(ratio: float) -> None:
    """``ratio`` is the fraction of gradient entries dropped, 0 < ratio <= 1
    (backend/src/engine/core.cpp:197-200)."""
    if not (0.0 < ratio <= 1.0):
        raise ValueError("compression ratio must be in (0, 1]")
    if _S.engine is not None:
        _S.engine.set_compression_ratio(float(ratio))
    _S.engine_cfg.ratio = float(ratio)


def set_optimizer(optimizer_name: str) -> None:
    """backend/src/engine/core.cpp:206-216."""
    if optimizer_name not in ("sgd", "adam"):
        raise ValueError("optimizer must be 'sgd' or 'adam'")
    if _S.engine is not None and optimizer_name != _S.engine_cfg.optimizer:
        raise RuntimeError("the optimizer cannot change after the first batch")
    _S.engine_cfg.optimizer = optimizer_name


_SGD_OPTS = {"lr", "momentum", "weight_decay", "dampening", "nestrov", "nesterov", "maximize", "smart_momentum"}
_ADAM_OPTS = {"lr", "b1", "b2", "weight_decay", "eps", "amsgrad", "maximize"}


def configure_optimizer(option_name: str, option_val: Union[float, bool]) -> None:
    """Options by the reference's names; an unknown one raises ``RuntimeError("NO OPTION")``
    (backend/src/optim/sgd.cpp:266-297, backend/src/optim/adam.cpp:91-122)."""
    allowed = _SGD_OPTS if _S.engine_cfg.optimizer == "sgd" else _ADAM_OPTS
    if option_name not in allowed:
        raise RuntimeError("NO OPTION")
    if option_name == "smart_momentum":
        _S.engine_cfg.smart_momentum = _S.engine_cfg.smart_momentum or bool(option_val)
    if option_name == "amsgrad":
        _S.engine_cfg.amsgrad = _S.engine_cfg.amsgrad or bool(option_val)
    _S.engine_cfg.optimizer_options[option_name] = option_val
    if _S.engine is not None:
        _S.engine.configure_optimizer(**{option_name: option_val})


def gradient_accumulation() -> int:
    return _S.engine_cfg.grad_accumulation


def is_debug_accuracy_mode() -> bool:
    """The reference's compile-time DEBUG_ACCURACY switch (backend/src/engine/config.h:37-59) as a
    runtime flag (env STELLATRAIN_DEBUG_ACCURACY)."""
    return _S.debug_accuracy


def barrier() -> None:
    if _S.engine is not None:
        _S.engine.barrier()
    elif dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dist.barrier()


def synchronize() -> None:
    """backend/src/engine/core.cpp:1097-1140."""
    if _S.engine is not None:
        _S.engine.synchronize()


def attach(module: torch.nn.Module, **overrides) -> SparseDPEngine:
    """Create the engine for ``module`` from the global configuration (idempotent per process)."""
    if _S.engine is not None and _S.engine.module is module:
        return _S.engine
    cfg = _S.engine_cfg
    for k, v in overrides.items():
        setattr(cfg, k, v)
    if _S.tier == "cpu":
        from .cpu_tier import CpuOffloadEngine

        _S.engine = CpuOffloadEngine(
            module, master_addr=_S.master_addr, master_port=_S.master_port, world_size=_S.world_size, rank=_S.rank,
            session=_S.session_id, local_world_size=_S.local_world_size, local_rank=_S.local_rank, method=cfg.compressor,
            gradient_accumulation=cfg.grad_accumulation, staleness=cfg.staleness, ratio=cfg.ratio, optimizer=cfg.optimizer,
            optimizer_options=dict(cfg.optimizer_options), timeout_ms=max(30000, int(cfg.timeout_s * 1000)),
            debug_accuracy=_S.debug_accuracy)
        _S.pending_params.clear()
        return _S.engine
    _S.engine = SparseDPEngine(module, cfg)
    _S.pending_params.clear()
    return _S.engine


def detach() -> None:
    if _S.engine is not None:
        _S.engine.synchronize()
        _S.engine.close()
        _S.engine = None


def pre_train_init(layer_idx: int, name: str, param_tensor: torch.Tensor) -> None:
    """Register one parameter (backend/src/engine/core.cpp:761-834). Parameters registered this way are
    grouped into an engine by :func:`finish_train_init`, which the model wrapper calls."""
    _S.pending_params.append((int(layer_idx), name, param_tensor))


def finish_train_init(module: torch.nn.Module) -> SparseDPEngine:
    return attach(module)


def pre_forward_process(layer_idx: int, name: str) -> None:
    """Make the compute stream wait for the update the coming forward must see
    (backend/src/engine/core.cpp:712-758); the wait is an event on the stream, the host never blocks."""
    eng = _S.engine
    if eng is None or _S.tier == "cpu":      # the CPU tier waits in its own forward hook
        return
    cur = torch.cuda.current_stream(eng.device)
    for rt in eng.buckets:
        if rt.apply_done is not None:
            cur.wait_event(rt.apply_done)


def post_backward_process(layer_idx: int, name: str, grad_tensor: torch.Tensor, param_tensor: torch.Tensor) -> None:
    """The engine's own post-accumulate hooks do this work; kept so that code written against the
    reference's hook protocol (backend/src/engine/core.cpp:1025-1095) keeps running."""
    return None


def force_model_sync(layer_idx: int, name: str, dry_run: bool = False) -> float:
    """dry_run: measure replica drift; otherwise re-broadcast rank 0's parameters
    (backend/src/engine/core.cpp:836-885)."""
    eng = _S.engine
    if eng is None:
        return 0.0
    if dry_run:
        return eng.replica_drift()
    eng.synchronize()
    eng.broadcast_parameters()
    return 0.0


def gather(lst) -> None:
    """No-op, as in the reference (backend/src/python/pybind.cpp:38-40)."""
    return None


def compress(name: str, tensor: torch.Tensor, ratio: float):
    """Standalone compression of one tensor: ``(idx:int32, val:float32)`` with
    ``k = floor((1 - ratio) * numel)`` (backend/src/engine/core.cpp:1210-1245).  CUDA tensors go through
    the sm_100a kernels, CPU tensors through the SIMD tier."""
    from .ops.select import compress_tensor

    return compress_tensor(name, tensor, ratio, _S.engine_cfg.compressor)
