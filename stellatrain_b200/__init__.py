"""stellatrain_b200: sparse data-parallel training on NVIDIA B200 (sm_100a).

Public surface, by the names of the reference's ``fasterdp`` module (backend/src/python/pybind.cpp:18-103)
plus the engine classes of this package::

    import stellatrain_b200 as fasterdp
    fasterdp.configure(addr, port, world_size, rank, session, local_world_size, local_rank, "thresholdv16", 1)
    fasterdp.configure_compression_ratio(0.99)
    model = fasterdp.FasterDpModelWrapper(torchvision.models.resnet152(num_classes=100).cuda())
    fasterdp.set_optimizer("adam"); fasterdp.configure_optimizer("lr", 1e-3)
    for x, y in fasterdp.StellaTrainDataLoader(loader): loss = F.cross_entropy(model(x), y); loss.backward()
    fasterdp.synchronize()
"""
from .frontend import (  # noqa: F401
    __version__, attach, barrier, compress, configure, configure_compression, configure_compression_ratio,
    configure_optimizer, detach, force_model_sync, gather, global_rank, global_world, gradient_accumulation,
    is_debug_accuracy_mode, post_backward_process, pre_forward_process, pre_train_init, set_optimizer,
    state, synchronize,
)
from .models.wrapper import FasterDpModelWrapper, SparseDPModelWrapper, to_sequential  # noqa: F401
from .parallel.engine import EngineConfig, SparseDPEngine  # noqa: F401
from .parallel.gpu_bucket import SparseStepError  # noqa: F401
from .utils.loader import StellaTrainDataLoader  # noqa: F401


def __getattr__(name: str):
    # the CPU-offload tier is imported on first use: its native module is not needed by GPU-only runs
    if name in ("CpuOffloadEngine", "CpuTierTelemetry"):
        from . import cpu_tier

        return getattr(cpu_tier, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
