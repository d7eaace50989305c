"""Standalone compression of single tensors (the reference's ``fasterdp.compress``,
backend/src/engine/core.cpp:1210-1245): no residual is kept between calls, but threshold compressors
keep their per-name threshold exactly like the engine path does."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..parallel import buckets as B

_gpu_cache: Dict[tuple, object] = {}
_cpu_cache: Dict[tuple, object] = {}


def _k_for(numel: int, ratio: float) -> int:
    return max(0, min(numel, int((1.0 - ratio) * numel)))


def compress_tensor(name: str, tensor: torch.Tensor, ratio: float, method: str = "thresholdv16"
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    if tensor.dtype != torch.float32:
        raise TypeError("compress expects a float32 tensor")
    flat = tensor.detach().reshape(-1)
    n = flat.numel()
    k = _k_for(n, ratio)
    if k == 0 or n == 0:
        return (torch.empty(0, dtype=torch.int32, device=tensor.device),
                torch.empty(0, dtype=torch.float32, device=tensor.device))
    if tensor.is_cuda:
        return _compress_cuda(name, flat, k, method)
    return _compress_cpu(name, flat, k, method)


def _compress_cuda(name: str, flat: torch.Tensor, k: int, method: str):
    from ..parallel.gpu_bucket import GpuBucket

    n = flat.numel()
    key = (name, n, method, flat.device.index)
    b = _gpu_cache.get(key)
    if b is None:
        layout = B.BucketLayout([name], [n])
        b = GpuBucket(0, layout, flat.device, compressor=method, ratio=0.0, world=1, rank=0)
        b.wire_local()
        _gpu_cache[key] = b
    # one tensor, explicit k: patch the segment table
    seg = b.layout.segments[0]
    if seg.k != k:
        seg.k, seg.out_off, b.layout.cap = k, 0, k
        from ..parallel.gpu_bucket import _dev_bytes
        b.segs.copy_(_dev_bytes(b.layout.seg_table(), flat.device))
        b._bind()
    b.resid.zero_()
    b.grad[:n].copy_(flat)
    epoch = int(b.counters[0].item())
    b.select()
    torch.cuda.current_stream(flat.device).synchronize()
    b.check_status()
    idx, val = b.stream_of(epoch & 1, 0)
    # the epochs of select and apply advance together in the engine; keep them aligned here too
    b.counters[1] = b.counters[0]
    keep = idx != -1
    keep &= idx < n   # threshold-v16 may name zero padding behind the tensor
    return idx[keep].to(torch.int32), val[keep]


def _compress_cpu(name: str, flat: torch.Tensor, k: int, method: str):
    try:
        from .. import cpu_tier
    except Exception:  # noqa: BLE001 - the native CPU tier is optional for this helper
        cpu_tier = None
    if cpu_tier is not None and cpu_tier.available():
        return cpu_tier.compress(name, flat, k, method)
    from . import oracle as O

    st = _cpu_cache.setdefault((name, flat.numel(), method), O.ThresholdState())
    idx, val, _ = O.compress_step(method, flat, torch.zeros_like(flat), k, st)
    keep = idx < flat.numel()
    return idx[keep].to(torch.int32), val[keep]
