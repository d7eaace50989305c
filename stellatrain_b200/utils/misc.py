"""Small helpers of the training scripts (role of the reference's util/util.py:11-172): byte accounting
over nested tensors and autograd graphs, running averages, top-k accuracy, run bookkeeping for a
TensorBoard-style writer, and an EMA of model weights."""
from __future__ import annotations

import json
import shutil
import sys
from argparse import Namespace
from pathlib import Path
from typing import Any, Callable, Iterable, Tuple

import torch


def traverse_tensor_sum(obj: Any, fn: Callable[[torch.Tensor], int]) -> int:
    """Sum of fn(t) over every tensor reachable through lists, tuples, sets and dict values."""
    if isinstance(obj, torch.Tensor):
        return int(fn(obj))
    if isinstance(obj, dict):
        return sum(traverse_tensor_sum(v, fn) for v in obj.values())
    if isinstance(obj, (list, tuple, set)):
        return sum(traverse_tensor_sum(v, fn) for v in obj)
    return 0


def get_logical_bytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def get_bytes(obj: Any) -> int:
    """Bytes of the storages behind the tensors in ``obj`` (views of one storage are counted once)."""
    seen = set()

    def one(t: torch.Tensor) -> int:
        st = t.untyped_storage()
        key = st.data_ptr()
        if key in seen:
            return 0
        seen.add(key)
        return st.nbytes()

    return traverse_tensor_sum(obj, one)


def get_bytes_recursive(t: torch.Tensor) -> int:
    """Bytes kept alive by ``t``'s autograd graph: ``t`` itself plus every tensor saved for backward."""
    seen_fn, seen_storage, total = set(), set(), 0

    def add(x: torch.Tensor) -> None:
        nonlocal total
        st = x.untyped_storage()
        if st.data_ptr() not in seen_storage:
            seen_storage.add(st.data_ptr())
            total += st.nbytes()

    add(t)
    stack = [t.grad_fn] if t.grad_fn is not None else []
    while stack:
        fn = stack.pop()
        if fn is None or fn in seen_fn:
            continue
        seen_fn.add(fn)
        for name in dir(fn):
            if name.startswith("_saved_"):
                try:
                    v = getattr(fn, name)
                except RuntimeError:
                    continue
                for x in (v if isinstance(v, (list, tuple)) else [v]):
                    if isinstance(x, torch.Tensor):
                        add(x)
        stack.extend(f for f, _ in fn.next_functions)
    return total


def get_shape(obj: Any):
    if isinstance(obj, torch.Tensor):
        return tuple(obj.shape)
    if isinstance(obj, dict):
        return {k: get_shape(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(get_shape(v) for v in obj)
    return None


class AverageMeter:
    def __init__(self) -> None:
        self.reset()

    def reset(self) -> None:
        self.val = self.sum = self.avg = 0.0
        self.count = 0

    def update(self, val: float, n: int = 1) -> None:
        self.val = val
        self.sum += val * n
        self.count += n
        self.avg = self.sum / max(self.count, 1)


def accuracy(output: torch.Tensor, target: torch.Tensor, topk: Iterable[int] = (1,)) -> Tuple[torch.Tensor, ...]:
    """Top-k accuracies in percent."""
    topk = tuple(topk)
    with torch.no_grad():
        if target.ndim == 2:
            target = target.argmax(1)
        _, pred = output.topk(max(topk), 1, True, True)
        hit = pred.eq(target.view(-1, 1))
        return tuple(hit[:, :k].any(1).float().mean() * 100.0 for k in topk)


def copy_script_file(writer, file_name: str) -> None:
    """Keep a copy of the launching script next to the run's logs."""
    dst = Path(writer.log_dir) / "scripts"
    dst.mkdir(parents=True, exist_ok=True)
    shutil.copy(file_name, dst / Path(file_name).name)


def log_current_config(writer, args: Namespace) -> None:
    d = Path(writer.log_dir)
    d.mkdir(parents=True, exist_ok=True)
    (d / "cmdline.txt").write_text(" ".join(sys.argv))
    (d / "config.json").write_text(json.dumps({k: (v if isinstance(v, (int, float, str, bool, type(None))) else str(v))
                                               for k, v in vars(args).items()}, indent=2))


class ExponentialMovingAverage(torch.optim.swa_utils.AveragedModel):
    """EMA of parameters: avg <- decay * avg + (1 - decay) * param."""

    def __init__(self, model: torch.nn.Module, decay: float, device="cpu") -> None:
        super().__init__(model, device, lambda avg, p, n: decay * avg + (1.0 - decay) * p, use_buffers=True)
