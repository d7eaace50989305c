"""Micro-batch loader: splits every batch of a wrapped iterable into ``gradient_accumulation`` chunks
along dim 0 and publishes the micro-step (backend/src/python/fasterdp/model_wrapper.py:11-61)."""
from __future__ import annotations

import contextvars
from typing import Any, Iterable, Iterator, Optional

import torch

_micro_step: contextvars.ContextVar[int] = contextvars.ContextVar("stellatrain_micro_step", default=-1)


def current_micro_step() -> int:
    """Index of the micro-iteration being processed, or -1 outside a loader loop."""
    return _micro_step.get()


def _split(obj: Any, parts: int) -> list:
    if isinstance(obj, torch.Tensor):
        chunks = list(torch.chunk(obj, parts, dim=0))
        if len(chunks) != parts:
            raise ValueError(f"cannot split a batch of {obj.shape[0]} into {parts} micro-batches")
        return chunks
    if isinstance(obj, (list, tuple)):
        cols = [_split(o, parts) for o in obj]
        return [type(obj)(c[i] for c in cols) for i in range(parts)]
    if isinstance(obj, dict):
        cols = {k: _split(v, parts) for k, v in obj.items()}
        return [{k: v[i] for k, v in cols.items()} for i in range(parts)]
    return [obj] * parts


class StellaTrainDataLoader:
    def __init__(self, iterable: Iterable, gradient_accumulation: Optional[int] = None) -> None:
        self._iterable = iterable
        self._ga = gradient_accumulation

    def _parts(self) -> int:
        if self._ga is not None:
            return self._ga
        from .. import frontend

        return frontend.gradient_accumulation()

    def __len__(self) -> int:
        return len(self._iterable) * self._parts()

    def __iter__(self) -> Iterator:
        parts = self._parts()
        try:
            for batch in self._iterable:
                for i, micro in enumerate(_split(batch, parts)):
                    _micro_step.set(i)
                    yield micro
        finally:
            _micro_step.set(-1)

    @property
    def is_eoi(self) -> bool:
        """True while the last micro-iteration of an iteration is being processed."""
        step = _micro_step.get()
        if step < 0:
            raise RuntimeError("is_eoi is only defined inside the loader loop")
        return step == self._parts() - 1
