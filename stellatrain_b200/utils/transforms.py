"""Batch-level augmentations: mixup and cutmix on (B, C, H, W) float batches with integer labels
(the reference vendors torchvision's reference implementations, util/transforms.py:11-180; these are
written against the published definitions: Zhang et al. 2018, Yun et al. 2019)."""
from __future__ import annotations

import math
from typing import Tuple

import torch
from torch import Tensor


def _one_hot(target: Tensor, num_classes: int, dtype) -> Tensor:
    if target.ndim == 1:
        return torch.nn.functional.one_hot(target, num_classes).to(dtype)
    return target.to(dtype)


class _BatchMix(torch.nn.Module):
    def __init__(self, num_classes: int, p: float = 0.5, alpha: float = 1.0, inplace: bool = False) -> None:
        super().__init__()
        if num_classes < 1 or alpha <= 0:
            raise ValueError("num_classes >= 1 and alpha > 0 are required")
        self.num_classes, self.p, self.alpha, self.inplace = num_classes, p, alpha, inplace

    def _check(self, batch: Tensor, target: Tensor) -> Tuple[Tensor, Tensor]:
        if batch.ndim != 4 or not batch.is_floating_point():
            raise TypeError("expected a float batch of shape (B, C, H, W)")
        if not self.inplace:
            batch, target = batch.clone(), target.clone()
        return batch, _one_hot(target, self.num_classes, batch.dtype)

    def _lam(self) -> float:
        return float(torch.distributions.Beta(self.alpha, self.alpha).sample())

    def extra_repr(self) -> str:
        return f"num_classes={self.num_classes}, p={self.p}, alpha={self.alpha}, inplace={self.inplace}"


class RandomMixup(_BatchMix):
    """x <- lam x + (1 - lam) roll(x), same for the one-hot targets, with probability p."""

    def forward(self, batch: Tensor, target: Tensor) -> Tuple[Tensor, Tensor]:
        batch, target = self._check(batch, target)
        if torch.rand(1).item() >= self.p:
            return batch, target
        lam = self._lam()
        mixed = batch * lam + batch.roll(1, 0) * (1.0 - lam)
        return mixed, target * lam + target.roll(1, 0) * (1.0 - lam)


class RandomCutmix(_BatchMix):
    """A random box of area (1 - lam) is pasted from the rolled batch; targets are mixed by the actual
    area ratio, with probability p."""

    def forward(self, batch: Tensor, target: Tensor) -> Tuple[Tensor, Tensor]:
        batch, target = self._check(batch, target)
        if torch.rand(1).item() >= self.p:
            return batch, target
        lam = self._lam()
        h, w = batch.shape[-2:]
        cy, cx = int(torch.randint(h, (1,))), int(torch.randint(w, (1,)))
        r = 0.5 * math.sqrt(1.0 - lam)
        rh, rw = int(r * h), int(r * w)
        y1, y2 = max(cy - rh, 0), min(cy + rh, h)
        x1, x2 = max(cx - rw, 0), min(cx + rw, w)
        rolled = batch.roll(1, 0)
        batch[:, :, y1:y2, x1:x2] = rolled[:, :, y1:y2, x1:x2]
        lam = 1.0 - (y2 - y1) * (x2 - x1) / float(h * w)
        return batch, target * lam + target.roll(1, 0) * (1.0 - lam)
