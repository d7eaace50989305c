"""Models by name, the way the reference's driver builds them
(``torchvision.models.<name>(num_classes=...)``, backend/test/test_end_to_end.py:39-45), plus the GPT-2
family and synthetic batches of the matching shape (util/dataloader.py:74-86)."""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn as nn

from .gpt import GPT, GPT2_PRESETS

MODEL_FAMILIES = {
    "resnet": ["resnet18", "resnet34", "resnet50", "resnet101", "resnet152"],
    "vgg": ["vgg11", "vgg16", "vgg19"],
    "vit": ["vit_b_16", "vit_b_32", "vit_l_16"],
    "swin": ["swin_t", "swin_s", "swin_b"],
    "gpt": list(GPT2_PRESETS),
}


def build_model(name: str, num_classes: int = 100, **kw) -> nn.Module:
    if name in GPT2_PRESETS:
        return GPT.from_name(name, **kw)
    import torchvision.models as tvm

    if not hasattr(tvm, name):
        raise ValueError(f"unknown model {name!r}")
    return getattr(tvm, name)(num_classes=num_classes, **kw)


def is_language_model(name: str) -> bool:
    return name in GPT2_PRESETS


def synthetic_batch(name: str, batch: int, num_classes: int = 100, seq_len: int = 1024, device="cpu",
                    generator: torch.Generator | None = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Images N(0,1) of 3x224x224 with labels uniform over the classes, or token ids uniform over the
    vocabulary with next-token targets."""
    if is_language_model(name):
        vocab = GPT2_PRESETS[name].get("vocab_size", 50257)
        t = min(seq_len, GPT2_PRESETS[name].get("block_size", 1024))
        ids = torch.randint(0, vocab, (batch, t + 1), generator=generator, device=device)
        return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    x = torch.randn(batch, 3, 224, 224, generator=generator, device=device)
    y = torch.randint(0, num_classes, (batch,), generator=generator, device=device)
    return x, y
