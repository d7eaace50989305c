"""Training frontend: wraps an ordinary ``nn.Module`` so that ``model(x)`` / ``loss.backward()`` drive the
sparse data-parallel engine.

Covers the reference's ``FasterDpModelWrapper`` and ``StellaTrainDataLoader`` protocol
(backend/src/python/fasterdp/model_wrapper.py:13-184): the first forward registers the parameters, the
first micro-iteration of an iteration waits for the model updates it must see, ``step()`` checks
replica parity in debug mode, ``zero_grad()`` is a warning because gradients are zeroed by the engine.

Model families the reference can cut into a layer sequence (torchvision ResNet, VGG, VisionTransformer,
SwinTransformer, and a GPT class: model_wrapper.py:113-184) are handled by :func:`to_sequential`.  The
engine here gates per bucket of parameters rather than per layer, so *any* module can be wrapped; the
sequence form is kept for users who relied on it and for per-stage inspection.
"""
from __future__ import annotations

import warnings
from typing import Callable, Dict, List, Optional, Type

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import frontend
from ..utils.loader import current_micro_step


# ------------------------------------------------------------------------------------------------
# stage adapters: small modules that turn non-module glue of a model's forward() into stages
# ------------------------------------------------------------------------------------------------
class Lambda(nn.Module):
    """A parameter-free stage defined by a function."""

    def __init__(self, fn: Callable, label: str = "lambda"):
        super().__init__()
        self.fn, self.label = fn, label

    def forward(self, x):
        return self.fn(x)

    def extra_repr(self) -> str:
        return self.label


class PatchEmbedStage(nn.Module):
    """ViT input stage: patch projection, flatten to tokens, prepend the class token."""

    def __init__(self, vit: nn.Module):
        super().__init__()
        self.conv_proj = vit.conv_proj
        self.class_token = vit.class_token
        self.patch, self.image, self.dim = vit.patch_size, vit.image_size, vit.hidden_dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n, _, h, w = x.shape
        if h != self.image or w != self.image:
            raise ValueError(f"expected {self.image}x{self.image} images, got {h}x{w}")
        tokens = self.conv_proj(x).flatten(2).transpose(1, 2)          # (n, patches, dim)
        return torch.cat([self.class_token.expand(n, -1, -1), tokens], dim=1)


class AddPositionStage(nn.Module):
    def __init__(self, pos_embedding: nn.Parameter):
        super().__init__()
        self.pos_embedding = pos_embedding

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.pos_embedding


class CarryTargets(nn.Module):
    """Applies ``net`` to the activations of an ``(activations, targets)`` pair."""

    def __init__(self, net: nn.Module):
        super().__init__()
        self.net = net

    def forward(self, pair):
        x, targets = pair
        return self.net(x), targets


class GPTEmbedStage(nn.Module):
    def __init__(self, gpt: nn.Module):
        super().__init__()
        self.wte, self.wpe, self.drop = gpt.transformer.wte, gpt.transformer.wpe, gpt.transformer.drop
        self.block_size = gpt.config.block_size

    def forward(self, pair):
        idx, targets = pair
        t = idx.size(1)
        if t > self.block_size:
            raise ValueError(f"sequence length {t} exceeds block size {self.block_size}")
        pos = torch.arange(t, dtype=torch.long, device=idx.device)
        return self.drop(self.wte(idx) + self.wpe(pos)), targets


class GPTHeadStage(nn.Module):
    """Final stage: logits, and the loss when targets were given."""

    def __init__(self, gpt: nn.Module):
        super().__init__()
        self.lm_head = gpt.lm_head

    def forward(self, pair):
        x, targets = pair
        if targets is None:
            return self.lm_head(x[:, [-1], :]), None
        logits = self.lm_head(x)
        return logits, F.cross_entropy(logits.view(-1, logits.size(-1)), targets.view(-1), ignore_index=-1)


# ------------------------------------------------------------------------------------------------
# family registry
# ------------------------------------------------------------------------------------------------
def _resnet_stages(m) -> List[nn.Module]:
    body = [blk for stage in (m.layer1, m.layer2, m.layer3, m.layer4) for blk in stage]
    return [m.conv1, m.bn1, m.relu, m.maxpool, *body, m.avgpool, nn.Flatten(1), m.fc]


def _vgg_stages(m) -> List[nn.Module]:
    return [*m.features, m.avgpool, nn.Flatten(1), *m.classifier]


def _vit_stages(m) -> List[nn.Module]:
    enc = m.encoder
    return [PatchEmbedStage(m), AddPositionStage(enc.pos_embedding), enc.dropout, *enc.layers, enc.ln,
            Lambda(lambda x: x[:, 0], "take class token"), *m.heads]


def _swin_stages(m) -> List[nn.Module]:
    return [*m.features, m.norm, Lambda(lambda x: x.permute(0, 3, 1, 2), "NHWC->NCHW"), m.avgpool,
            nn.Flatten(1), m.head]


def _gpt_stages(m) -> List[nn.Module]:
    return [GPTEmbedStage(m), *[CarryTargets(b) for b in m.transformer.h], CarryTargets(m.transformer.ln_f),
            GPTHeadStage(m)]


def _family_table() -> Dict[Type, Callable]:
    table: Dict[Type, Callable] = {}
    try:
        from torchvision.models.resnet import ResNet
        from torchvision.models.swin_transformer import SwinTransformer
        from torchvision.models.vgg import VGG
        from torchvision.models.vision_transformer import VisionTransformer

        table.update({ResNet: _resnet_stages, VGG: _vgg_stages, VisionTransformer: _vit_stages,
                      SwinTransformer: _swin_stages})
    except ImportError:  # torchvision is optional
        pass
    return table


def to_sequential(module: nn.Module) -> nn.Sequential:
    """Cut a supported model into an ``nn.Sequential`` of stages that computes the same function."""
    if isinstance(module, nn.Sequential):
        return module
    for cls, fn in _family_table().items():
        if isinstance(module, cls):
            return nn.Sequential(*fn(module))
    if module.__class__.__name__ == "GPT" and hasattr(module, "transformer") and hasattr(module, "lm_head"):
        return nn.Sequential(*_gpt_stages(module))
    raise NotImplementedError(f"{module.__class__.__name__} cannot be cut into stages; wrap it with "
                              f"sequential=False to train it as a whole")


# ------------------------------------------------------------------------------------------------
# wrapper
# ------------------------------------------------------------------------------------------------
class SparseDPModelWrapper(nn.Module):
    """``model = SparseDPModelWrapper(torchvision.models.resnet152(num_classes=100)).cuda()``

    ``sequential=True`` reproduces the reference's layer sequence; ``False`` keeps the module as is
    (needed for models whose forward takes several arguments)."""

    def __init__(self, module: nn.Module, sequential: bool = True, **engine_overrides) -> None:
        super().__init__()
        if sequential:
            try:
                module = to_sequential(module)
            except NotImplementedError:
                sequential = False
        self.module = module
        self.sequential = sequential
        self._overrides = engine_overrides
        self.engine = None

    def _ensure_engine(self) -> None:
        if self.engine is not None:
            return
        layers = list(self.module) if isinstance(self.module, nn.Sequential) else [self.module]
        for li, layer in enumerate(layers):
            for name, p in layer.named_parameters():
                if p.requires_grad:
                    frontend.pre_train_init(li, name, p)
        self.engine = frontend.attach(self.module, **self._overrides)

    def forward(self, *args, **kwargs):
        if current_micro_step() < 0 and frontend.gradient_accumulation() > 1:
            raise RuntimeError("gradient accumulation needs StellaTrainDataLoader around the data iterable")
        self._ensure_engine()
        return self.module(*args, **kwargs)

    def step(self) -> Optional[float]:
        """In debug-accuracy mode, measure how far replicas drifted (must be exactly 0)."""
        if self.engine is not None and frontend.is_debug_accuracy_mode():
            drift = self.engine.replica_drift()
            if drift != 0.0:
                raise RuntimeError(f"model replicas diverged: max |delta| = {drift}")
            return drift
        return None

    def zero_grad(self, set_to_none: bool = False) -> None:
        warnings.warn("zero_grad is a no-op: the engine zeroes gradients when it consumes them")

    def synchronize(self) -> None:
        if self.engine is not None:
            self.engine.synchronize()

    def state_dict(self, *args, **kwargs):
        if self.engine is not None:
            self.engine.synchronize()
        return super().state_dict(*args, **kwargs)


FasterDpModelWrapper = SparseDPModelWrapper
