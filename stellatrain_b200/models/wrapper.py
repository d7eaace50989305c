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
    (needed for models whose forward takes several arguments).

    Two ways to run an iteration.  The reference's: ``loss = criterion(model(x), y); loss.backward()``
    (backend/test/test_end_to_end.py:62-76).  Or ``loss = model.train_step(x, y)``, which does the same and, with
    ``graph=True``, captures the whole iteration (forward, loss, backward and the sparse kernels of every bucket)
    in a CUDA graph after ``graph_warmup`` eager iterations and replays it from then on: one launch per iteration
    instead of one host round trip per parameter tensor.  A change of the compression ratio, of the batch shape
    or of the input types makes the capture stale; the next iterations run eagerly and a new capture follows."""

    def __init__(self, module: nn.Module, sequential: bool = True, graph: bool = False, graph_warmup: int = 3,
                 loss_fn: Optional[Callable] = None, autocast_dtype: Optional[torch.dtype] = None,
                 **engine_overrides) -> None:
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
        self.graph = bool(graph)
        self.graph_warmup = max(1, int(graph_warmup))
        self.loss_fn = loss_fn
        self.autocast_dtype = autocast_dtype
        self._graphs: Dict[tuple, object] = {}       # input signature -> GraphedStep
        self._eager_by_key: Dict[tuple, int] = {}
        self._ever_captured = False
        self._seen_version = -1
        self._side_stream = None

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

    # ------------------------------------------------------------------ whole iterations
    def _loss_of(self, *inputs: torch.Tensor) -> torch.Tensor:
        """Forward and loss.  Default rule: a module that computes its own loss from (input, target) and returns
        (output, loss) is called with both (the GPT path of the reference, model_wrapper.py:175-182); any other module
        gets the first tensor and its output meets the second in cross entropy."""
        if self.loss_fn is not None:
            return self.loss_fn(self, *inputs)
        if self.sequential and getattr(self.module[-1], "__class__", type(None)).__name__ == "GPTHeadStage":
            return self((inputs[0], inputs[1]))[1]
        if self.module.__class__.__name__ == "GPT":
            return self(*inputs)[1]
        return F.cross_entropy(self(inputs[0]), inputs[1])

    def _iteration(self, *inputs: torch.Tensor) -> torch.Tensor:
        eng = self.engine
        if eng is not None and not eng.cfg.step_clock:
            eng.stamp(0)                # with the step clock on, the engine stamps behind its forward gate
        if self.autocast_dtype is not None:
            with torch.autocast("cuda", dtype=self.autocast_dtype):
                loss = self._loss_of(*inputs)
        else:
            loss = self._loss_of(*inputs)
        if self.engine is not None and eng is None:
            eng = self.engine           # attached by the first forward
        if eng is not None:
            eng.stamp(1)
        loss.backward()
        if eng is not None:
            eng.stamp(2)
        return loss

    def train_step(self, *inputs: torch.Tensor) -> torch.Tensor:
        """One iteration (forward, loss, backward; the engine updates the parameters).  Returns the loss tensor; with
        ``graph=True`` it is the captured step's output buffer, overwritten by the next replay."""
        self._ensure_engine()
        eng = self.engine
        if not (self.graph and eng.device.type == "cuda") or frontend.gradient_accumulation() > 1:
            return self._iteration(*inputs)
        if self._seen_version != eng.capture_version:       # the ratio changed: captured steps are stale
            self._graphs.clear()
            self._eager_by_key.clear()
            self._seen_version = eng.capture_version
        key = tuple((tuple(t.shape), t.dtype, t.is_contiguous(memory_format=torch.channels_last) if t.dim() == 4 else False)
                    for t in inputs)
        g = self._graphs.get(key)
        if g is not None:
            g.copy_inputs(*inputs)
            return g.replay()
        # Eager iterations run on the stream the capture will use, so that library handles, tuned kernels and the
        # allocator's blocks of that stream are warm when the capture begins.  The first capture waits for
        # ``graph_warmup`` of them; a later one (new ratio, new batch shape) for one, which also brings the engine
        # back to its steady state after the drain that a ratio change implies.
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=eng.device)
        cur = torch.cuda.current_stream(eng.device)
        done = self._eager_by_key.get(key, 0)
        # a drained pipeline (after synchronize(), a checkpoint, a ratio change) is not the state a replay continues
        # from: with staleness 1 every bucket must have an update outstanding, which one more eager iteration restores
        steady = eng.cfg.staleness == 0 or all(rt.has_pending_apply for rt in eng.buckets)
        if done < (1 if self._ever_captured else self.graph_warmup) or not steady:
            self._side_stream.wait_stream(cur)
            with torch.cuda.stream(self._side_stream):
                loss = self._iteration(*inputs)
            cur.wait_stream(self._side_stream)
            for t in inputs:
                t.record_stream(self._side_stream)
            loss.record_stream(cur)
            self._eager_by_key[key] = done + 1
            return loss
        from ..parallel.graphs import GraphedStep

        while len(self._graphs) >= 2:                         # every capture owns a private memory pool
            self._graphs.pop(next(iter(self._graphs)))
        g = GraphedStep(eng, self._iteration, inputs, warmup=0, stream=self._side_stream)
        self._graphs[key] = g
        self._ever_captured = True
        return g.replay()

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
