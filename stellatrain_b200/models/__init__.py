"""Model zoo entry points and the training wrapper."""
from .gpt import GPT, GPTConfig, GPT2_PRESETS
from .registry import build_model, synthetic_batch, MODEL_FAMILIES
from .wrapper import FasterDpModelWrapper, SparseDPModelWrapper, to_sequential

__all__ = ["GPT", "GPTConfig", "GPT2_PRESETS", "build_model", "synthetic_batch", "MODEL_FAMILIES",
           "FasterDpModelWrapper", "SparseDPModelWrapper", "to_sequential"]
