from . import linonex, movarax, qwen3, temetar, tilulorn  # noqa: F401  (register Qwen3ForCausalLM, Temetar, Movarax, Linonex and Tilulorn)
from .layout import ModelLayout
from .model import Model, expected_tensors

__all__ = ["ModelLayout", "Model", "expected_tensors"]
