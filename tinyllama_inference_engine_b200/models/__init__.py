from . import llama, marutar, redasun, zirutar  # noqa: F401  (register LlamaForCausalLM, Marutar, Redasun and Zirutar)
from .model import DecoderModel, cache_needs, expected_tensors

__all__ = ["DecoderModel", "cache_needs", "expected_tensors"]
