from . import kilurax, llama, marutar, redasun, zirutar  # noqa: F401  (register Kilurax, LlamaForCausalLM, Marutar, Redasun and Zirutar)
from .model import DecoderModel, cache_needs, expected_tensors

__all__ = ["DecoderModel", "cache_needs", "expected_tensors"]
