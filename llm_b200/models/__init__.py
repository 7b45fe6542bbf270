from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = ["LayerSpec", "ModelSpec", "PartSpec"]
