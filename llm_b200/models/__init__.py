from . import llama, tevudra  # noqa: F401  (register LlamaForCausalLM, Tevudra)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = ["LayerSpec", "ModelSpec", "PartSpec"]
