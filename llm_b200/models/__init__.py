from . import fopivik, llama, tevudra  # noqa: F401  (register Fopivik, LlamaForCausalLM, Tevudra)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = ["LayerSpec", "ModelSpec", "PartSpec"]
