from . import famupel, luporax, qwen3, rikanex, vugudra  # noqa: F401  (register the architectures)
from .spec import LayerRun, ModelSpec

__all__ = ["LayerRun", "ModelSpec"]
