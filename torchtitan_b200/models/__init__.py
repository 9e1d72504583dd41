"""Model families. ``get_model_spec(name, flavor)`` resolves a registered architecture."""

from .spec import SUPPORTED_MODELS, ModelSpec, get_model_spec

__all__ = ["SUPPORTED_MODELS", "ModelSpec", "get_model_spec"]
