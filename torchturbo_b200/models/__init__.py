from .base import TurboModel, TurboVLMModel
from .registry import get_model, list_models, register_model

__all__ = ["TurboModel", "TurboVLMModel", "get_model", "list_models", "register_model"]
