from .model import TurboQwen3_5ForConditionalGeneration
from .modeling import Qwen3_5Config, Qwen3_5TextConfig

__all__ = ["Qwen3_5Config", "Qwen3_5TextConfig", "TurboQwen3_5ForConditionalGeneration"]
