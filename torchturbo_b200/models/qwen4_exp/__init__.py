from .model import TurboQwen4ExpForConditionalGeneration
from .modeling import Qwen4ExpConfig, Qwen4ExpTextConfig

__all__ = ["Qwen4ExpConfig", "Qwen4ExpTextConfig", "TurboQwen4ExpForConditionalGeneration"]
