from .model import TurboDeepseekV4ForCausalLM
from .modeling import DeepseekV4Config

__all__ = ["DeepseekV4Config", "TurboDeepseekV4ForCausalLM"]
