from .model import TurboBailingMoeV3ForCausalLM
from .modeling import BailingMoeV3Config

__all__ = ["BailingMoeV3Config", "TurboBailingMoeV3ForCausalLM"]
