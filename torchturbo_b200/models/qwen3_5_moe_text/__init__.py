from .model import Qwen3_5MoeTextOnlyConfig, TurboQwen3_5MoeTextForCausalLM

__all__ = ["Qwen3_5MoeTextOnlyConfig", "TurboQwen3_5MoeTextForCausalLM"]
