from .model import Qwen3_5MoeConfig, Qwen3_5MoeTextConfig, TurboQwen3_5MoeForConditionalGeneration

__all__ = ["Qwen3_5MoeConfig", "Qwen3_5MoeTextConfig", "TurboQwen3_5MoeForConditionalGeneration"]
