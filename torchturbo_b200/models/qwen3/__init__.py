from .model import TurboQwen3ForCausalLM, get_parallel_plan
from .modeling import Qwen3Config, Qwen3ForCausalLMBase, Qwen3Model

__all__ = ["TurboQwen3ForCausalLM", "Qwen3Config", "Qwen3ForCausalLMBase", "Qwen3Model", "get_parallel_plan"]
