from .model import (Qwen3MoeConfig, Qwen3MoeLayerWrapper, Qwen3MoeModel, TurboQwen3MoeForCausalLM, get_parallel_plan,
                    moe_layer_config)

__all__ = ["Qwen3MoeConfig", "Qwen3MoeLayerWrapper", "Qwen3MoeModel", "TurboQwen3MoeForCausalLM", "get_parallel_plan",
           "moe_layer_config"]
