from .model import TurboQwen3VLForConditionalGeneration, get_parallel_plan
from .modeling import Qwen3VLConfig, Qwen3VLForConditionalGenerationBase, Qwen3VLVisionConfig, VisionTower

__all__ = ["TurboQwen3VLForConditionalGeneration", "get_parallel_plan", "Qwen3VLConfig",
           "Qwen3VLForConditionalGenerationBase", "Qwen3VLVisionConfig", "VisionTower"]
