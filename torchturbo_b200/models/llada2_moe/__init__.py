from .bd import BDDataset, block_diffusion_allow, build_bd_row, first_fit_decreasing, mask_noise
from .generate import generate
from .model import LLaDA2MoeConfig, TurboLLaDA2MoeForCausalLM

__all__ = ["BDDataset", "LLaDA2MoeConfig", "TurboLLaDA2MoeForCausalLM", "block_diffusion_allow", "build_bd_row",
           "first_fit_decreasing", "generate", "mask_noise"]
