from .lora import (GroupedLoRA, GroupedMLPLoRA, LoraConfig, LoRALinear, apply_lora_delta, apply_peft, build_lora_delta_map,
                   compute_dora_magnitude, expand_all_linear_targets, init_lora_tensor)

__all__ = ["GroupedLoRA", "GroupedMLPLoRA", "LoraConfig", "LoRALinear", "apply_lora_delta", "apply_peft",
           "build_lora_delta_map", "compute_dora_magnitude", "expand_all_linear_targets", "init_lora_tensor"]
