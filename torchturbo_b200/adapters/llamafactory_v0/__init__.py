"""LlamaFactory 0.9.x adapter: SFT, PT (continued pre-training) and DPO through LlamaFactory's HF Trainer loops.

Activation installs `DictFieldPatch` and `RunExpPatch`.  When `run_exp` is then called for a supported stage, the
engine is built from LlamaFactory's parsed arguments (+ `--tt_*` flags / env / config file), the remaining patches
are applied for the duration of the run (model loading through the engine, reference-model factory, trainer classes
with the engine mixins, accelerate pass-through, collator normalisation, logging and pre-training fixes) and reverted
afterwards; other stages run stock LlamaFactory.  The framework is not part of this environment, so every target is
looked up lazily (adapters/llamafactory_v0/__init__.py:56-157 of the reference).
"""
from __future__ import annotations

from typing import Any

from ...registry import BaseAdapter, register_adapter
from .compat import get_llamafactory_version, is_llamafactory_installed, is_llamafactory_v0, is_llamafactory_v1
from .patches import (ADAPTER_PATCHES, ENGINE_PATCHES, AcceleratorPatch, CreateRefModelPatch, DictFieldPatch, LoadModelPatch,
                      LogCallbackPatch, PackedInputCollatorPatch, PretrainProcessorPatch, RegisterAutoclassPatch, RunExpPatch,
                      TrainerClassPatch, find_base_model_class)
from .trainer import (LlamaFactoryInputCollator, TorchTurboDPOTrainer, TorchTurboTrainerBase, copy_model_state,
                      make_torchturbo_trainer, unwrap_torchturbo_trainer_class)
from .utils import (SUPPORTED_STAGES, build_config_from_lf_args, build_lora_config_from_lf_args, compute_sft_loss,
                    fsdp_options_from_raw_args, pack_with_vision_boundaries, preprocess_multimodal_pretrain,
                    raise_if_unsupported_lf_args, resolve_cpu_offload, strip_lora_args, take_over_gradient_checkpointing)


@register_adapter("llamafactory_v0")
class LlamaFactoryV0Adapter(BaseAdapter):
    name, priority, package = "llamafactory_v0", 10, "llamafactory"

    def __init__(self) -> None:
        super().__init__()
        self.engine: Any = None
        self.peft_config: Any = None
        self.model: Any = None
        self.stage: str | None = None
        self._entry = [DictFieldPatch(), RunExpPatch(self)]
        for cls in ADAPTER_PATCHES:
            self.add_patch(cls(self))
        for cls in ENGINE_PATCHES:
            self.add_patch(cls())

    def framework_version(self) -> str | None:
        return get_llamafactory_version() or super().framework_version()

    def detect(self) -> bool:
        return is_llamafactory_v0()

    def activate(self) -> None:
        if not is_llamafactory_installed():
            raise RuntimeError("LlamaFactory is not installed in this environment")
        if is_llamafactory_v1():
            raise RuntimeError("this adapter targets the LlamaFactory 0.9 code base (llamafactory.train.tuner); "
                               "the v1 layout is not supported")
        for p in self._entry:
            p.patch()
        super().activate()

    def deactivate(self) -> None:
        for p in reversed(self._entry):
            p.revert()
        super().deactivate()


__all__ = ["LlamaFactoryV0Adapter", "SUPPORTED_STAGES", "build_config_from_lf_args", "build_lora_config_from_lf_args",
           "compute_sft_loss", "fsdp_options_from_raw_args", "pack_with_vision_boundaries", "preprocess_multimodal_pretrain",
           "raise_if_unsupported_lf_args", "resolve_cpu_offload", "strip_lora_args", "take_over_gradient_checkpointing",
           "LlamaFactoryInputCollator", "TorchTurboTrainerBase", "TorchTurboDPOTrainer", "make_torchturbo_trainer",
           "unwrap_torchturbo_trainer_class", "copy_model_state", "find_base_model_class", "DictFieldPatch", "RunExpPatch",
           "PackedInputCollatorPatch", "LoadModelPatch", "CreateRefModelPatch", "TrainerClassPatch", "AcceleratorPatch",
           "RegisterAutoclassPatch", "LogCallbackPatch", "PretrainProcessorPatch"]
