"""LlamaFactory 0.9.x adapter: SFT, PT (continued pre-training) and DPO through LlamaFactory's HF Trainer loops.

Activation patches `llamafactory.train.tuner.run_exp`: for the supported stages the engine is built from the
LlamaFactory arguments (+ `--tt_*` flags), model loading goes through `engine.prepare_model`, and the stage's trainer
class gains `TurboTrainerMixin`; other stages fall through to stock LlamaFactory.  The framework is not part of this
environment, so everything here is import-guarded (adapters/llamafactory_v0/* of the reference)."""
from __future__ import annotations

import importlib.util
from typing import Any

from ...engine.args import get_torchturbo_args
from ...engine.config import build_from_args
from ...registry import BaseAdapter, BasePatch, register_adapter

SUPPORTED_STAGES = ("sft", "pt", "dpo")


def build_config_from_lf_args(model_args: Any, training_args: Any, finetuning_args: Any, tt_args=None):
    """Adapter-derived defaults: bf16 follows `--bf16`, activation checkpointing follows LlamaFactory's
    gradient-checkpointing switch (which is then turned off on its side), CPU offload follows `--fsdp offload`."""
    defaults: dict[str, Any] = {"mixed_precision": "bf16" if getattr(training_args, "bf16", False) else "fp32"}
    gc = not getattr(model_args, "disable_gradient_checkpointing", False)
    defaults["activation_checkpointing"] = {"enabled": bool(gc)}
    if "offload" in str(getattr(training_args, "fsdp", "") or ""):
        defaults["backend_config"] = {"cpu_offload": {"enabled": True}}
    if hasattr(model_args, "disable_gradient_checkpointing"):
        model_args.disable_gradient_checkpointing = True
    return build_from_args(tt_args or get_torchturbo_args(), defaults=defaults)


def build_lora_config_from_lf_args(finetuning_args: Any):
    if getattr(finetuning_args, "finetuning_type", "full") != "lora":
        return None
    from ...engine.peft import LoraConfig

    target = getattr(finetuning_args, "lora_target", "all")
    targets = ["all-linear"] if target in ("all", ["all"]) else (target if isinstance(target, list) else str(target).split(","))
    return LoraConfig(r=finetuning_args.lora_rank, lora_alpha=finetuning_args.lora_alpha or 2 * finetuning_args.lora_rank,
                      lora_dropout=getattr(finetuning_args, "lora_dropout", 0.0), target_modules=targets,
                      use_dora=getattr(finetuning_args, "use_dora", False), use_rslora=getattr(finetuning_args, "use_rslora", False))


class RunExpPatch(BasePatch):
    name = "run_exp"
    version_spec = ">=0.9.0,<0.10"

    def _patch(self, engine=None) -> None:
        import llamafactory.train.tuner as tuner

        self._orig = tuner.run_exp
        adapter = self.adapter

        def patched(args=None, callbacks=None):
            from llamafactory.hparams import get_train_args

            model_args, data_args, training_args, finetuning_args, gen_args = get_train_args(args)
            if finetuning_args.stage not in SUPPORTED_STAGES:
                return self._orig(args, callbacks)
            from ...engine import TorchTurboEngine

            adapter.engine = TorchTurboEngine(build_config_from_lf_args(model_args, training_args, finetuning_args))
            adapter.peft_config = build_lora_config_from_lf_args(finetuning_args)
            adapter.apply_patches(adapter.engine)
            return self._orig(args, callbacks)

        tuner.run_exp = patched

    def _revert(self) -> None:
        import llamafactory.train.tuner as tuner

        tuner.run_exp = self._orig


class LoadModelPatch(BasePatch):
    """`load_model` -> `engine.prepare_model` (meta build, sharding, shard-wise weight load)."""

    name = "load_model"
    version_spec = ">=0.9.0,<0.10"

    def _patch(self, engine=None) -> None:
        import llamafactory.model.loader as loader

        self._orig = loader.load_model
        adapter = self.adapter

        def patched(tokenizer, model_args, finetuning_args, is_trainable=False, add_valuehead=False):
            if not is_trainable:
                ref = adapter.engine.build_model(model_args.model_name_or_path)
                for p in ref.parameters():
                    p.requires_grad_(False)
                return ref.eval()
            return adapter.engine.prepare_model(model_args.model_name_or_path, peft_config=adapter.peft_config)

        loader.load_model = patched

    def _revert(self) -> None:
        import llamafactory.model.loader as loader

        loader.load_model = self._orig


class TrainerClassPatch(BasePatch):
    """Insert `TurboTrainerMixin` in front of LlamaFactory's stage trainers."""

    name = "trainer_class"
    version_spec = ">=0.9.0,<0.10"
    _targets = (("llamafactory.train.sft.trainer", "CustomSeq2SeqTrainer"), ("llamafactory.train.pt.trainer", "CustomTrainer"),
                ("llamafactory.train.dpo.trainer", "CustomDPOTrainer"))

    def _patch(self, engine=None) -> None:
        import importlib

        from ..hf_trainer import TurboTrainerMixin

        self._saved = []
        for mod_name, cls_name in self._targets:
            try:
                mod = importlib.import_module(mod_name)
            except ImportError:
                continue
            orig = getattr(mod, cls_name)
            new = type(f"Turbo{cls_name}", (TurboTrainerMixin, orig), {"turbo_engine": engine})
            setattr(mod, cls_name, new)
            self._saved.append((mod, cls_name, orig))

    def _revert(self) -> None:
        for mod, cls_name, orig in self._saved:
            setattr(mod, cls_name, orig)


@register_adapter("llamafactory_v0")
class LlamaFactoryV0Adapter(BaseAdapter):
    name, priority, package = "llamafactory_v0", 10, "llamafactory"

    def __init__(self) -> None:
        super().__init__()
        self.engine = None
        self.peft_config = None
        self._run_exp = RunExpPatch()
        self._run_exp.adapter = self
        for cls in (LoadModelPatch, TrainerClassPatch):
            p = cls()
            p.adapter = self
            self.add_patch(p)

    def detect(self) -> bool:
        return importlib.util.find_spec("llamafactory") is not None

    def activate(self) -> None:
        if not self.detect():
            raise RuntimeError("LlamaFactory is not installed in this environment")
        self._run_exp.patch()
        super().activate()

    def deactivate(self) -> None:
        self._run_exp.revert()
        super().deactivate()
