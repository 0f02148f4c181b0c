"""Engine-backed swift pipelines.

`make_pipeline(stage)` derives `(EnginePipelineMixin, Swift<Sft|Pretrain|RLHF>)`.  Construction parses swift's
arguments *without* loading the model, builds the engine from them (+ `--tt_*` flags), parks it in `session`, registers
the engine's model types and trainers with swift, and only then lets swift run its usual preparation: its model
factory now reaches `EngineModelMixin.get_model`.  `prepare_model` (swift's tuner / freeze / LoRA step) is bypassed,
because the engine has applied those before sharding.  The DPO pipeline marks the reference load so that it comes
back frozen.  (adapters/msswift/pipeline.py:24-136 of the reference.)"""
from __future__ import annotations

import importlib
from typing import Any

from ...logging import get_logger
from . import session
from .plugins import SwiftPluginHost
from .stages import get_stage
from .utils import build_config_from_swift_args, build_lora_config_from_swift_args

logger = get_logger(__name__)
_CACHE: dict[str, type] = {}


class EnginePipelineMixin:
    turbo_stage = "sft"

    def __init__(self, args: Any = None) -> None:
        from swift.pipelines.base import SwiftPipeline

        SwiftPipeline.__init__(self, args)          # argument parsing only; the concrete __init__ would load the model
        self.train_msg: dict = {}
        self._build_engine()
        for step in ("_prepare_model_tokenizer", "_prepare_template", "_prepare_flash_ckpt"):
            fn = getattr(self, step, None)
            if fn is not None:
                fn()

    def _build_engine(self) -> None:
        from ...engine import TorchTurboEngine
        from .model_registry import register_models_to_swift, register_trainers_to_swift

        cfg = build_config_from_swift_args(self.args, type(self).turbo_stage)
        eng = TorchTurboEngine(cfg)
        self._plugin_host = SwiftPluginHost()
        self._plugin_host.install_plugins(eng.plugins)
        eng.peft_config = build_lora_config_from_swift_args(self.args)
        session.set_engine(eng, stage=type(self).turbo_stage)
        register_models_to_swift()
        register_trainers_to_swift()
        mt = getattr(self.args, "model_type", None)
        if mt and not str(mt).startswith("turbo_"):
            from ...models.registry import list_models

            if mt in list_models():
                self.args.model_type = f"turbo_{mt}"
        logger.info_rank0("%s: engine ready (precision %s)", type(self).__name__, cfg.mixed_precision.value)

    def prepare_model(self, args=None, model=None, template=None, train_dataset=None, **kwargs):
        return model if model is not None else self.model

    def _prepare_dataset(self):
        taken = self._plugin_host.dataset_bridge.try_takeover(args=self.args, template=self.template,
                                                              show_dataset=getattr(self, "_show_dataset", None))
        return taken if taken is not None else super()._prepare_dataset()

    def _get_trainer_kwargs(self):
        base = super()._get_trainer_kwargs() if hasattr(super(), "_get_trainer_kwargs") else {}
        return {**base, "plugin_collator": self._plugin_host.dataset_bridge.collator_for(self.args)}


class _PretrainChecks:
    def _get_dataset(self):
        from .data_check import validate_raw_dataset

        train, val = super()._get_dataset()
        validate_raw_dataset(train, "train")
        validate_raw_dataset(val, "val")
        return train, val


class _ReferenceRole:
    def _prepare_single_model(self, key, origin_key, model_type, model_revision):
        if (origin_key or key) != "ref":
            return super()._prepare_single_model(key, origin_key, model_type, model_revision)
        with session.loading_role("reference"):
            return super()._prepare_single_model(key, origin_key, model_type, model_revision)


def make_pipeline(stage: str) -> type:
    if stage in _CACHE:
        return _CACHE[stage]
    spec = get_stage(stage)
    native = getattr(importlib.import_module(spec.pipeline_module), spec.pipeline_attr)
    native = getattr(native, "_tt_native", native)
    extra = {"pt": (_PretrainChecks,), "dpo": (_ReferenceRole,)}.get(stage, ())
    name = f"Engine{spec.pipeline_attr}"
    cls = type(name, (EnginePipelineMixin, *extra, native), {"turbo_stage": stage, "_tt_native": native, "__module__": __name__})
    globals()[name] = cls
    _CACHE[stage] = cls
    return cls
