"""ms-swift 4.x adapter: SFT, PT and DPO through swift's pipelines.

Activation swaps `SwiftSft` / `SwiftPretrain` / `SwiftRLHF` in their modules for engine-backed subclasses
(`pipeline.make_pipeline`).  Such a pipeline builds the engine before the model is loaded, parks it in `session`,
registers the engine's model types (`turbo_<name>`, loader = engine `get_model` in front of the model's native swift
loader) and trainers, forces swift's own gradient checkpointing / sequence parallel / FSDP / DeepSpeed switches off,
bridges the template collator's output to packed rows and mixes the engine trainer in.  Import-guarded: swift is not
part of this environment (adapters/msswift/* of the reference)."""
from __future__ import annotations

import importlib
from typing import Any

from ...registry import BaseAdapter, BasePatch, register_adapter
from . import session
from .compat import SUPPORTED, get_swift_version, is_swift_installed, is_swift_supported
from .data_check import check_row, validate_raw_dataset
from .inputs_bridging import (SwiftInputCollator, bake_loss_scale_into_labels, bridge_packed_inputs,  # noqa: F401
                              bridge_swift_inputs, bridge_unpacked_inputs)
from .plugins import DatasetPluginBridge, SwiftPluginHost
from .stages import SwiftStageSpec, get_stage, iter_stages, register_stage
from .utils import (FORCED_OFF, build_config_from_swift_args, build_lora_config_from_swift_args, raise_if_unsupported,
                    take_over_swift_switches)


class PipelinePatch(BasePatch):
    """Swap every registered stage's pipeline class (and keep the module's `*_main` entry points working: they
    instantiate the class through the module global)."""

    name = "pipelines"
    version_spec = SUPPORTED

    def __init__(self) -> None:
        super().__init__()
        self._saved: list[tuple[Any, str, Any]] = []

    def _patch(self, engine=None) -> None:
        from .pipeline import make_pipeline

        for spec in iter_stages():
            try:
                mod = importlib.import_module(spec.pipeline_module)
            except ImportError:
                continue
            if not hasattr(mod, spec.pipeline_attr):
                continue
            self._saved.append((mod, spec.pipeline_attr, getattr(mod, spec.pipeline_attr)))
            setattr(mod, spec.pipeline_attr, make_pipeline(spec.name))

    def _revert(self) -> None:
        for mod, attr, orig in reversed(self._saved):
            setattr(mod, attr, orig)
        self._saved.clear()
        session.clear()


@register_adapter("msswift")
class MSSwiftAdapter(BaseAdapter):
    name, priority, package = "msswift", 5, "ms-swift"

    def __init__(self) -> None:
        super().__init__()
        self.add_patch(PipelinePatch())

    @property
    def engine(self):
        return session.get_engine_or_none()

    def framework_version(self) -> str | None:
        return get_swift_version() or super().framework_version()

    def detect(self) -> bool:
        return is_swift_installed()

    def activate(self) -> None:
        if not self.detect():
            raise RuntimeError("ms-swift is not installed in this environment")
        if not is_swift_supported():
            raise RuntimeError(f"ms-swift {get_swift_version()} is not supported (need {SUPPORTED})")
        self.apply_patches()
        super().activate()

    def main(self, stage: str, args: Any = None):
        """Run a stage through swift's own entry function (`sft_main`, `pretrain_main`, `rlhf_main`)."""
        spec = get_stage(stage)
        return getattr(importlib.import_module(spec.pipeline_module), spec.main_attr)(args)
