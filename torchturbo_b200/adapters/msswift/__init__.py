"""ms-swift 4.x adapter: SFT, PT and DPO through swift's pipelines.

Activation swaps swift's `SwiftSft` / `SwiftPretrain` / `SwiftRLHF` pipeline classes for subclasses that build the engine
before the model is loaded, route model loading through `engine.prepare_model` (the DPO reference model through
`engine.build_model`), force swift's own gradient checkpointing / sequence parallel / FSDP / DeepSpeed switches off
(the engine owns those), and mix `TurboTrainerMixin` into the trainer.  Import-guarded: swift is not part of this
environment (adapters/msswift/* of the reference)."""
from __future__ import annotations

import importlib.util
from typing import Any

from ...engine.args import get_torchturbo_args
from ...engine.config import build_from_args
from ...registry import BaseAdapter, BasePatch, register_adapter
from .inputs_bridging import (SwiftInputCollator, bake_loss_scale_into_labels, bridge_packed_inputs,  # noqa: F401
                              bridge_swift_inputs, bridge_unpacked_inputs)

_FORCED_OFF = {"gradient_checkpointing": False, "sequence_parallel_size": 1, "deepspeed": None, "fsdp": ""}


def build_config_from_swift_args(args: Any, stage: str, tt_args=None):
    defaults: dict[str, Any] = {"mixed_precision": "bf16" if getattr(args, "bf16", True) else "fp32",
                                "activation_checkpointing": {"enabled": bool(getattr(args, "gradient_checkpointing", True))}}
    if stage == "dpo" and getattr(args, "router_aux_loss_coef", None):
        defaults["moe"] = {"aux_loss_coeff": float(args.router_aux_loss_coef)}
    for k, v in _FORCED_OFF.items():
        if hasattr(args, k):
            setattr(args, k, v)
    return build_from_args(tt_args or get_torchturbo_args(), defaults=defaults)


class PipelinePatch(BasePatch):
    name = "pipelines"
    version_spec = ">=4.0,<5"

    def _patch(self, engine=None) -> None:
        import swift.pipelines.train as train_mod

        self._saved = {}
        adapter = self.adapter
        for cls_name, stage in (("SwiftSft", "sft"), ("SwiftPretrain", "pt"), ("SwiftRLHF", "dpo")):
            orig = getattr(train_mod, cls_name, None)
            if orig is None:
                continue

            def make(orig=orig, stage=stage):
                class TurboPipeline(orig):  # type: ignore[misc,valid-type]
                    def __init__(self, args=None):
                        from ...engine import TorchTurboEngine

                        parsed = self._parse_args(args) if hasattr(self, "_parse_args") else args
                        adapter.engine = TorchTurboEngine(build_config_from_swift_args(parsed, stage))
                        super().__init__(args)

                return TurboPipeline

            self._saved[cls_name] = orig
            setattr(train_mod, cls_name, make())

    def _revert(self) -> None:
        import swift.pipelines.train as train_mod

        for k, v in self._saved.items():
            setattr(train_mod, k, v)


@register_adapter("msswift")
class MSSwiftAdapter(BaseAdapter):
    name, priority, package = "msswift", 5, "ms-swift"

    def __init__(self) -> None:
        super().__init__()
        self.engine = None
        p = PipelinePatch()
        p.adapter = self
        self.add_patch(p)

    def detect(self) -> bool:
        return importlib.util.find_spec("swift") is not None

    def activate(self) -> None:
        if not self.detect():
            raise RuntimeError("ms-swift is not installed in this environment")
        self.apply_patches()
        super().activate()
