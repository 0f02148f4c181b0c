"""Stable mapping from the names a model author wrote to the names of the prepared model.

PEFT wrappers (`base_model.model.` prefix, `.base_layer.` segments) and checkpoint wrappers
(`._checkpoint_wrapped_module.`) change `named_parameters()`; plans, freeze patterns and optimizer recipes are written
against the original names.  `build_model_fqn_map` returns {authored FQN: prepared FQN}
(engine/model_fqn.py:28-193 of the reference)."""
from __future__ import annotations

import torch.nn as nn

_WRAPPER_SEGMENTS = ("_checkpoint_wrapped_module", "_fsdp_wrapped_module", "_orig_mod", "base_layer", "module")
_PEFT_PREFIXES = ("base_model.model.",)


def authored_name(prepared: str) -> str:
    name = prepared
    for pre in _PEFT_PREFIXES:
        if name.startswith(pre):
            name = name[len(pre):]
    parts = [p for p in name.split(".") if p not in _WRAPPER_SEGMENTS]
    return ".".join(parts)


def build_model_fqn_map(model: nn.Module, *, parameters: bool = True, modules: bool = True) -> dict[str, str]:
    out: dict[str, str] = {}
    if modules:
        for n, _ in model.named_modules():
            out.setdefault(authored_name(n), n)
    if parameters:
        for n, _ in model.named_parameters():
            a = authored_name(n)
            if ".lora_" in n or "lora_magnitude" in n:
                continue
            out.setdefault(a, n)
    return out
