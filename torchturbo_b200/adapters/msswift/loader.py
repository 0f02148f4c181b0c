"""Model loading for swift through the engine.

swift resolves a model type to a `ModelMeta` whose `loader` class builds config, processor and model.  The engine
only replaces the *model* part: `EngineModelMixin.get_model` is placed in front of the model's own swift loader, so
`get_processor` / `get_config` and their side effects (vision pre-processing limits read from the environment, custom
tokenizer patches) stay swift's.  Classes are created on demand, cached, and published in this module under their
name so that pickling by reference (dill, dataloader workers) finds them.
(adapters/msswift/loader.py:55-165 of the reference.)"""
from __future__ import annotations

from typing import Any

import torch

from ...logging import get_logger
from . import session

logger = get_logger(__name__)
_CACHE: dict[type | None, type] = {}


def resolve_dtype(raw: Any) -> torch.dtype | None:
    if raw is None or isinstance(raw, torch.dtype):
        return raw
    name = str(raw).replace("torch.", "")
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
             "float32": torch.float32, "fp32": torch.float32, "auto": None}
    if name not in table:
        raise ValueError(f"unknown torch dtype {raw!r}")
    return table[name]


class EngineModelMixin:
    """`get_model(model_dir, config, processor, model_kwargs)` through the running job's engine: the trainable model
    via `prepare_model` (meta build, plan, sharding, LoRA, shard-wise weight load), a frozen one via `build_model`
    while the loading role is "reference"."""

    def get_model(self, model_dir, config, processor, model_kwargs):
        eng = session.get_engine()
        init_kwargs = {"config": config}
        if session.get_loading_role() == "reference":
            logger.info_rank0("building the reference model through the engine (%s)", model_dir)
            ref = eng.build_model(model_dir, init_kwargs=init_kwargs)
            ref.requires_grad_(False)
            return ref.eval()
        logger.info_rank0("building the model through the engine (%s, lora=%s)", model_dir,
                          getattr(eng, "peft_config", None) is not None)
        return eng.prepare_model(model_dir, peft_config=getattr(eng, "peft_config", None), init_kwargs=init_kwargs)

    def _postprocess_model(self, model_dir, model):
        inner = getattr(model, "base_model", None)
        if inner is not None and hasattr(inner, "model") and type(model).__name__.startswith("Peft"):
            model = inner.model
        parent = super()
        if hasattr(parent, "_postprocess_model"):
            parent._postprocess_model(model_dir, model)


def get_engine_model_loader(native_loader_cls: type | None = None) -> type:
    """`(EngineModelMixin, native loader)`; with no native loader, swift's base `ModelLoader`."""
    if native_loader_cls in _CACHE:
        return _CACHE[native_loader_cls]
    base = native_loader_cls
    if base is None:
        from swift.model import ModelLoader as base  # type: ignore[no-redef]
    name = "EngineModelLoader" if native_loader_cls is None else f"EngineModelLoader_{native_loader_cls.__name__}"
    cls = type(name, (EngineModelMixin, base), {"__module__": __name__})
    globals()[name] = cls
    _CACHE[native_loader_cls] = cls
    return cls
