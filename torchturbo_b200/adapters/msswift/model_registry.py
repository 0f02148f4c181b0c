"""Registration of the engine's model families and trainers in swift's registries.

Every family is registered as model type `turbo_<name>`; its meta inherits swift's native meta for `<name>` where one
exists (template, requirements, tags, multimodal flag and above all the native loader, see `loader.py`).  Families may
ship a `swift_template.py` with a `register()` function.  (adapters/msswift/model_registry.py:28-92 of the reference.)"""
from __future__ import annotations

import importlib

from ...logging import get_logger
from .loader import get_engine_model_loader
from .stages import iter_stages

logger = get_logger(__name__)
TRAINER_PATHS = {"causal_lm": "torchturbo_b200.adapters.msswift.trainer_factory.EngineSeq2SeqTrainer",
                 "dpo": "torchturbo_b200.adapters.msswift.trainer_factory.EngineDPOTrainer"}


def register_models_to_swift() -> list[str]:
    from swift.model import Model, ModelGroup, ModelMeta, register_model
    from swift.model.model_meta import MODEL_MAPPING

    from ...models import TurboVLMModel
    from ...models.registry import get_all_models

    done = []
    for name, model_cls in get_all_models().items():
        native = MODEL_MAPPING.get(name)
        loader = get_engine_model_loader(getattr(native, "loader", None) if native is not None else None)
        template = getattr(native, "template", None)
        meta = ModelMeta(model_type=f"turbo_{name}", model_groups=[ModelGroup([Model()], template=template) if native else ModelGroup([Model()])],
                         loader=loader, template=template, architectures=[],
                         is_multimodal=isinstance(model_cls, type) and issubclass(model_cls, TurboVLMModel),
                         requires=list(getattr(native, "requires", []) or []), tags=list(getattr(native, "tags", []) or []),
                         task_type=getattr(native, "task_type", "causal_lm") if native else "causal_lm")
        register_model(meta, exist_ok=True)
        done.append(meta.model_type)
        try:
            mod = importlib.import_module(f"torchturbo_b200.models.{name}.swift_template")
        except ImportError:
            continue
        if hasattr(mod, "register"):
            try:
                mod.register()
            except Exception:  # noqa: BLE001 - a template that cannot register must not stop the job
                logger.warning_rank0("swift template of %s failed to register", name)
    try:
        from ..chat_templates import register_swift_templates, wrap_swift_native_templates

        register_swift_templates()
        wrap_swift_native_templates()
        from .mm_templates import register_swift_mm_templates

        register_swift_mm_templates()
    except Exception as e:  # noqa: BLE001 - another template API: the user's --template must exist already
        logger.warning_rank0("chat templates of the engine's model families were not registered: %s", e)
    logger.info_rank0("registered %d engine model types in swift", len(done))
    return done


def register_trainers_to_swift() -> list[str]:
    from swift.trainers import TrainerFactory

    keys = sorted({s.trainer_key for s in iter_stages()})
    for k in keys:
        TrainerFactory.TRAINER_MAPPING[k] = TRAINER_PATHS[k]
    return keys
