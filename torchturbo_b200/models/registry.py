"""model_type -> Turbo model class."""
from __future__ import annotations

import importlib
import pkgutil

_MODELS: dict[str, type] = {}
_BUILTINS_LOADED = False


def register_model(model_type: str):
    """Class decorator.  Registering the same type twice with a different class is an error."""

    def deco(cls):
        prev = _MODELS.get(model_type)
        if prev is not None and prev is not cls:
            raise ValueError(f"model_type {model_type!r} is already registered to {prev.__name__}")
        _MODELS[model_type] = cls
        cls.model_type = model_type
        return cls

    return deco


def _register_builtins() -> None:
    """Imports every `models/<package>/model.py` so their `@register_model` decorators run."""
    global _BUILTINS_LOADED
    if _BUILTINS_LOADED:
        return
    _BUILTINS_LOADED = True
    import torchturbo_b200.models as pkg

    for m in pkgutil.iter_modules(pkg.__path__):
        if m.ispkg and m.name not in ("modules",):
            try:
                importlib.import_module(f"{pkg.__name__}.{m.name}.model")
            except ModuleNotFoundError as e:
                if e.name and e.name.endswith(".model"):
                    continue
                raise


def get_model(model_type: str) -> type:
    _register_builtins()
    try:
        return _MODELS[model_type]
    except KeyError as e:
        raise KeyError(f"no Turbo model registered for model_type {model_type!r}; known: {sorted(_MODELS)}") from e


def list_models() -> list[str]:
    _register_builtins()
    return sorted(_MODELS)


def get_all_models() -> dict[str, type]:
    """model_type -> class for every registered family."""
    _register_builtins()
    return dict(_MODELS)
