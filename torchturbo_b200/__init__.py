"""torchturbo_b200: a B200-native (sm_100a) LLM / VLM post-training engine.

Importing the package registers the built-in models and framework adapters.  `activate(name)` switches a host
training framework (LlamaFactory, ms-swift) over to this engine; with no name the single detected framework is used.
Set `TORCH_TURBO_DISABLE=1` to make `activate()` a no-op.  The engine is fully usable without a host framework:
see `torchturbo_b200.engine.TorchTurboEngine` and `torchturbo_b200.loops`.
"""
from __future__ import annotations

import importlib
import os
import pkgutil

__version__ = "0.1.0"

from .logging import get_logger  # noqa: E402

logger = get_logger(__name__)
_ADAPTERS_LOADED = False


def _discover_builtin_adapters() -> None:
    """Import every direct sub-package of `adapters` so their `@register_adapter` decorators run."""
    global _ADAPTERS_LOADED
    if _ADAPTERS_LOADED:
        return
    _ADAPTERS_LOADED = True
    from . import adapters

    for m in pkgutil.iter_modules(adapters.__path__):
        if m.ispkg:
            try:
                importlib.import_module(f"{adapters.__name__}.{m.name}")
            except Exception as e:  # an adapter for an absent framework must not break the package
                logger.debug("adapter %s not loaded: %s", m.name, e)


def detect() -> str | None:
    from .detector import FrameworkDetector

    _discover_builtin_adapters()
    return FrameworkDetector().detect()


def activate(name: str | None = None):
    """Activate the adapter `name` (or the only detected one).  Returns the adapter, or None when disabled."""
    if os.environ.get("TORCH_TURBO_DISABLE", "").strip().lower() in {"1", "true", "yes"}:
        logger.info_rank0("TORCH_TURBO_DISABLE is set: not activating")
        return None
    from .detector import FrameworkDetector
    from .registry import get_adapter

    _discover_builtin_adapters()
    if name is None:
        found = FrameworkDetector().detect_all()
        if len(found) != 1:
            raise RuntimeError(f"cannot pick an adapter automatically: detected {found or 'none'}; pass a name")
        name = found[0]
    adapter = get_adapter(name)
    adapter.activate()
    return adapter


def _register_models() -> None:
    from .models.registry import _register_builtins

    _register_builtins()


_register_models()
