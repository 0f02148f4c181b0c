"""Version probing for LlamaFactory (the 0.9 "v0" code base is the supported one; the re-architected v1 layout is
detected only to refuse it with a clear message).  adapters/llamafactory_v0/compat.py:11-68 of the reference."""
from __future__ import annotations

import importlib
import importlib.util
from importlib import metadata


def get_llamafactory_version() -> str:
    for dist_name in ("llamafactory", "llama-factory", "llama_factory"):
        try:
            return metadata.version(dist_name)
        except metadata.PackageNotFoundError:
            continue
    try:
        mod = importlib.import_module("llamafactory")
        return str(getattr(mod, "__version__", "") or getattr(getattr(mod, "extras", None), "env", object()).__dict__.get("VERSION", ""))
    except Exception:  # noqa: BLE001
        return ""


def _has_module(name: str) -> bool:
    import sys

    if name in sys.modules:
        return True
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError, AttributeError):  # parent missing, or a module object without a spec
        return False


def is_llamafactory_installed() -> bool:
    return _has_module("llamafactory")


def is_llamafactory_v0() -> bool:
    """The layout this adapter patches: `llamafactory.train.tuner.run_exp`, `llamafactory.model.loader.load_model`."""
    if not is_llamafactory_installed():
        return False
    return all(_has_module(m) for m in ("llamafactory.train.tuner", "llamafactory.model.loader"))


def is_llamafactory_v1() -> bool:
    return is_llamafactory_installed() and _has_module("llamafactory.v1") and not is_llamafactory_v0()
