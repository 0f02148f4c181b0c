"""The engine of the running swift job.

swift's pipeline builds the model through its own factory chain (`get_model_processor -> ModelLoader.get_model`), which
offers no argument to carry an engine through; the pipeline therefore parks the engine here before the model is
loaded, and the loader picks it up.  One training process runs one job, so a module-level slot is enough.  A
"loading role" marks secondary loads (the DPO reference model) so the loader builds a frozen model instead of the
trainable one.  (adapters/msswift/engine_registry.py:20-65 of the reference.)"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Iterator

_state: dict[str, Any] = {"engine": None, "stage": None, "role": None}


def set_engine(engine: Any, stage: str | None = None) -> None:
    _state["engine"] = engine
    if stage is not None:
        _state["stage"] = stage


def get_engine() -> Any:
    if _state["engine"] is None:
        raise RuntimeError("no active engine: an engine-backed pipeline must be constructed before swift loads the model")
    return _state["engine"]


def get_engine_or_none() -> Any:
    return _state["engine"]


def get_stage() -> str | None:
    return _state["stage"]


@contextmanager
def loading_role(role: str | None) -> Iterator[str | None]:
    previous, _state["role"] = _state["role"], role
    try:
        yield role
    finally:
        _state["role"] = previous


def get_loading_role() -> str | None:
    return _state["role"]


def clear() -> None:
    _state.update(engine=None, stage=None, role=None)
