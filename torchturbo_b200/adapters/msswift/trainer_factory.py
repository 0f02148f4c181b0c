"""Module-level names for the engine-backed swift trainers.

swift's `TrainerFactory` stores dotted paths and imports the class by name, and worker processes un-pickle trainer
classes by reference, so the classes must be attributes of a module; but deriving them needs swift's trainer classes,
which must not be imported when this package is.  PEP 562 `__getattr__` builds them on first access.
(adapters/msswift/trainer_factory.py:5-43 of the reference.)"""
from __future__ import annotations

_NAMES = ("EngineSeq2SeqTrainer", "EngineDPOTrainer")


def __getattr__(name: str):
    if name == "EngineSeq2SeqTrainer":
        from .trainer import get_engine_seq2seq_trainer

        cls = get_engine_seq2seq_trainer()
    elif name == "EngineDPOTrainer":
        from .trainer import get_engine_dpo_trainer

        cls = get_engine_dpo_trainer()
    else:
        raise AttributeError(name)
    globals()[name] = cls
    return cls


def __dir__():
    return sorted(list(globals()) + list(_NAMES))
