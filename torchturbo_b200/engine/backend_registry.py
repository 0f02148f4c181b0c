from __future__ import annotations

_BACKENDS: dict[str, type] = {}


def register_backend(name: str):
    def deco(cls):
        _BACKENDS[str(name)] = cls
        return cls

    return deco


def get_backend(name) -> type:
    key = getattr(name, "value", name)
    if key not in _BACKENDS:
        from .backends.fsdp2 import backend  # noqa: F401  (registers "fsdp2")
    try:
        return _BACKENDS[key]
    except KeyError as e:
        raise KeyError(f"unknown backend {key!r}; known: {sorted(_BACKENDS)}") from e
