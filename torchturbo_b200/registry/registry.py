from __future__ import annotations

from .adapter import BaseAdapter

_ADAPTERS: dict[str, BaseAdapter] = {}


def register_adapter(name: str | None = None):
    """Class decorator: instantiate the adapter once and make it discoverable by name."""

    def deco(cls):
        inst = cls()
        key = name or inst.name
        inst.name = key
        if key in _ADAPTERS and type(_ADAPTERS[key]) is not cls:
            raise ValueError(f"adapter {key!r} is already registered")
        _ADAPTERS[key] = inst
        return cls

    return deco


def get_adapter(name: str) -> BaseAdapter:
    try:
        return _ADAPTERS[name]
    except KeyError as e:
        raise KeyError(f"unknown adapter {name!r}; known: {sorted(_ADAPTERS)}") from e


def list_adapters() -> list[BaseAdapter]:
    return sorted(_ADAPTERS.values(), key=lambda a: (-a.priority, a.name))
