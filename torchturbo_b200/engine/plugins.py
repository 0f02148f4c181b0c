"""User extension points loaded from `--tt_plugin path[:config]`.

A plugin file defines one or more `Plugin` subclasses decorated with `@register_plugin`.  Two built-in
flavours exist: `DatasetPlugin` (wrap or replace the training dataset) and `CheckpointExportPlugin` (called on
rank 0 after a Hugging Face export finished).  (engine/plugins.py:18-179 of the reference)"""
from __future__ import annotations

import importlib.util
import os
from typing import Any

_REGISTERED: list[type] = []


class Plugin:
    name: str = "plugin"

    def __init__(self, config: str | None = None) -> None:
        self.config = config

    def setup(self, engine: Any) -> None:
        pass


class CheckpointExportPlugin(Plugin):
    def on_hf_export(self, export_dir: str, *, step: int | None = None, final: bool = False) -> None:
        pass


class DatasetPlugin(Plugin):
    def wrap_dataset(self, dataset):
        return dataset


def register_plugin(cls: type) -> type:
    if not issubclass(cls, Plugin):
        raise TypeError("plugins must subclass Plugin")
    if cls not in _REGISTERED:
        _REGISTERED.append(cls)
    return cls


class PluginManager:
    def __init__(self, paths: list[str] | None = None) -> None:
        self.plugins: list[Plugin] = []
        for spec in paths or []:
            self.load(spec)

    def load(self, spec: str) -> None:
        path, _, cfg = spec.partition(":")
        if not os.path.isfile(path):
            raise FileNotFoundError(f"plugin file not found: {path}")
        before = len(_REGISTERED)
        mod_spec = importlib.util.spec_from_file_location(f"tt_plugin_{len(self.plugins)}_{abs(hash(path))}", path)
        module = importlib.util.module_from_spec(mod_spec)
        mod_spec.loader.exec_module(module)
        new = _REGISTERED[before:]
        if not new:
            new = [v for v in vars(module).values() if isinstance(v, type) and issubclass(v, Plugin)
                   and v.__module__ == module.__name__]
        if not new:
            raise ValueError(f"{path} defines no Plugin subclass")
        for cls in new:
            self.plugins.append(cls(cfg or None))

    def setup(self, engine: Any) -> None:
        for p in self.plugins:
            p.setup(engine)

    def dataset_plugins(self) -> list[DatasetPlugin]:
        return [p for p in self.plugins if isinstance(p, DatasetPlugin)]

    def export_plugins(self) -> list[CheckpointExportPlugin]:
        return [p for p in self.plugins if isinstance(p, CheckpointExportPlugin)]
