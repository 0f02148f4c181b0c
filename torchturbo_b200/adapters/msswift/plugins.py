"""`--tt_plugin` dataset plugins inside a swift job.

A `DatasetPlugin` may name datasets (`dataset_names`), build them (`load(name, ctx) -> dataset`), encode rows
(`encode(row, ctx) -> dict`) and bring its own collator.  `DatasetPluginBridge` (a) registers every named dataset with
swift's dataset registry so `--dataset <name>` resolves, and (b) lets a plugin take the whole dataset preparation over
when all requested datasets belong to it: the pipeline then skips swift's own loading / encoding and the trainer uses
the plugin's collator.  Plugins that only wrap a dataset keep working through `engine.create_dataloader`.
(adapters/msswift/plugins.py:17-231 of the reference.)"""
from __future__ import annotations

from typing import Any, Callable

from ...engine.plugins import DatasetPlugin, PluginManager
from ...logging import get_logger

logger = get_logger(__name__)


class DatasetPluginBridge:
    def __init__(self) -> None:
        self.by_name: dict[str, DatasetPlugin] = {}
        self.plugins: list[DatasetPlugin] = []

    def add(self, plugin: DatasetPlugin) -> None:
        self.plugins.append(plugin)
        names = list(getattr(plugin, "dataset_names", []) or [])
        for n in names:
            if n in self.by_name and self.by_name[n] is not plugin:
                raise ValueError(f"dataset name {n!r} is claimed by two plugins")
            self.by_name[n] = plugin
        if names:
            self._register_with_swift(plugin, names)

    def _register_with_swift(self, plugin: DatasetPlugin, names: list[str]) -> None:
        try:
            from swift.dataset import DatasetMeta, register_dataset
        except Exception:  # noqa: BLE001 - swift absent or another layout: names still resolve through try_takeover
            return
        for n in names:
            try:
                register_dataset(DatasetMeta(dataset_name=n, load_function=self._make_loader(plugin, n)), exist_ok=True)
            except Exception:  # noqa: BLE001
                logger.warning_rank0("could not register plugin dataset %s with swift", n)

    @staticmethod
    def _make_loader(plugin: DatasetPlugin, name: str) -> Callable:
        def load(dataset_syntax=None, dataset_meta=None, *args, **kwargs):
            return plugin.load(name, {"syntax": dataset_syntax, "meta": dataset_meta, **kwargs})

        return load

    @staticmethod
    def requested_names(args: Any) -> list[str]:
        out = []
        for entry in list(getattr(args, "dataset", None) or []):
            out.append(str(entry).split("#", 1)[0].split(":", 1)[0])
        return out

    def resolve(self, args: Any) -> DatasetPlugin | None:
        """The plugin that owns *all* requested datasets (None when swift should load them; a mix is an error)."""
        names = self.requested_names(args)
        owners = {self.by_name.get(n) for n in names}
        if owners == {None} or not names:
            return None
        if None in owners or len(owners) > 1:
            raise ValueError(f"datasets {names} mix plugin-provided and native datasets (or two plugins); "
                             "a plugin must provide all datasets of a run")
        return owners.pop()

    def make_ctx(self, args: Any, template: Any, **extra: Any) -> dict[str, Any]:
        return {"args": args, "template": template, "max_length": getattr(args, "max_length", None),
                "seed": getattr(args, "data_seed", None) or getattr(args, "seed", 0), **extra}

    def try_takeover(self, *, args: Any, template: Any, show_dataset: Callable | None = None):
        plugin = self.resolve(args)
        if plugin is None or not hasattr(plugin, "load"):
            return None
        ctx = self.make_ctx(args, template)
        names = self.requested_names(args)
        train = [plugin.load(n, ctx) for n in names]
        train_ds = train[0] if len(train) == 1 else _Concat(train)
        if hasattr(plugin, "encode"):
            train_ds = _Encoded(train_ds, plugin, ctx)
        val_ds = plugin.load_validation(ctx) if hasattr(plugin, "load_validation") else None
        if show_dataset is not None:
            try:
                show_dataset(train_ds, val_ds)
            except Exception:  # noqa: BLE001 - a preview only
                pass
        logger.info_rank0("dataset plugin %s provides %s", type(plugin).__name__, names)
        return [train_ds, val_ds]

    def collator_for(self, args: Any) -> Callable | None:
        plugin = self.resolve(args)
        if plugin is None:
            return None
        if hasattr(plugin, "collate"):
            return plugin.collate
        return getattr(plugin, "collator", None)


class _Concat:
    def __init__(self, parts):
        self.parts = parts
        self.offsets = [0]
        for p in parts:
            self.offsets.append(self.offsets[-1] + len(p))

    def __len__(self):
        return self.offsets[-1]

    def __getitem__(self, i):
        if i < 0:
            i += len(self)
        for k in range(len(self.parts)):
            if i < self.offsets[k + 1]:
                return self.parts[k][i - self.offsets[k]]
        raise IndexError(i)


class _Encoded:
    def __init__(self, inner, plugin, ctx):
        self.inner, self.plugin, self.ctx = inner, plugin, ctx

    def __len__(self):
        return len(self.inner)

    def __getitem__(self, i):
        return self.plugin.encode(self.inner[i], self.ctx)


class SwiftPluginHost:
    """Receives the plugins the engine loaded and routes dataset plugins to the bridge."""

    def __init__(self) -> None:
        self.dataset_bridge = DatasetPluginBridge()

    def install_plugins(self, manager: PluginManager) -> None:
        for p in manager.dataset_plugins():
            self.dataset_bridge.add(p)
