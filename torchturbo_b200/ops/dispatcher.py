"""Chooses one implementation per operator and exposes them as `ops.<name>(...)`.

Selection = (device of the runtime) x (global policy) x (per-op override):
  * `auto`   - best ranked implementation that reports itself available;
  * `native` - torch formulations only;
  * `custom` - a hand-written kernel is required; raises when none is available;
  * an implementation name pins that implementation.
Availability is probed lazily, once per implementation.  `log_ops_selection()` prints the table the
engine logs at start-up.  Same role as ops/dispatcher.py:30-660 in the reference.
"""
from __future__ import annotations

import importlib
from typing import Any

from ..logging import get_logger
from ..runtime import DeviceRuntime, get_device_runtime
from .base import OpImpl, OpImplKind, OpPolicy
from .registry import REGISTRY

logger = get_logger(__name__)

_PROVIDER_MODULES = ("torchturbo_b200.ops.providers.native", "torchturbo_b200.ops.providers.native_linear_attention",
                     "torchturbo_b200.ops.providers.native_sparse_attention",
                     "torchturbo_b200.ops.providers.b200", "torchturbo_b200.ops.providers.b200_linear_attention")


def load_providers() -> None:
    for m in _PROVIDER_MODULES:
        importlib.import_module(m)
    try:
        importlib.import_module("torchturbo_b200.ops.providers.b200_attention")
    except ModuleNotFoundError:
        pass


class OpDispatcher:
    def __init__(self, policy: OpPolicy | str = OpPolicy.AUTO, overrides: dict[str, str] | None = None,
                 runtime: DeviceRuntime | None = None) -> None:
        load_providers()
        self._runtime = runtime or get_device_runtime()
        self._policy = OpPolicy(policy)
        self._overrides = dict(overrides or {})
        for op, choice in self._overrides.items():
            if op not in REGISTRY.ops():
                raise KeyError(f"override for unknown op {op!r}")
            if choice not in {p.value for p in OpPolicy}:
                REGISTRY.get(op, choice)  # raises for unknown names
        self._instances: dict[tuple[str, str], OpImpl] = {}
        self._selected: dict[str, OpImpl] = {}

    # -- introspection -------------------------------------------------------------------------
    @property
    def device_runtime(self) -> DeviceRuntime:
        return self._runtime

    @property
    def default_policy(self) -> OpPolicy:
        return self._policy

    @property
    def overrides(self) -> dict[str, str]:
        return dict(self._overrides)

    # -- selection -----------------------------------------------------------------------------
    def _instance(self, cls: type[OpImpl]) -> OpImpl:
        s = cls.op_spec()
        key = (s.op_name, s.impl_name)
        if key not in self._instances:
            self._instances[key] = cls()
        return self._instances[key]

    def _select(self, op_name: str, impl: str | None = None) -> OpImpl:
        if op_name not in REGISTRY.ops():
            raise AttributeError(f"unknown op {op_name!r}")
        choice = impl or self._overrides.get(op_name) or self._policy.value
        device = self._runtime.turbo_device
        if choice not in {p.value for p in OpPolicy}:
            inst = self._instance(REGISTRY.get(op_name, choice))
            if not inst.available():
                raise RuntimeError(f"implementation {choice!r} of op {op_name!r} is not available here")
            return inst
        policy = OpPolicy(choice)
        for cls in REGISTRY.list(op_name, device):
            kind = cls.op_spec().kind
            if policy is OpPolicy.NATIVE and kind is not OpImplKind.NATIVE:
                continue
            if policy is OpPolicy.CUSTOM and kind is not OpImplKind.CUSTOM:
                continue
            inst = self._instance(cls)
            if inst.available():
                return inst
        raise RuntimeError(f"no {policy.value} implementation of op {op_name!r} is available on {device.value}")

    def resolve(self, op_name: str) -> OpImpl:
        if op_name not in self._selected:
            self._selected[op_name] = self._select(op_name)
        return self._selected[op_name]

    def selection_table(self) -> list[tuple[str, str, str]]:
        rows = []
        for op in REGISTRY.ops():
            try:
                s = self.resolve(op).op_spec()
                rows.append((op, s.impl_name, s.kind.value))
            except RuntimeError as e:
                rows.append((op, "<unavailable>", str(e)))
        return rows

    def log_ops_selection(self) -> None:
        rows = self.selection_table()
        w = max(len(r[0]) for r in rows)
        lines = [f"ops selection (policy={self._policy.value}, device={self._runtime.turbo_device.value}):"]
        lines += [f"  {op:<{w}}  {impl}  [{kind}]" for op, impl, kind in rows]
        logger.info_rank0("\n".join(lines))

    # -- call ----------------------------------------------------------------------------------
    def _dispatch(self, op_name: str, *args: Any, impl: str | None = None, **kwargs: Any):
        inst = self._select(op_name, impl) if impl is not None else self.resolve(op_name)
        return inst(*args, **kwargs)

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        if name not in REGISTRY.ops():
            raise AttributeError(f"unknown op {name!r}")

        def facade(*args: Any, impl: str | None = None, **kwargs: Any):
            return self._dispatch(name, *args, impl=impl, **kwargs)

        facade.__name__ = name
        self.__dict__[name] = facade   # later `ops.<name>` lookups skip __getattr__ (selection still happens per call)
        return facade
