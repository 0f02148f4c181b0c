"""Process-wide table of operator implementations."""
from __future__ import annotations

from collections import defaultdict

from ..runtime import TurboDevice
from .base import OpImpl, OpImplKind, OpSpec


class OpRegistry:
    def __init__(self) -> None:
        self._impls: dict[str, dict[str, type[OpImpl]]] = defaultdict(dict)

    def register(self, cls: type[OpImpl]) -> None:
        spec = cls.op_spec()
        table = self._impls[spec.op_name]
        if spec.impl_name in table and table[spec.impl_name] is not cls:
            raise ValueError(f"duplicate implementation {spec.impl_name!r} for op {spec.op_name!r}")
        table[spec.impl_name] = cls

    def ops(self) -> list[str]:
        return sorted(self._impls)

    def get(self, op_name: str, impl_name: str) -> type[OpImpl]:
        try:
            return self._impls[op_name][impl_name]
        except KeyError as e:
            raise KeyError(f"op {op_name!r} has no implementation {impl_name!r}") from e

    def list(self, op_name: str, device: TurboDevice | None = None) -> list[type[OpImpl]]:
        """Implementations ranked best first: higher priority, then device-specific over generic, then
        custom kernels over native formulations, then name (ops/registry.py:35-53 in the reference)."""
        cands = [c for c in self._impls.get(op_name, {}).values() if device is None or c.op_spec().supports(device)]

        def key(c):
            s = c.op_spec()
            return (-s.priority, 0 if s.devices else 1, 0 if s.kind is OpImplKind.CUSTOM else 1, s.impl_name)

        return sorted(cands, key=key)


REGISTRY = OpRegistry()


def register_op(*, op_name: str, impl_name: str, kind: OpImplKind = OpImplKind.NATIVE, priority: int = 0,
                devices: tuple = ()):
    def deco(cls: type[OpImpl]) -> type[OpImpl]:
        cls.__op_spec__ = OpSpec(op_name, impl_name, kind, priority, tuple(devices))
        REGISTRY.register(cls)
        return cls

    return deco
