"""Operator metadata: what an implementation provides, on which devices, and how it ranks."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from enum import Enum
from typing import Any, ClassVar

from ..runtime import TurboDevice


class OpPolicy(str, Enum):
    """`auto`: best available implementation; `native`: torch formulations only; `custom`: require a kernel."""

    AUTO = "auto"
    NATIVE = "native"
    CUSTOM = "custom"


class OpImplKind(str, Enum):
    NATIVE = "native"
    CUSTOM = "custom"


_RESERVED = {p.value for p in OpPolicy}


@dataclass(frozen=True)
class OpSpec:
    op_name: str
    impl_name: str
    kind: OpImplKind = OpImplKind.NATIVE
    priority: int = 0
    devices: tuple[TurboDevice, ...] = ()

    def __post_init__(self) -> None:
        if not self.op_name or not self.impl_name:
            raise ValueError("OpSpec needs both op_name and impl_name")
        if self.impl_name in _RESERVED:
            raise ValueError(f"impl_name {self.impl_name!r} collides with a policy name")
        if not isinstance(self.kind, OpImplKind):
            raise TypeError("OpSpec.kind must be an OpImplKind")
        object.__setattr__(self, "priority", int(self.priority))
        object.__setattr__(self, "devices", tuple(TurboDevice(d) for d in self.devices))

    def supports(self, device: TurboDevice) -> bool:
        return not self.devices or device in self.devices


class OpImpl(ABC):
    """One implementation of one operator.  Instances are created lazily by the dispatcher."""

    __op_spec__: ClassVar[OpSpec | None] = None

    @classmethod
    def op_spec(cls) -> OpSpec:
        if cls.__op_spec__ is None:
            raise RuntimeError(f"{cls.__name__} was not registered with @register_op")
        return cls.__op_spec__

    def available(self) -> bool:
        return True

    @abstractmethod
    def __call__(self, *args: Any, **kwargs: Any): ...
