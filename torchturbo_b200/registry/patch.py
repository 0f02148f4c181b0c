from __future__ import annotations

from abc import ABC, abstractmethod


class BasePatch(ABC):
    """One reversible monkey patch of a host framework.  `patch()` installs it, `revert()` restores the original."""

    name: str = "patch"
    version_spec: str | None = None  # PEP 440 specifier of the host-framework versions this patch targets

    def __init__(self) -> None:
        self.applied = False

    @abstractmethod
    def _patch(self, engine=None) -> None: ...

    @abstractmethod
    def _revert(self) -> None: ...

    def patch(self, engine=None) -> None:
        if not self.applied:
            self._patch(engine)
            self.applied = True

    def revert(self) -> None:
        if self.applied:
            self._revert()
            self.applied = False
