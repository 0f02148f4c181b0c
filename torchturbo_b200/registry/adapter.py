"""Framework adapters: a named bundle of version-gated patches that lets a host training framework drive the engine
(registry/adapter.py:41-120 of the reference)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from importlib import metadata

from packaging.specifiers import InvalidSpecifier, SpecifierSet
from packaging.version import InvalidVersion, Version

from ..logging import get_logger
from .patch import BasePatch

logger = get_logger(__name__)


def _version_matches(installed: str | None, spec: str | None) -> bool:
    if spec is None:
        return True
    if installed is None:
        return False
    try:
        return Version(installed) in SpecifierSet(spec, prereleases=True)
    except (InvalidVersion, InvalidSpecifier):
        return False


class BaseAdapter(ABC):
    name: str = "adapter"
    priority: int = 0
    package: str | None = None  # distribution name of the host framework

    def __init__(self) -> None:
        self.patches: list[BasePatch] = []
        self.active = False

    @abstractmethod
    def detect(self) -> bool:
        """Is the host framework importable (and is this process being run by it)?"""

    def framework_version(self) -> str | None:
        if self.package is None:
            return None
        try:
            return metadata.version(self.package)
        except metadata.PackageNotFoundError:
            return None

    def add_patch(self, patch: BasePatch) -> None:
        self.patches.append(patch)

    def apply_patches(self, engine=None) -> list[str]:
        v = self.framework_version()
        done = []
        for p in self.patches:
            if _version_matches(v, p.version_spec):
                p.patch(engine)
                done.append(p.name)
            else:
                logger.warning_rank0("patch %s skipped: %s %s does not satisfy %s", p.name, self.package, v, p.version_spec)
        return done

    def revert_patches(self) -> None:
        for p in reversed(self.patches):
            p.revert()

    def activate(self) -> None:
        self.active = True

    def deactivate(self) -> None:
        self.revert_patches()
        self.active = False
