"""Version probing for ms-swift (the 4.x pipeline layout `swift.pipelines.train.*` is the supported one).
adapters/msswift/compat.py:9-37 of the reference."""
from __future__ import annotations

import importlib.util
import sys
from importlib import metadata

SUPPORTED = ">=4.0,<5"


def _has_module(name: str) -> bool:
    if name in sys.modules:
        return True
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError, AttributeError):
        return False


def is_swift_installed() -> bool:
    return _has_module("swift")


def get_swift_version() -> str:
    for dist_name in ("ms-swift", "ms_swift", "swift"):
        try:
            return metadata.version(dist_name)
        except metadata.PackageNotFoundError:
            continue
    mod = sys.modules.get("swift")
    return str(getattr(mod, "__version__", "")) if mod is not None else ""


def is_swift_supported() -> bool:
    if not is_swift_installed():
        return False
    from packaging.specifiers import SpecifierSet
    from packaging.version import InvalidVersion, Version

    try:
        return Version(get_swift_version()) in SpecifierSet(SUPPORTED, prereleases=True)
    except InvalidVersion:
        return _has_module("swift.pipelines.train")
