"""Finds out which host training framework (if any) is driving this process."""
from __future__ import annotations

from .registry import list_adapters


class FrameworkDetector:
    def detect_all(self) -> list[str]:
        found = []
        for a in list_adapters():
            try:
                if a.detect():
                    found.append(a.name)
            except Exception:
                continue
        return found

    def detect(self) -> str | None:
        """Highest-priority adapter whose framework is present, or None."""
        found = self.detect_all()
        return found[0] if found else None
