"""Fully-qualified-name pattern matching shared by plans, freeze policies and optimizer recipes."""
from __future__ import annotations

import re
from functools import lru_cache


@lru_cache(maxsize=4096)
def _compile(pattern: str) -> re.Pattern:
    out = []
    i = 0
    while i < len(pattern):
        if pattern.startswith("**", i):
            out.append(".*")
            i += 2
        elif pattern[i] == "*":
            out.append("[^.]+")
            i += 1
        else:
            out.append(re.escape(pattern[i]))
            i += 1
    return re.compile("^" + "".join(out) + "$")


def match_fqn(pattern: str, fqn: str) -> bool:
    """Whole-string match where ``*`` stays inside one dotted segment and ``**`` may span segments.

    Same semantics as the reference helper (engine/utils.py:28-49): ``layers.*.weight`` matches
    ``layers.0.weight`` but not ``layers.0.attn.weight``; ``layers.**.weight`` matches both.
    """
    return _compile(pattern).match(fqn) is not None
