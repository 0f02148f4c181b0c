from .fqn import match_fqn
from .functools import cache

__all__ = ["match_fqn", "cache"]
