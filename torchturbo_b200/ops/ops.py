"""Process-wide operator facade: `from torchturbo_b200.ops import ops; ops.rms_norm(x, w)`."""
from __future__ import annotations

from .base import OpPolicy
from .dispatcher import OpDispatcher

_DISPATCHER: OpDispatcher | None = None


def get_or_create_ops(policy: OpPolicy | str | None = None, overrides: dict[str, str] | None = None,
                      runtime=None, *, reset: bool = False) -> OpDispatcher:
    """Returns the process singleton, (re)building it when a policy/override set is given explicitly."""
    global _DISPATCHER
    if _DISPATCHER is None or reset or policy is not None or overrides is not None or runtime is not None:
        _DISPATCHER = OpDispatcher(policy or OpPolicy.AUTO, overrides, runtime)
    return _DISPATCHER


class _OpsProxy:
    def __getattr__(self, name: str):
        return getattr(get_or_create_ops(), name)


ops = _OpsProxy()
