"""Process-wide marker for "this forward pass is an activation-checkpoint replay".

Modules that keep statistics across a step (router token counts for the expert-bias update, reported auxiliary
losses) consult `in_recompute()` so that the replay of a checkpointed segment during backward does not count a
micro-batch twice; the backend enters `recompute_ctx()` around every replay, in both checkpoint modes.  The reference
carries the same information through `MoERuntimeInputs.accumulate_tokens_per_expert`
(engine/backends/fsdp2/activation_checkpointing.py:25-49, models/modules/moe/router.py:336-354 of the reference)."""
from __future__ import annotations

import contextlib

_STATE = {"active": False}


def in_recompute() -> bool:
    return _STATE["active"]


@contextlib.contextmanager
def recompute_ctx():
    prev = _STATE["active"]
    _STATE["active"] = True
    try:
        yield
    finally:
        _STATE["active"] = prev
