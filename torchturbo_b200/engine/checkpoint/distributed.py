"""Error fan-out for collective checkpoint steps: one rank's exception is raised on every rank *before* the
next collective, so nobody waits in a collective that the failing rank will never join
(engine/checkpoint/distributed.py:13-48 of the reference)."""
from __future__ import annotations

from typing import Any, Callable

import torch.distributed as dist


class RemoteRankError(RuntimeError):
    pass


def _active() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def collective_check(fn: Callable[[], Any], what: str = "step") -> Any:
    """Run `fn` on every rank; if any rank raised, all ranks raise."""
    err, result = None, None
    try:
        result = fn()
    except Exception as e:  # noqa: BLE001 - reported to every rank below
        err = e
    if _active():
        msgs: list[Any] = [None] * dist.get_world_size()
        dist.all_gather_object(msgs, None if err is None else f"{type(err).__name__}: {err}")
        bad = [(r, m) for r, m in enumerate(msgs) if m is not None]
        if bad and err is None:
            raise RemoteRankError(f"{what} failed on rank {bad[0][0]}: {bad[0][1]}")
    if err is not None:
        raise err
    return result


def rank_zero_call(fn: Callable[[], Any], what: str = "step") -> Any:
    """Run `fn` on rank 0 only; its result (or failure) is broadcast to every rank."""
    if not _active():
        return fn()
    payload: list[Any] = [None, None]
    if dist.get_rank() == 0:
        try:
            payload[0] = fn()
        except Exception as e:  # noqa: BLE001
            payload[1] = f"{type(e).__name__}: {e}"
    dist.broadcast_object_list(payload, src=0)
    if payload[1] is not None:
        raise RemoteRankError(f"{what} failed on rank 0: {payload[1]}")
    return payload[0]
