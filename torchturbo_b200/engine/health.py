"""Failure detection for multi-GPU runs: host-side heartbeats and the status words of the peer-memory kernels.

Two facts shape this module.  (1) A kernel that waits on a peer flag gives up after a time budget, records
`{site, peer}` in its workspace's status word and stops touching remote memory, so the GPU keeps answering; but
the result of that step is garbage and must become a Python exception.  (2) A collective (NCCL, or one of the
peer-memory kernels) that a dead rank never joins only ends by its timeout, so the surviving ranks should learn
about the death on the host *before* their next launch.

`Heartbeat` publishes `(step, wall time)` of this rank in the process group's key-value store at step boundaries
(or from a host thread) and reports peers whose last beat is older than `max_age` seconds.
`check_peer_status()` reads every status word (one small device-to-host copy each; call it at logging / checkpoint
boundaries, not per layer) and raises on *every* rank if any rank saw a timeout or overflow, using the same
all-gather-of-messages fan-out as the checkpoint steps.

The reference has no heartbeat or elastic recovery (its failure handling is the process-group timeout,
engine/distributed.py:17,84-87, plus the error fan-out helpers of engine/checkpoint/distributed.py:13-48); recovery
here is the same: restart and resume from the last committed checkpoint.
"""
from __future__ import annotations

import threading
import time
from typing import Any, Iterable

import torch.distributed as dist

from .checkpoint.distributed import RemoteRankError, collective_check


class RankFailure(RuntimeError):
    """Raised on a healthy rank when a peer stopped beating."""


class Heartbeat:
    def __init__(self, store=None, *, rank: int | None = None, world_size: int | None = None, prefix: str = "tt_hb",
                 max_age: float = 60.0, clock=time.time):
        if store is None:
            from torch.distributed.distributed_c10d import _get_default_store

            store = _get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.prefix, self.max_age, self.clock = prefix, float(max_age), clock
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()
        self.step = 0

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int | None = None) -> None:
        if step is not None:
            self.step = step
        self.store.set(self._key(self.rank), f"{self.step}:{self.clock():.3f}")

    def last(self, r: int) -> tuple[int, float] | None:
        """(step, wall time) of rank r's last beat, or None if it never beat."""
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            s, t = self.store.get(self._key(r)).decode().split(":")
            return int(s), float(t)
        except Exception:  # noqa: BLE001 - a store that cannot answer counts as "no beat"
            return None

    def stale_ranks(self) -> list[int]:
        now = self.clock()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            b = self.last(r)
            if b is None or now - b[1] > self.max_age:
                out.append(r)
        return out

    def check(self) -> None:
        """Beat, then raise `RankFailure` if a peer is stale.  Call between steps, before the next launch."""
        self.beat()
        stale = self.stale_ranks()
        if stale:
            raise RankFailure(f"rank {self.rank}: no heartbeat from rank(s) {stale} for more than {self.max_age:.0f}s; "
                              "stop launching collectives and restart from the last committed checkpoint")

    # -- background beating (for long steps) -----------------------------------------------------------
    def start(self, interval: float = 5.0) -> None:
        if self._thread is not None:
            return
        self._stop.clear()

        def run():
            while not self._stop.wait(interval):
                try:
                    self.beat()
                except Exception:  # noqa: BLE001 - the store is gone: the job is ending
                    return

        self._thread = threading.Thread(target=run, name="tt-heartbeat", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None


def peer_workspaces(backend: Any = None) -> list[Any]:
    """Every live peer-memory workspace of this process (expert-parallel, Ulysses, row exchange, FSDP arenas)."""
    from ..comm import ep_p2p, rows_p2p, ulysses_p2p

    out: list[Any] = list(ep_p2p._WORKSPACES.values()) + list(ulysses_p2p._WORKSPACES.values()) + list(rows_p2p._WS.values())
    try:
        from ..comm import fsdp_p2p

        out += list(fsdp_p2p._ARENAS.values())
    except Exception:  # noqa: BLE001 - torch build without the custom-collective hook
        pass
    if backend is not None:
        out += [a for a in getattr(backend, "peer_arenas", []) if a not in out]
    return out


def check_peer_status(workspaces: Iterable[Any] | None = None, *, what: str = "peer-memory exchange") -> None:
    """Raise on every rank if any rank's peer-memory kernels recorded a timeout / overflow since the last check."""

    from ..comm.ep_p2p import CAPACITY_MARK, EPCapacityExceeded

    def local():
        for ws in (peer_workspaces() if workspaces is None else workspaces):
            ws.check()

    try:
        collective_check(local, what)
    except RemoteRankError as e:
        # the same class on every rank: the caller's recovery (grow the buffers, repeat the step) is collective
        if CAPACITY_MARK in str(e):
            raise EPCapacityExceeded(str(e)) from None
        raise


def reset_peer_status(backend: Any = None) -> None:
    """Clear every status word (workspaces, arenas and the per-unit words of the kernels) after a handled failure."""
    import torch

    from .. import kernels as K

    for ws in peer_workspaces(backend):
        st = getattr(ws, "status", None)
        if isinstance(st, torch.Tensor):
            st.zero_()
    if K.available():
        K.status(reset=True)
        K.comm_status(reset=True)


__all__ = ["Heartbeat", "RankFailure", "RemoteRankError", "check_peer_status", "peer_workspaces", "reset_peer_status"]
