"""Failure detection without a GPU fault: every failure is made on the host (a rank that raises, stops beating,
or never joins a collective) and the healthy ranks must learn of it as a Python exception."""
import datetime
import os
import time

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed


def _w_fanout(rank, world):
    from torchturbo_b200.engine.checkpoint import RemoteRankError, collective_check, rank_zero_call

    # one rank fails: the failing rank sees its own error, every other rank a RemoteRankError naming it
    def step():
        if rank == 1:
            raise ValueError("disk full")
        return rank

    try:
        collective_check(step, "save")
        raise AssertionError("must raise")
    except ValueError:
        assert rank == 1
    except RemoteRankError as e:
        assert rank != 1 and "rank 1" in str(e) and "disk full" in str(e)
    # everybody is still in step with everybody else: a collective right after the failure works
    t = torch.ones(1)
    dist.all_reduce(t)
    assert t.item() == world
    assert collective_check(lambda: 7, "ok") == 7
    # rank-0-only work: result and failure reach all ranks
    assert rank_zero_call(lambda: {"n": 3}, "prepare")["n"] == 3
    with pytest.raises(RemoteRankError, match="rank 0"):
        rank_zero_call(lambda: (_ for _ in ()).throw(OSError("read-only file system")), "prepare")


def test_error_fan_out_reaches_every_rank():
    run_distributed(_w_fanout, 3)


def _w_heartbeat(rank, world):
    from torchturbo_b200.engine.health import Heartbeat, RankFailure

    hb = Heartbeat(max_age=6.0)            # generous: the test machine may be busy
    dist.barrier()          # the first collective also sets up the connections: keep it out of the timed part
    hb.beat(step=0)
    dist.barrier()
    assert hb.stale_ranks() == [] and hb.last((rank + 1) % world)[0] == 0
    if rank == 1:
        # this rank "dies" between steps: no kernel or collective of it is in flight, it just stops beating
        time.sleep(15.0)
        return
    for step in range(1, 3):
        hb.check()          # healthy while everybody's beat is fresh
        hb.beat(step)
        time.sleep(0.2)
    time.sleep(7.5)
    with pytest.raises(RankFailure, match=r"rank\(s\) \[1\]"):
        hb.check()          # learned on the host, before the next launch
    # background beating keeps a slow-but-alive rank fresh
    hb2 = Heartbeat(prefix="bg", max_age=3.0)
    hb2.start(interval=0.1)
    time.sleep(1.0)
    assert hb2.last(rank) is not None and time.time() - hb2.last(rank)[1] < 2.5
    hb2.stop()


def test_heartbeat_reports_a_rank_that_stopped_between_steps():
    run_distributed(_w_heartbeat, 2)


def test_heartbeat_with_a_fake_clock_and_store():
    from torchturbo_b200.engine.health import Heartbeat

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

        def check(self, ks):
            return all(k in self for k in ks)

    now = [100.0]
    st = Store()
    a = Heartbeat(st, rank=0, world_size=3, max_age=10.0, clock=lambda: now[0])
    b = Heartbeat(st, rank=1, world_size=3, max_age=10.0, clock=lambda: now[0])
    a.beat(5); b.beat(5)
    assert a.stale_ranks() == [2]            # rank 2 never beat
    now[0] = 105.0
    b.beat(6)
    now[0] = 112.0
    assert b.stale_ranks() == [0, 2] and a.last(1) == (6, 105.0)


def _w_missing_rank(rank, world, init_file):
    # a second, short-timeout group: the collective of the rank that shows up must end with an error, not hang
    g = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=2))
    if rank == 1:
        time.sleep(4.0)      # never joins the collective below
        return
    t0 = time.time()
    with pytest.raises(RuntimeError):
        dist.all_reduce(torch.ones(1), group=g)
    assert time.time() - t0 < 30.0


def test_short_group_timeout_ends_a_collective_nobody_joins(tmp_path):
    run_distributed(_w_missing_rank, 2, str(tmp_path / "x"))


def test_peer_status_check_raises_from_a_fake_workspace():
    from torchturbo_b200.engine.health import check_peer_status

    class WS:
        def __init__(self, code):
            self.code = code

        def check(self):
            if self.code:
                raise RuntimeError(f"peer wait timed out (code {self.code:#x})")

    check_peer_status([WS(0), WS(0)])
    with pytest.raises(RuntimeError, match="0x10203"):
        check_peer_status([WS(0), WS(0x10203)])
