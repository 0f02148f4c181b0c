"""Process-group bootstrap and cross-rank sanity checks."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from ..runtime import DeviceRuntime, get_device_runtime

DEFAULT_PG_TIMEOUT_S = 1800


def init_process_group_if_needed(runtime: DeviceRuntime | None = None, *, with_cpu_backend: bool = False,
                                 timeout_s: int | None = None) -> None:
    """Initialise the default group from the torchrun environment.  With `with_cpu_backend` the group gets
    a gloo side (`"cuda:nccl,cpu:gloo"`) so CPU tensors (offloaded state, control messages) can be reduced."""
    if dist.is_initialized():
        return
    runtime = runtime or get_device_runtime()
    backend = runtime.dist_backend
    if with_cpu_backend and backend != "gloo":
        backend = f"{runtime.turbo_device.value}:{backend},cpu:gloo"
    if "RANK" not in os.environ:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
    kw = {}
    if runtime.turbo_device.value == "cuda":
        kw["device_id"] = runtime.device
    dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s or DEFAULT_PG_TIMEOUT_S), **kw)


def assert_finite(value: torch.Tensor, what: str = "loss", group=None) -> None:
    """Raise on every rank if `value` is non-finite on any rank (one MIN all-reduce of an int flag)."""
    ok = torch.isfinite(value.detach()).all().to(torch.int32).reshape(1)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 0:
        raise FloatingPointError(f"{what} is not finite on at least one rank")


def get_rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1
