"""Device runtime abstraction: one object answers "which device, which collective backend, how do I
get a stream / event / memory figure / profiler" so the rest of the engine never branches on device type.

The reference has CUDA, NPU and CPU runtimes (runtime/base.py:41-138).  This build targets B200 only,
so there is a CUDA runtime (NCCL) and a CPU runtime (gloo) that serves tests and host-side logic.
"""
from __future__ import annotations

import contextlib
from abc import ABC, abstractmethod
from enum import Enum

import torch


class TurboDevice(str, Enum):
    CUDA = "cuda"
    CPU = "cpu"


class BaseProfiler(ABC):
    """start() / step() / stop() life cycle driven by the training loop."""

    def __init__(self, output_dir: str, worker_name: str, profiling_enabled: bool,
                 memory_snapshot_steps: int | None) -> None:
        self.output_dir = output_dir
        self.worker_name = worker_name
        self.profiling_enabled = profiling_enabled
        self.memory_snapshot_steps = memory_snapshot_steps

    @abstractmethod
    def start(self) -> None: ...

    @abstractmethod
    def step(self) -> None: ...

    @abstractmethod
    def stop(self) -> None: ...


class DeviceRuntime(ABC):
    turbo_device: TurboDevice
    dist_backend: str

    @property
    def device(self) -> torch.device:
        return torch.device(self.turbo_device.value)

    @property
    def supports_async_streams(self) -> bool:
        return False

    @abstractmethod
    def available(self) -> bool: ...

    def initialize(self) -> None:
        pass

    def use_deterministic_algorithms(self) -> None:
        torch.use_deterministic_algorithms(True)

    @abstractmethod
    def current_device(self): ...

    @abstractmethod
    def set_device(self, device: int) -> None: ...

    @abstractmethod
    def synchronize(self) -> None: ...

    def empty_cache(self) -> None:
        pass

    @abstractmethod
    def memory_info(self) -> tuple[int, int]:
        """(free bytes, total bytes)"""

    def memory_reserved(self) -> int:
        return 0

    def memory_allocated(self) -> int:
        return 0

    def stream(self, stream=None):
        return contextlib.nullcontext()

    def current_stream(self):
        return None

    def new_stream(self, priority: int = 0):
        return None

    def new_event(self):
        return None

    def record_stream(self, tensor: torch.Tensor, stream) -> None:
        if stream is not None and tensor.is_cuda:
            tensor.record_stream(stream)

    def synchronize_stream(self, stream) -> None:
        if stream is not None:
            stream.synchronize()

    @abstractmethod
    def manual_seed_all(self, seed: int) -> None: ...

    @abstractmethod
    def profiler(self, *, output_dir: str, worker_name: str, profiling_enabled: bool,
                 memory_snapshot_steps: int | None) -> BaseProfiler: ...
