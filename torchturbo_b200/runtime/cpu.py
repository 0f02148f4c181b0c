"""CPU runtime (gloo): used by the unit tests, the host-side control plane and the oracle runs."""
from __future__ import annotations

import psutil
import torch

from .base import BaseProfiler, DeviceRuntime, TurboDevice


class _NullProfiler(BaseProfiler):
    def start(self) -> None:
        if self.profiling_enabled or self.memory_snapshot_steps:
            raise NotImplementedError("profiling is only implemented for the CUDA runtime")

    def step(self) -> None:
        pass

    def stop(self) -> None:
        pass


class CpuRuntime(DeviceRuntime):
    turbo_device = TurboDevice.CPU
    dist_backend = "gloo"

    def available(self) -> bool:
        return True

    def current_device(self):
        return torch.device("cpu")

    def set_device(self, device: int) -> None:
        pass

    def synchronize(self) -> None:
        pass

    def memory_info(self) -> tuple[int, int]:
        vm = psutil.virtual_memory()
        return vm.available, vm.total

    def manual_seed_all(self, seed: int) -> None:
        torch.manual_seed(seed)

    def profiler(self, *, output_dir, worker_name, profiling_enabled, memory_snapshot_steps):
        return _NullProfiler(output_dir, worker_name, profiling_enabled, memory_snapshot_steps)
