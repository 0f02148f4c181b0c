"""CUDA (B200) runtime: NCCL backend, streams/events, memory figures, torch.profiler + memory snapshots
and NVTX ranges around the fused paths (the reference's profiler has no NVTX: runtime/cuda.py:11-70)."""
from __future__ import annotations

import contextlib
import os

import torch

from .base import BaseProfiler, DeviceRuntime, TurboDevice


class CudaProfiler(BaseProfiler):
    """torch.profiler trace (wait 0 / warmup 10 / active 1, first step skipped) written as a TensorBoard
    trace under `<out>/profiling`, plus an allocator-history snapshot dumped at a chosen step under
    `<out>/memory_snapshot/<worker>.pickle`."""

    def __init__(self, output_dir, worker_name, profiling_enabled, memory_snapshot_steps):
        super().__init__(output_dir, worker_name, profiling_enabled, memory_snapshot_steps)
        self._prof = None
        self._step = 0
        self._recording_memory = False

    def start(self) -> None:
        if self.profiling_enabled:
            from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler

            self._prof = profile(
                activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                schedule=schedule(wait=0, warmup=10, active=1, repeat=1, skip_first=1),
                on_trace_ready=tensorboard_trace_handler(os.path.join(self.output_dir, "profiling"),
                                                         worker_name=self.worker_name),
                record_shapes=True, with_stack=False,
            )
            self._prof.start()
        if self.memory_snapshot_steps:
            torch.cuda.memory._record_memory_history(max_entries=200000)
            self._recording_memory = True

    def step(self) -> None:
        self._step += 1
        if self._prof is not None:
            self._prof.step()
        if self._recording_memory and self._step == self.memory_snapshot_steps:
            d = os.path.join(self.output_dir, "memory_snapshot")
            os.makedirs(d, exist_ok=True)
            torch.cuda.memory._dump_snapshot(os.path.join(d, f"{self.worker_name}.pickle"))
            torch.cuda.memory._record_memory_history(enabled=None)
            self._recording_memory = False

    def stop(self) -> None:
        if self._prof is not None:
            self._prof.stop()
            self._prof = None
        if self._recording_memory:
            torch.cuda.memory._record_memory_history(enabled=None)
            self._recording_memory = False


class CudaRuntime(DeviceRuntime):
    turbo_device = TurboDevice.CUDA
    dist_backend = "nccl"

    @property
    def supports_async_streams(self) -> bool:
        return True

    def available(self) -> bool:
        return torch.cuda.is_available()

    def initialize(self) -> None:
        """Bind the process to its GPU.  Under a launcher `LOCAL_RANK` names it.  Without that variable the
        process keeps whatever device it already selected: the runtime is created lazily (first op dispatch), and
        switching devices then would launch kernels on one GPU with pointers of another."""
        local = os.environ.get("LOCAL_RANK")
        if local is None or torch.cuda.device_count() == 0:
            return
        want = int(local) % torch.cuda.device_count()
        if torch.cuda.is_initialized() and torch.cuda.current_device() != want:
            # the application chose another device explicitly before the first op; respect it
            return
        torch.cuda.set_device(want)

    def use_deterministic_algorithms(self) -> None:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        torch.use_deterministic_algorithms(True)
        torch.backends.cudnn.benchmark = False

    @property
    def device(self) -> torch.device:
        return torch.device("cuda", torch.cuda.current_device())

    def current_device(self):
        return torch.cuda.current_device()

    def set_device(self, device: int) -> None:
        torch.cuda.set_device(device)

    def synchronize(self) -> None:
        torch.cuda.synchronize()

    def empty_cache(self) -> None:
        torch.cuda.empty_cache()

    def memory_info(self) -> tuple[int, int]:
        return torch.cuda.mem_get_info()

    def memory_reserved(self) -> int:
        return torch.cuda.memory_reserved()

    def memory_allocated(self) -> int:
        return torch.cuda.memory_allocated()

    def stream(self, stream=None):
        return torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext()

    def current_stream(self):
        return torch.cuda.current_stream()

    def new_stream(self, priority: int = 0):
        return torch.cuda.Stream(priority=priority)

    def new_event(self):
        return torch.cuda.Event()

    def manual_seed_all(self, seed: int) -> None:
        torch.manual_seed(seed)
        torch.cuda.manual_seed_all(seed)

    def profiler(self, *, output_dir, worker_name, profiling_enabled, memory_snapshot_steps):
        return CudaProfiler(output_dir, worker_name, profiling_enabled, memory_snapshot_steps)

    @staticmethod
    @contextlib.contextmanager
    def nvtx(name: str):
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
