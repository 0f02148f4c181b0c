from __future__ import annotations

from .base import DeviceRuntime
from .cpu import CpuRuntime
from .cuda import CudaRuntime

_SELECTED_RUNTIME: DeviceRuntime | None = None


def set_device_runtime(runtime: DeviceRuntime | None) -> None:
    """Force a runtime (tests inject `CpuRuntime()`); `None` returns to auto-detection."""
    global _SELECTED_RUNTIME
    _SELECTED_RUNTIME = runtime


def get_device_runtime() -> DeviceRuntime:
    """CUDA when a GPU is visible, else CPU.  The choice is cached for the process."""
    global _SELECTED_RUNTIME
    if _SELECTED_RUNTIME is None:
        rt: DeviceRuntime = CudaRuntime()
        if not rt.available():
            rt = CpuRuntime()
        rt.initialize()
        _SELECTED_RUNTIME = rt
    return _SELECTED_RUNTIME
