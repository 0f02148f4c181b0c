from .base import BaseProfiler, DeviceRuntime, TurboDevice
from .cpu import CpuRuntime
from .cuda import CudaRuntime
from .runtime import get_device_runtime, set_device_runtime

__all__ = ["BaseProfiler", "DeviceRuntime", "TurboDevice", "CpuRuntime", "CudaRuntime", "get_device_runtime",
           "set_device_runtime"]
