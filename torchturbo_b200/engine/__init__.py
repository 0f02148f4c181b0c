from .args import TorchTurboArgs, parse_torchturbo_args
from .config import EngineConfig, build_from_args
from .core import DPBlockDistributedSampler, EpochDrivenDataLoader, TorchTurboEngine

__all__ = ["TorchTurboArgs", "parse_torchturbo_args", "EngineConfig", "build_from_args", "DPBlockDistributedSampler",
           "EpochDrivenDataLoader", "TorchTurboEngine"]
