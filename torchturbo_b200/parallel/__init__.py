from .fsdp import FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec, VisionBalanceMode, VisionBalanceSpec
from .parallel import ParallelPlan

__all__ = ["ParallelPlan", "FSDPParallelPlan", "FSDPPlacementSpec", "FSDPPlanSpec", "VisionBalanceMode",
           "VisionBalanceSpec"]
