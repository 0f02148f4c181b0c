from .adamw_swap import AdamWSwap
from .container import OptimizersContainer
from .fused_adamw import FusedAdamW
from .lr_scheduler import create_lr_scheduler
from .plan import OptimizerClassPlan, OptimizerPlan, ParamGroup

__all__ = ["AdamWSwap", "OptimizersContainer", "FusedAdamW", "create_lr_scheduler", "OptimizerClassPlan", "OptimizerPlan", "ParamGroup"]
