from .container import OptimizersContainer
from .fused_adamw import FusedAdamW
from .lr_scheduler import create_lr_scheduler
from .plan import OptimizerClassPlan, OptimizerPlan, ParamGroup

__all__ = ["OptimizersContainer", "FusedAdamW", "create_lr_scheduler", "OptimizerClassPlan", "OptimizerPlan", "ParamGroup"]
