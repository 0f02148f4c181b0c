from .balance import (FanoutPlan, MediaMeta, MediaPool, PixelPlan, VisionBalanceState, lpt_weight,
                      register_vision_balance)
from .io import BaseVisionBalanceIO, GridVisionBalanceIO, VisionBatch

__all__ = ["FanoutPlan", "MediaMeta", "MediaPool", "PixelPlan", "VisionBalanceState", "lpt_weight",
           "register_vision_balance", "BaseVisionBalanceIO", "GridVisionBalanceIO", "VisionBatch"]
