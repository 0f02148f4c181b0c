from .base import OpImpl, OpImplKind, OpPolicy, OpSpec
from .dispatcher import OpDispatcher
from .moe import MoEPermutation, get_expert_indices
from .ops import get_or_create_ops, ops
from .packed_params import PackedParams, build_packed_params, get_packed_params
from .registry import REGISTRY, OpRegistry, register_op

__all__ = ["OpImpl", "OpImplKind", "OpPolicy", "OpSpec", "OpDispatcher", "MoEPermutation", "get_expert_indices",
           "get_or_create_ops", "ops", "PackedParams", "build_packed_params", "get_packed_params", "REGISTRY",
           "OpRegistry", "register_op"]
