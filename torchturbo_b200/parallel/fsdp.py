"""Declarative FSDP plan: FQN pattern -> how that module is sharded, replaced, checkpointed or balanced.

Public surface kept from the reference (parallel/fsdp.py:18-187): `VisionBalanceMode`, `VisionBalanceSpec`,
`FSDPPlacementSpec`, `FSDPPlanSpec`, `FSDPParallelPlan` with tuple/placement normalisation, `to_dict`,
`from_dict` (partial overrides keep `None` for unset fields) and first-match `match`.
"""
from __future__ import annotations

import copy
from collections.abc import Mapping
from dataclasses import dataclass, field, fields
from enum import Enum
from typing import Any

from ..utils.fqn import match_fqn
from .parallel import ParallelPlan


class VisionBalanceMode(str, Enum):
    """Weight of one media item when whole images are redistributed over ranks."""

    PATCH = "patch"        # number of patches
    PATCH_SQ = "patch_sq"  # patches squared (attention cost)


@dataclass
class VisionBalanceSpec:
    mode: VisionBalanceMode | None = None
    io: Any | None = None  # BaseVisionBalanceIO

    def __post_init__(self) -> None:
        if self.mode is not None and not isinstance(self.mode, VisionBalanceMode):
            raise TypeError("VisionBalanceSpec.mode must be a VisionBalanceMode")


@dataclass
class FSDPPlacementSpec:
    placement: Any            # DTensor placement, e.g. Shard(0)
    mesh_dim: str | int | None = None  # "edp", "dp", ... ; None lets the backend pick


@dataclass
class FSDPPlanSpec:
    placement: FSDPPlacementSpec | None = None
    no_shard: bool = False
    standalone_world_shard: bool = False
    activation_checkpoint: bool = False
    replace_module: Any | None = None
    module_kwargs: dict[str, Any] = field(default_factory=dict)
    vision_balance: VisionBalanceSpec | None = None

    def __post_init__(self) -> None:
        if self.vision_balance is not None and not isinstance(self.vision_balance, VisionBalanceSpec):
            raise TypeError("FSDPPlanSpec.vision_balance must be a VisionBalanceSpec")
        if self.no_shard and (self.standalone_world_shard or self.placement is not None):
            raise ValueError("no_shard excludes standalone_world_shard and placement")
        if self.standalone_world_shard and self.placement is not None:
            raise ValueError("standalone_world_shard is redundant with an explicit placement")


_SPEC_FIELDS = tuple(f.name for f in fields(FSDPPlanSpec))


@dataclass
class FSDPParallelPlan(ParallelPlan):
    plan: dict[str, Any] = field(default_factory=dict)
    sp_size: int = 1
    ep_size: int = 1
    tp_size: int = 1  # accepted for config compatibility; tensor parallelism is not part of the engine

    def __post_init__(self) -> None:
        for key, value in list(self.plan.items()):
            if isinstance(value, FSDPPlanSpec):
                continue
            if isinstance(value, FSDPPlacementSpec):
                self.plan[key] = FSDPPlanSpec(placement=value)
            elif isinstance(value, tuple) and len(value) == 2:
                self.plan[key] = FSDPPlanSpec(placement=FSDPPlacementSpec(value[0], value[1]))
            else:
                self.plan[key] = FSDPPlanSpec(placement=FSDPPlacementSpec(value))

    def to_dict(self) -> dict[str, Any]:
        snap = copy.deepcopy(self)
        out: dict[str, Any] = {"sp_size": snap.sp_size, "ep_size": snap.ep_size, "tp_size": snap.tp_size, "plan": {}}
        for fqn, spec in snap.plan.items():
            d = {name: getattr(spec, name) for name in _SPEC_FIELDS}
            if d["placement"] is not None:
                d["placement"] = {"placement": d["placement"].placement, "mesh_dim": d["placement"].mesh_dim}
            if d["vision_balance"] is not None:
                d["vision_balance"] = {"mode": d["vision_balance"].mode, "io": d["vision_balance"].io}
            out["plan"][fqn] = d
        return out

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "FSDPParallelPlan":
        """Full plans and partial overrides alike: fields absent from an entry stay `None`, which the
        engine reads as "inherit the model's default"."""
        entries: dict[str, FSDPPlanSpec] = {}
        for fqn, raw in (data.get("plan") or {}).items():
            kw: dict[str, Any] = dict.fromkeys(_SPEC_FIELDS)
            kw.update(raw)
            if isinstance(kw["placement"], Mapping):
                kw["placement"] = FSDPPlacementSpec(**kw["placement"])
            vb = kw["vision_balance"]
            if isinstance(vb, Mapping):
                mode = vb.get("mode")
                kw["vision_balance"] = VisionBalanceSpec(mode=VisionBalanceMode(mode) if mode is not None else None,
                                                         io=vb.get("io"))
            spec = FSDPPlanSpec.__new__(FSDPPlanSpec)  # partial specs may hold None in boolean fields
            for name in _SPEC_FIELDS:
                setattr(spec, name, kw[name])
            entries[fqn] = spec
        plan = cls.__new__(cls)
        plan.plan = entries
        plan.sp_size = data.get("sp_size")
        plan.ep_size = data.get("ep_size")
        plan.tp_size = data.get("tp_size")
        return plan

    def match(self, fqn: str) -> FSDPPlanSpec | None:
        for pattern, spec in self.plan.items():
            if match_fqn(pattern, fqn):
                return spec
        return None
