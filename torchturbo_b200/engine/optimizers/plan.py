"""Optimizer construction contract.

An `OptimizerPlan` lists parameter groups (each with its own hyper-parameters and optimizer class); an
`OptimizerClassPlan(cls, lr=..., weight_decay=...)` is the common single-class case and splits trainable
parameters into decay / no-decay groups (biases and 1-D tensors get `weight_decay=0`).  The backend further
splits groups by sharding topology, because fused/foreach optimizers cannot mix DTensor meshes
(engine/optimizers/plan.py:19-343 of the reference)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Iterable

import torch
import torch.nn as nn


@dataclass
class ParamGroup:
    name: str
    params: list[nn.Parameter]
    param_names: list[str]
    optimizer_cls: type | Callable[..., torch.optim.Optimizer]
    hyperparameters: dict[str, Any] = field(default_factory=dict)

    def as_torch_group(self) -> dict[str, Any]:
        return {"params": self.params, **self.hyperparameters}


@dataclass
class OptimizerPlan:
    groups: list[ParamGroup] = field(default_factory=list)

    def by_class(self) -> dict[Any, list[ParamGroup]]:
        out: dict[Any, list[ParamGroup]] = {}
        for g in self.groups:
            out.setdefault(g.optimizer_cls, []).append(g)
        return out

    def validate(self, model: nn.Module) -> None:
        seen: set[int] = set()
        for g in self.groups:
            for p in g.params:
                if id(p) in seen:
                    raise ValueError(f"parameter appears in more than one optimizer group ({g.name})")
                seen.add(id(p))
        missing = [n for n, p in model.named_parameters() if p.requires_grad and id(p) not in seen]
        if missing:
            raise ValueError(f"trainable parameters without an optimizer group: {missing[:5]}{'...' if len(missing) > 5 else ''}")


def is_no_decay(name: str, p: torch.Tensor) -> bool:
    return p.ndim <= 1 or name.endswith(".bias")


@dataclass
class OptimizerClassPlan:
    optimizer_cls: type | Callable[..., torch.optim.Optimizer]
    lr: float = 1e-3
    weight_decay: float = 0.0
    kwargs: dict[str, Any] = field(default_factory=dict)

    def __init__(self, optimizer_cls, lr: float = 1e-3, weight_decay: float = 0.0, **kwargs: Any):
        self.optimizer_cls, self.lr, self.weight_decay, self.kwargs = optimizer_cls, lr, weight_decay, kwargs

    def resolve(self, named_params: Iterable[tuple[str, nn.Parameter]]) -> OptimizerPlan:
        decay_p, decay_n, nodecay_p, nodecay_n = [], [], [], []
        for n, p in named_params:
            if not p.requires_grad:
                continue
            if is_no_decay(n, p):
                nodecay_p.append(p); nodecay_n.append(n)
            else:
                decay_p.append(p); decay_n.append(n)
        groups = []
        hp = dict(lr=self.lr, **self.kwargs)
        if decay_p:
            groups.append(ParamGroup("decay", decay_p, decay_n, self.optimizer_cls, {**hp, "weight_decay": self.weight_decay}))
        if nodecay_p:
            groups.append(ParamGroup("no_decay", nodecay_p, nodecay_n, self.optimizer_cls, {**hp, "weight_decay": 0.0}))
        return OptimizerPlan(groups)
