"""One facade over several optimizers (e.g. Muon for matrices + AdamW for the rest, or one AdamW per
sharding topology).  It quacks like a `torch.optim.Optimizer` for schedulers and trainers: `param_groups`
is the concatenation, `step`/`zero_grad` fan out, and `state_dict` is versioned and keyed per child
(engine/optimizers/container.py:16-213 of the reference)."""
from __future__ import annotations

from typing import Any, Callable

import torch

_STATE_VERSION = 1


class OptimizersContainer(torch.optim.Optimizer):
    def __init__(self, optimizers: list[torch.optim.Optimizer], names: list[str] | None = None):
        if not optimizers:
            raise ValueError("OptimizersContainer needs at least one optimizer")
        self.optimizers = list(optimizers)
        self.names = list(names) if names else [f"opt{i}" for i in range(len(optimizers))]
        if len(set(self.names)) != len(self.names):
            raise ValueError("optimizer names must be unique")
        # torch.optim.Optimizer.__init__ is intentionally not called: groups and state live in the children
        self.defaults = dict(optimizers[0].defaults)
        self._optimizer_step_pre_hooks, self._optimizer_step_post_hooks = {}, {}
        self._pre: list[Callable] = []
        self._post: list[Callable] = []

    @property
    def param_groups(self):
        return [g for o in self.optimizers for g in o.param_groups]

    @param_groups.setter
    def param_groups(self, v):  # schedulers never assign; ignore attempts from base-class helpers
        pass

    @property
    def state(self):
        merged = {}
        for o in self.optimizers:
            merged.update(o.state)
        return merged

    @state.setter
    def state(self, v):
        pass

    def register_step_pre_hook(self, hook):
        self._pre.append(hook)
        return hook

    def register_step_post_hook(self, hook):
        self._post.append(hook)
        return hook

    def step(self, closure=None, **kwargs):
        for h in self._pre:
            h(self, (), {})
        loss = closure() if closure is not None else None
        for o in self.optimizers:
            try:
                o.step(**kwargs)
            except TypeError:
                o.step()
        for h in self._post:
            h(self, (), {})
        return loss

    def zero_grad(self, set_to_none: bool = True):
        for o in self.optimizers:
            o.zero_grad(set_to_none=set_to_none)

    def state_dict(self) -> dict[str, Any]:
        return {"version": _STATE_VERSION, "optimizers": {n: o.state_dict() for n, o in zip(self.names, self.optimizers)}}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        if sd.get("version") != _STATE_VERSION:
            raise ValueError(f"unsupported optimizer container state version {sd.get('version')!r}")
        children = sd["optimizers"]
        if set(children) != set(self.names):
            raise ValueError(f"optimizer set mismatch: saved {sorted(children)}, current {sorted(self.names)}")
        for n, o in zip(self.names, self.optimizers):
            o.load_state_dict(children[n])

    def __len__(self):
        return len(self.optimizers)

    def __iter__(self):
        return iter(self.optimizers)
