"""Explicit all-gather prefetch topology for FSDP2 units of MoE models.

FSDP2 by itself prefetches "the next unit in execution order".  With expert containers as separate units
that order interleaves layer / experts / layer / experts, so the implicit rule only ever overlaps one small
gather.  The manager discovers the chain of decoder-layer units and the chain of expert units and sets
`set_modules_to_forward_prefetch` / `set_modules_to_backward_prefetch` so that, depending on the strategy,
  * `layer`             : layer i prefetches layers i+1 .. i+depth;
  * `expert_with_layer` : layer i additionally prefetches the experts of layers i+1 .. i+depth;
  * `expert_lookahead`  : experts form their own rolling chain (experts i prefetch experts i+1 .. i+depth);
  * `auto`              : `expert_with_layer` when expert units exist, else `layer`; `native` leaves FSDP alone.
Same role as engine/backends/fsdp2/prefetch.py:153-562 of the reference.
"""
from __future__ import annotations

import contextlib

import torch.nn as nn

from ...config import FSDPConfig, FSDPPrefetchDirection, FSDPPrefetchStrategy


def _is_fsdp(m: nn.Module) -> bool:
    return getattr(m, "_tt_unit", None) == "fsdp" and hasattr(m, "set_modules_to_forward_prefetch")


class FSDPPrefetchManager:
    def __init__(self, config: FSDPConfig):
        self.config = config
        self.layer_chain: list[nn.Module] = []
        self.expert_chain: list[nn.Module | None] = []
        self.expert_groups: list[list[nn.Module]] = []
        self._suspended = False
        self._saved: dict[int, list] = {}

    # -- discovery ---------------------------------------------------------------------------------
    def _discover(self, model: nn.Module) -> None:
        best: list[nn.Module] = []
        for mod in model.modules():
            if isinstance(mod, nn.ModuleList):
                units = [c for c in mod if _is_fsdp(c)]
                if len(units) > len(best):
                    best = units
        self.layer_chain = best
        self.expert_chain = []
        self.expert_groups: list[list[nn.Module]] = []
        for layer in best:
            # a unit may hold several merged decoder layers: its expert units are those of all its members;
            # the first one is the handle that carries expert -> expert prefetch lists
            members = getattr(layer, "_tt_group", None) or [layer]
            ex = [m for member in members for m in member.modules() if m not in members and _is_fsdp(m)]
            self.expert_groups.append(ex)
            self.expert_chain.append(ex[0] if ex else None)

    def resolved_strategy(self) -> FSDPPrefetchStrategy:
        s = self.config.prefetch_strategy
        if s is FSDPPrefetchStrategy.AUTO:
            has_experts = any(e is not None for e in self.expert_chain)
            return FSDPPrefetchStrategy.EXPERT_WITH_LAYER if has_experts else FSDPPrefetchStrategy.LAYER
        return s

    # -- plan ----------------------------------------------------------------------------------------
    def build_targets(self, n: int, depth: int, strategy: FSDPPrefetchStrategy, has_expert: list[bool]):
        """Pure planning function (unit-tested without FSDP): for source index i returns
        (layer targets, expert targets of the layer source, expert targets of the expert source)."""
        plan = []
        covered_layer, covered_expert = set(), set()
        for i in range(n):
            lt = [j for j in range(i + 1, min(n, i + 1 + depth)) if j not in covered_layer]
            covered_layer.update(lt)
            et_layer, et_expert = [], []
            if strategy is FSDPPrefetchStrategy.EXPERT_WITH_LAYER:
                et_layer = [j for j in range(i + 1, min(n, i + 1 + depth)) if has_expert[j] and j not in covered_expert]
                covered_expert.update(et_layer)
            elif strategy is FSDPPrefetchStrategy.EXPERT_LOOKAHEAD and has_expert[i]:
                et_expert = [j for j in range(i + 1, min(n, i + 1 + depth)) if has_expert[j] and j not in covered_expert]
                covered_expert.update(et_expert)
            plan.append((lt, et_layer, et_expert))
        return plan

    def setup(self, model: nn.Module) -> None:
        self._discover(model)
        strategy = self.resolved_strategy()
        if strategy is FSDPPrefetchStrategy.NATIVE or len(self.layer_chain) < 2:
            return
        n = len(self.layer_chain)
        has = [e is not None for e in self.expert_chain]
        fwd = self.build_targets(n, self.config.forward_prefetch_depth, strategy, has)
        for i, (lt, el, ee) in enumerate(fwd):
            mods = [self.layer_chain[j] for j in lt] + [e for j in el for e in self.expert_groups[j]]
            if mods:
                self.layer_chain[i].set_modules_to_forward_prefetch(mods)
            if ee and self.expert_chain[i] is not None:
                self.expert_chain[i].set_modules_to_forward_prefetch([self.expert_chain[j] for j in ee])
        if self.config.prefetch_direction is FSDPPrefetchDirection.FORWARD_BACKWARD:
            bwd = self.build_targets(n, self.config.backward_prefetch_depth, strategy, has[::-1])
            rl, re_, rg = self.layer_chain[::-1], self.expert_chain[::-1], self.expert_groups[::-1]
            for i, (lt, el, ee) in enumerate(bwd):
                mods = [rl[j] for j in lt] + [e for j in el for e in rg[j][::-1]]
                if mods:
                    rl[i].set_modules_to_backward_prefetch(mods)
                if ee and re_[i] is not None:
                    re_[i].set_modules_to_backward_prefetch([re_[j] for j in ee])

    @contextlib.contextmanager
    def suspend_expert_forward_prefetch(self):
        """During activation-checkpoint recomputation of one layer the experts of later layers must not be
        gathered again; the explicit forward lists of expert units are emptied for the duration."""
        touched = []
        for e in [e for g in self.expert_groups for e in g]:
            if e is not None and hasattr(e, "set_modules_to_forward_prefetch"):
                st = e._get_fsdp_state() if hasattr(e, "_get_fsdp_state") else None
                prev = list(getattr(st, "_states_to_forward_prefetch", [])) if st is not None else []
                touched.append((e, st, prev))
                e.set_modules_to_forward_prefetch([])
        try:
            yield
        finally:
            for e, st, prev in touched:
                if st is not None:
                    st._states_to_forward_prefetch = prev
