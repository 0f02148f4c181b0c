"""Windowed mean of per-module metrics.

Modules that want to report something expose `pop_metrics() -> dict[str, Tensor]`; the engine calls
`collect(model)` after every micro-step and `report(logs, gather)` at log time, which averages over
micro-steps and ranks (engine/metrics/tracker.py:6-27 of the reference)."""
from __future__ import annotations

from collections import defaultdict
from typing import Callable

import torch


class MetricTracker:
    def __init__(self) -> None:
        self._sums: dict[str, torch.Tensor] = {}
        self._counts: dict[str, int] = defaultdict(int)

    def add(self, name: str, value: torch.Tensor | float) -> None:
        v = value.detach().float() if isinstance(value, torch.Tensor) else torch.tensor(float(value))
        self._sums[name] = self._sums[name] + v if name in self._sums else v
        self._counts[name] += 1

    def collect(self, model: torch.nn.Module) -> None:
        per_step: dict[str, list[torch.Tensor]] = defaultdict(list)
        producers = getattr(model, "_tt_metric_modules", None)
        if producers is None:   # the modules that can report metrics are found once per model
            producers = [m for m in model.modules() if callable(getattr(m, "pop_metrics", None))]
            object.__setattr__(model, "_tt_metric_modules", producers)
        for m in producers:
            for k, v in m.pop_metrics().items():
                per_step[k].append(v)
        for k, vs in per_step.items():
            self.add(k, torch.stack([v.float() for v in vs]).mean())

    def report(self, logs: dict, gather: Callable[[torch.Tensor], torch.Tensor] | None = None) -> dict:
        for k, s in self._sums.items():
            mean = s / max(self._counts[k], 1)
            if gather is not None:
                mean = gather(mean.reshape(1)).float().mean()
            logs[k] = float(mean)
        self._sums, self._counts = {}, defaultdict(int)
        return logs
