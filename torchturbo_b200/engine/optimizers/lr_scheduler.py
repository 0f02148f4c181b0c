"""Learning-rate schedules: linear / cosine / constant with warm-up, plus cosine variants whose floor is
an *absolute* per-group `min_lr` (groups with different base rates share one floor rule)
(engine/optimizers/lr_scheduler.py:15-130 of the reference)."""
from __future__ import annotations

import math
from typing import Any

import torch
from torch.optim.lr_scheduler import LambdaLR


def _warmup(step: int, warmup: int) -> float | None:
    if warmup > 0 and step < warmup:
        return float(step) / float(max(1, warmup))
    return None


def _cosine_min_lr_lambdas(optimizer, warmup, total, min_lr, num_cycles=0.5, warmup_from_min=False):
    lambdas = []
    for g in optimizer.param_groups:
        base = g.get("initial_lr", g["lr"])
        floor = g.get("min_lr", min_lr)
        ratio = min(floor / base, 1.0) if base > 0 else 0.0

        def fn(step, ratio=ratio):
            w = _warmup(step, warmup)
            if w is not None:
                return ratio + (1 - ratio) * w if warmup_from_min else w
            prog = min(1.0, (step - warmup) / max(1, total - warmup))
            cos = 0.5 * (1.0 + math.cos(math.pi * 2.0 * num_cycles * prog))
            return ratio + (1.0 - ratio) * cos

        lambdas.append(fn)
    return lambdas


def create_lr_scheduler(name: str, optimizer: torch.optim.Optimizer, num_warmup_steps: int = 0,
                        num_training_steps: int | None = None, **kwargs: Any):
    name = str(name).lower()
    total = num_training_steps
    if name in ("cosine_with_min_lr", "cosine_warmup_with_min_lr"):
        if total is None:
            raise ValueError(f"{name} needs num_training_steps")
        min_lr = kwargs.get("min_lr")
        if min_lr is None:
            rate = kwargs.get("min_lr_rate")
            if rate is None:
                raise ValueError(f"{name} needs min_lr or min_lr_rate")
            min_lr = None
        if min_lr is None:
            for g in optimizer.param_groups:
                g.setdefault("min_lr", g["lr"] * kwargs["min_lr_rate"])
            min_lr = 0.0
        return LambdaLR(optimizer, _cosine_min_lr_lambdas(optimizer, num_warmup_steps, total, float(min_lr),
                                                          kwargs.get("num_cycles", 0.5),
                                                          warmup_from_min=(name == "cosine_warmup_with_min_lr")))
    if name == "constant":
        return LambdaLR(optimizer, lambda s: 1.0)
    if name == "constant_with_warmup":
        return LambdaLR(optimizer, lambda s: _warmup(s, num_warmup_steps) or 1.0 if s < num_warmup_steps else 1.0)
    if total is None:
        raise ValueError(f"{name} needs num_training_steps")
    if name == "linear":
        def fn(s):
            w = _warmup(s, num_warmup_steps)
            return w if w is not None else max(0.0, (total - s) / max(1, total - num_warmup_steps))
        return LambdaLR(optimizer, fn)
    if name == "cosine":
        cycles = kwargs.get("num_cycles", 0.5)

        def fn(s):
            w = _warmup(s, num_warmup_steps)
            if w is not None:
                return w
            prog = (s - num_warmup_steps) / max(1, total - num_warmup_steps)
            return max(0.0, 0.5 * (1.0 + math.cos(math.pi * 2.0 * cycles * prog)))
        return LambdaLR(optimizer, fn)
    if name == "polynomial":
        power, end = kwargs.get("power", 1.0), kwargs.get("lr_end", 1e-7)
        base = optimizer.defaults["lr"]

        def fn(s):
            w = _warmup(s, num_warmup_steps)
            if w is not None:
                return w
            if s > total:
                return end / base
            rem = 1 - (s - num_warmup_steps) / max(1, total - num_warmup_steps)
            return ((base - end) * rem ** power + end) / base
        return LambdaLR(optimizer, fn)
    raise ValueError(f"unknown lr scheduler {name!r}")
