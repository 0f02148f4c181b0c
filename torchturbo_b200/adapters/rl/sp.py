"""Sequence-parallel helpers for RL: per-token statistics are computed on the local shard and gathered along the
sequence so that every SP rank sees the full row (adapters/rl/sp.py:40-130 of the reference)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...models.modules.comm import all_gather_tensor


def gather_logprobs_and_shift(local_logp: torch.Tensor, sp_group, sp_size: int, total_len: int | None = None) -> torch.Tensor:
    """[T_local] per-token values of every SP rank -> [T] (padding tail trimmed to `total_len`)."""
    if sp_size <= 1:
        return local_logp if total_len is None else local_logp[:total_len]
    full = all_gather_tensor(local_logp.contiguous(), sp_group)
    return full if total_len is None else full[:total_len]


def gather_vocab_logits_stats(local_logits: torch.Tensor, sp_group, sp_size: int) -> dict[str, torch.Tensor]:
    """Mean / max of the logits over the *global* sequence (diagnostics that RL trainers log)."""
    s = local_logits.float()
    stats = torch.stack([s.sum(), torch.tensor(float(s.numel()), device=s.device)])
    mx = s.max().reshape(1)
    if sp_size > 1:
        dist.all_reduce(stats, group=sp_group)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=sp_group)
    return {"mean": stats[0] / stats[1], "max": mx[0]}
