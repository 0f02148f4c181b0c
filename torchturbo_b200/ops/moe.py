"""Provider-independent result of packing MoE tokens (contract of ops/moe.py:10-46 in the reference).

Rows of `tokens` are ordered by (expert id, source token id).  `row_indices[t, j]` is the packed row
holding token `t`'s j-th assignment and `expert_indices[t, j]` the expert of that assignment.

The B200 provider pads every expert segment to a multiple of 128 rows (zero rows) so that grouped
tcgen05 GEMM tiles never straddle experts; it then also fills `seg_start`, `counts` and `tile_group`
(all on the device: nothing is synchronised with the host).  The native provider leaves them `None`
and packs densely.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class MoEPermutation:
    tokens: torch.Tensor
    probs: torch.Tensor | None
    row_indices: torch.Tensor      # int32 [T, k]
    expert_indices: torch.Tensor   # int64 [T, k]
    counts: torch.Tensor | None = None      # int32 [E] tokens per expert
    seg_start: torch.Tensor | None = None   # int32 [E + 1] padded segment starts
    tile_group: torch.Tensor | None = None  # int32 [capacity / 128] expert of each 128-row tile (-1: unused)
    # optional preallocated [capacity, H] buffers the expert MLP writes its output (forward) and its input gradient
    # (backward) into, e.g. the peer-visible buffer of an expert-parallel dispatcher (saves a copy each way)
    out_buffer: torch.Tensor | None = None
    grad_buffer: torch.Tensor | None = None

    @property
    def padded(self) -> bool:
        return self.seg_start is not None


def get_expert_indices(routing_map: torch.Tensor) -> torch.Tensor:
    """Expert ids [T, k] (ascending per token) from a boolean [T, E] routing map with fixed k per token."""
    T = routing_map.shape[0]
    if T == 0:
        return routing_map.new_empty((0, 0), dtype=torch.long)
    rows, experts = routing_map.nonzero(as_tuple=True)
    if experts.numel() % T:
        raise ValueError("routing_map does not select the same number of experts for every token")
    k = experts.numel() // T
    if not torch.equal(rows, torch.arange(T, device=rows.device).repeat_interleave(k)):
        raise ValueError("routing_map does not select the same number of experts for every token")
    return experts.reshape(T, k)
