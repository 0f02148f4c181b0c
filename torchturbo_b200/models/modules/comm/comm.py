"""Differentiable collectives used by expert parallelism, sequence parallelism and vision balancing.

NCCL (or gloo on CPU) implementations; they are the control-plane/baseline path.  The fused in-kernel
NVLink variants live in `torchturbo_b200.comm` and are selected by the modules that own a hot path.
Semantics follow models/modules/comm/comm.py:5-276 of the reference: all-to-all-v whose backward swaps the
split lists, and a sequence-region gather whose backward either reduce-scatters (outputs consumed by
every rank) or just slices (outputs consumed identically everywhere).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _size(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def all_gather_tensor(x: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate equally shaped `x` of every rank along dim 0 (no autograd)."""
    n = _size(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = x.new_empty((n * x.shape[0],) + tuple(x.shape[1:]))
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def all_gather_tensor_chunked(x: torch.Tensor, group=None, max_bytes: int = 1 << 30) -> torch.Tensor:
    """`all_gather_tensor` in row chunks so the transient buffer stays below `max_bytes` per call."""
    n = _size(group)
    if n == 1:
        return x
    row_bytes = max(1, x[0].numel() * x.element_size()) if x.shape[0] else 1
    rows = max(1, max_bytes // (row_bytes * n))
    if rows >= x.shape[0]:
        return all_gather_tensor(x, group)
    parts = [all_gather_tensor(x[s:s + rows], group) for s in range(0, x.shape[0], rows)]
    # parts[i] is rank-major; re-interleave to a rank-major concatenation of full tensors
    per_rank = [[] for _ in range(n)]
    for p, s in zip(parts, range(0, x.shape[0], rows)):
        r = min(rows, x.shape[0] - s)
        for k in range(n):
            per_rank[k].append(p[k * r:(k + 1) * r])
    return torch.cat([torch.cat(c, 0) for c in per_rank], 0)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, x, output_split_sizes, input_split_sizes):
        ctx.group, ctx.out_splits, ctx.in_splits = group, output_split_sizes, input_split_sizes
        n = _size(group)
        if n == 1:
            return x
        x = x.contiguous()
        if output_split_sizes is None:
            out = torch.empty_like(x)
        else:
            out = x.new_empty((int(sum(output_split_sizes)),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, output_split_sizes=output_split_sizes, input_split_sizes=input_split_sizes,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return None, _AllToAll.apply(ctx.group, g, ctx.in_splits, ctx.out_splits), None, None


def all_to_all(group, x, output_split_sizes=None, input_split_sizes=None) -> torch.Tensor:
    """all-to-all(-v) along dim 0; the backward is the same exchange with the split lists swapped."""
    return _AllToAll.apply(group, x, output_split_sizes, input_split_sizes)


class _GatherFromSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, reduce_scatter_grad):
        ctx.group, ctx.rs = group, reduce_scatter_grad
        ctx.rank, ctx.n = (dist.get_rank(group), _size(group)) if dist.is_initialized() else (0, 1)
        return all_gather_tensor(x, group)

    @staticmethod
    def backward(ctx, g):
        if ctx.n == 1:
            return g, None, None
        g = g.contiguous()
        local = g.shape[0] // ctx.n
        if ctx.rs:
            out = g.new_empty((local,) + tuple(g.shape[1:]))
            dist.reduce_scatter_tensor(out, g, group=ctx.group)
            return out, None, None
        return g.narrow(0, ctx.rank * local, local).contiguous(), None, None


def gather_from_sequence_parallel_region(x, tensor_parallel_output_grad: bool = True, group=None) -> torch.Tensor:
    """All-gather along dim 0.  `tensor_parallel_output_grad=True`: every rank's loss may depend on every
    shard, so the backward reduce-scatters; `False`: the gathered value is consumed identically on every
    rank and the backward keeps the local slice."""
    return _GatherFromSequenceParallelRegion.apply(x, group, tensor_parallel_output_grad)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        if _size(group) == 1:
            return x
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        if _size(ctx.group) == 1:
            return g, None
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def all_reduce_sum_autograd(x: torch.Tensor, group=None) -> torch.Tensor:
    """SUM all-reduce whose backward is also a SUM all-reduce (loss terms shared by a group)."""
    return _AllReduceSum.apply(x, group)
