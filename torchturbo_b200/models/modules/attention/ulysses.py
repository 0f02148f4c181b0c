"""Ulysses sequence parallelism for packed attention and the SP input contract.

Around attention every rank trades its sequence shard of all heads for the full sequence of `heads/sp`
heads (seq -> head all-to-all for q, k, v) and back (head -> seq for the output).  Packed metadata
(`cu_seq_lens`, `max_length`) always describes the *global* sequence, so no position gather is needed.
Inputs are right-padded to a multiple of `sp` and sliced at a model-declared boundary.

Behavioural contract: models/modules/attention/ulysses/ulysses.py:30-649 and ulysses/utils.py:7-99 of the
reference.  Layout here is token-major `[T, heads, D]` (the batch dimension of a packed row is 1).
The exchange itself is pluggable: `nccl` (torch.distributed all_to_all_single, also gloo on CPU) or
`p2p` (the in-kernel NVLink path of `torchturbo_b200.comm.ulysses_p2p`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from functools import wraps
from types import MethodType
from typing import Any, Callable, Mapping

import torch
import torch.distributed as dist

from ..comm import gather_from_sequence_parallel_region


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[T, H, D] -> [T, H * n_rep, D] with each head repeated consecutively."""
    if n_rep == 1:
        return x
    T, H, D = x.shape
    return x[:, :, None, :].expand(T, H, n_rep, D).reshape(T, H * n_rep, D)


def slice_input_tensor(x: torch.Tensor, dim: int, group, rank: int) -> torch.Tensor:
    sp = dist.get_world_size(group)
    n = x.size(dim)
    if n % sp:
        raise ValueError(f"sequence length {n} is not divisible by the SP size {sp}; pad with ulysses_pad_inputs()")
    return x.narrow(dim, rank * (n // sp), n // sp).contiguous()


# --------------------------------------------------------------------------------------------------
# the two exchanges as autograd functions (each one's backward is the other)
# --------------------------------------------------------------------------------------------------
def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)
    return out


def _seq_to_head(x: torch.Tensor, group, sp: int) -> torch.Tensor:
    """[T_local, H, D] -> [T_local * sp, H / sp, D]"""
    Tl, H, D = x.shape
    send = x.view(Tl, sp, H // sp, D).permute(1, 0, 2, 3).contiguous()
    return _a2a(send, group).view(sp * Tl, H // sp, D)


def _head_to_seq(x: torch.Tensor, group, sp: int) -> torch.Tensor:
    """[T, H_local, D] -> [T / sp, H_local * sp, D]"""
    T, Hl, D = x.shape
    recv = _a2a(x.contiguous().view(sp, T // sp, Hl, D), group)
    return recv.permute(1, 0, 2, 3).reshape(T // sp, sp * Hl, D)


class SeqAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sp, to_heads):
        ctx.group, ctx.sp, ctx.to_heads = group, sp, to_heads
        return _seq_to_head(x, group, sp) if to_heads else _head_to_seq(x, group, sp)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = _head_to_seq(g, ctx.group, ctx.sp) if ctx.to_heads else _seq_to_head(g, ctx.group, ctx.sp)
        return out, None, None, None


def gather_seq_scatter_heads(x, group, sp):
    return x if sp <= 1 else SeqAllToAll.apply(x, group, sp, True)


def gather_heads_scatter_seq(x, group, sp):
    return x if sp <= 1 else SeqAllToAll.apply(x, group, sp, False)


def ulysses_attention(q, k, v, cu_seqlens, max_seqlen, *, sp_group=None, sp_size: int = 1, causal=True, scale=None,
                      attention_fn: Callable | None = None, want_max_logits: bool = False):
    """Attention over a sequence sharded across `sp_size` ranks.

    q: [T_local, Hq, D]; k, v: [T_local, Hkv, D]; `cu_seqlens` / `max_seqlen` are global.  KV heads are
    repeated up to `sp_size` when there are fewer of them; query heads are repeated to `lcm(sp, Hq)` when
    `Hq` is not a multiple of `sp` and de-duplicated afterwards."""
    from ....ops import ops

    attention_fn = attention_fn or (ops.attention_with_max_logits if want_max_logits else ops.attention)
    if sp_size <= 1:
        return attention_fn(q, k, v, cu_seqlens, max_seqlen, causal=causal, scale=scale)
    Hq, Hkv = q.shape[1], k.shape[1]
    q_rep = 1
    if Hq % sp_size:
        q_rep = math.lcm(Hq, sp_size) // Hq
        q = repeat_kv(q, q_rep)
    kv_target = max(sp_size, Hkv)
    if kv_target % Hkv or (q.shape[1] // sp_size) % max(kv_target // sp_size, 1):
        kv_target = q.shape[1]  # fall back to MHA layout when head groups would not align
    kv_rep = kv_target // Hkv
    k, v = repeat_kv(k, kv_rep), repeat_kv(v, kv_rep)
    qh = gather_seq_scatter_heads(q, sp_group, sp_size)
    kh = gather_seq_scatter_heads(k, sp_group, sp_size)
    vh = gather_seq_scatter_heads(v, sp_group, sp_size)
    res = attention_fn(qh, kh, vh, cu_seqlens, max_seqlen, causal=causal, scale=scale)
    out, max_logits = (res if want_max_logits else (res, None))
    out = gather_heads_scatter_seq(out, sp_group, sp_size)
    if q_rep > 1:
        out = out[:, ::q_rep, :]
    if want_max_logits:
        ml = max_logits.clone()
        dist.all_gather_into_tensor(full := ml.new_empty(sp_size * ml.numel()), ml, group=sp_group)
        full = full[::q_rep] if q_rep > 1 else full
        return out, full
    return out


# --------------------------------------------------------------------------------------------------
# SP input contract
# --------------------------------------------------------------------------------------------------
class SequencePadding(Enum):
    ZERO = "zero"
    IGNORE_INDEX = "ignore_index"
    POSITION = "position"


@dataclass(frozen=True)
class SequenceParallelInputSlicingSpec:
    """Which batch fields are right-padded to a multiple of `sp` and which call arguments of which module
    method are sliced to the local shard.  Packed metadata and media tensors stay global."""

    module: torch.nn.Module
    original_forward: Callable[..., Any]
    forward_name: str = "forward"
    sliced_inputs: tuple[tuple[str, int], ...] = (("inputs_embeds", 1), ("position_ids", -1))
    padded_inputs: tuple[tuple[str, SequencePadding], ...] = (
        ("input_ids", SequencePadding.ZERO),
        ("mm_token_type_ids", SequencePadding.ZERO),
        ("labels", SequencePadding.IGNORE_INDEX),
        ("position_ids", SequencePadding.POSITION),
        ("text_position_ids", SequencePadding.POSITION),
    )


def _pad_sequence(t: torch.Tensor, pad: int, how: SequencePadding) -> torch.Tensor:
    if how is SequencePadding.POSITION:
        tail = torch.arange(pad, device=t.device, dtype=t.dtype).expand(*t.shape[:-1], pad)
        return torch.cat((t, tail), dim=-1)
    return torch.nn.functional.pad(t, (0, pad), value=-100 if how is SequencePadding.IGNORE_INDEX else 0)


def ulysses_pad_inputs(inputs: Mapping[str, Any], spec: SequenceParallelInputSlicingSpec, sp_size: int) -> dict:
    """New batch whose declared fields are right-padded so `input_ids` is a multiple of `sp_size`.  Tail
    values: 0 for ids, -100 for labels, 0,1,2,... for positions.  `cu_seq_lens` keeps describing the
    valid prefix, so attention, MoE statistics and losses ignore the tail."""
    out = dict(inputs)
    pad = (-inputs["input_ids"].size(-1)) % sp_size
    if pad == 0:
        return out
    for name, how in spec.padded_inputs:
        t = inputs.get(name)
        if t is not None:
            out[name] = _pad_sequence(t, pad, how)
    return out


def patch_forward_for_sp_input_slicing(spec: SequenceParallelInputSlicingSpec, sp_group, sp_size: int,
                                       sp_rank: int) -> None:
    """Wrap `spec.module.<forward_name>` so that its declared keyword inputs arrive as local shards."""
    if sp_size <= 1:
        return

    @wraps(spec.original_forward)
    def sliced_forward(self, *args, **kwargs):
        kw = dict(kwargs)
        for name, dim in spec.sliced_inputs:
            v = kw.get(name)
            if v is None:
                continue
            if isinstance(v, tuple):
                kw[name] = tuple(slice_input_tensor(t, dim, sp_group, sp_rank) for t in v)
            else:
                kw[name] = slice_input_tensor(v, dim, sp_group, sp_rank)
        return spec.original_forward(self, *args, **kw)

    setattr(spec.module, spec.forward_name, MethodType(sliced_forward, spec.module))


def all_gather_sp_with_grad_reduce(t: torch.Tensor, dim: int, sp_group, sp_size: int) -> torch.Tensor:
    """Full-sequence copy on every SP rank (KV for sparse attention, conv halos); gradients of all ranks
    are summed back onto the owning shard (forward all-gather, backward reduce-scatter)."""
    if sp_size <= 1 or sp_group is None:
        return t
    dim = dim % t.dim()
    moved = t.movedim(dim, 0).contiguous()
    return gather_from_sequence_parallel_region(moved, True, sp_group).movedim(0, dim).contiguous()
