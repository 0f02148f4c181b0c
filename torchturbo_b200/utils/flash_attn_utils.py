"""Padding <-> packed conversions for attention inputs.

Host frameworks hand over either padded batches with a 0/1 `attention_mask`, padded batches whose mask holds packed
sample ids (1, 2, 3, ... per row, 0 = padding), or already flattened rows with `cu_seq_lens`.  These helpers turn all of
them into the packed `[T, heads, D]` + `cu_seqlens` form the attention operators take and back (same contracts as
utils/flash_attn_utils.py:110-313 of the reference)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def get_unpad_data(attention_mask: torch.Tensor):
    """attention_mask [B, S]: 0 = padding; values > 0 are sample ids inside the row (a plain 0/1 mask is the one-sample
    case).  Returns (indices [T] of kept tokens in the flattened batch, cu_seqlens int32 [n+1], max_seqlen)."""
    m = attention_mask.to(torch.int64)
    B, S = m.shape
    keep = m > 0
    indices = torch.nonzero(keep.flatten(), as_tuple=False).flatten()
    # a new sequence starts where the id changes or a row starts
    prev = F.pad(m[:, :-1], (1, 0), value=0)
    starts = keep & (m != prev)
    ids = starts.flatten().cumsum(0)[keep.flatten()]                       # 1-based sequence number per kept token
    n = int(ids.max()) if ids.numel() else 0
    lens = torch.bincount(ids - 1, minlength=n) if n else torch.zeros(0, dtype=torch.int64, device=m.device)
    cu = F.pad(lens.cumsum(0), (1, 0)).to(torch.int32)
    return indices, cu, int(lens.max()) if n else 0


def unpad_input(x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """[B, S, ...] -> [T, ...]"""
    return x.flatten(0, 1).index_select(0, indices)


def pad_input(x: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    """[T, ...] -> [B, S, ...] with zeros at padding."""
    out = x.new_zeros((batch * seqlen,) + tuple(x.shape[1:]))
    out.index_copy_(0, indices, x)
    return out.view(batch, seqlen, *x.shape[1:])


def unpad_varlen_inputs(q, k, v, attention_mask):
    """q [B, S, Hq, D], k / v [B, S, Hk, D] -> packed tensors + metadata dict."""
    indices, cu, mx = get_unpad_data(attention_mask)
    return unpad_input(q, indices), unpad_input(k, indices), unpad_input(v, indices), \
        {"indices": indices, "cu_seqlens": cu, "max_seqlen": mx, "batch": q.shape[0], "seqlen": q.shape[1]}


def cu_seqlens_to_segment_ids(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """[n+1] boundaries -> [total] ids 1..n (0 after the last boundary)."""
    cu = torch.as_tensor(cu_seqlens, dtype=torch.long)
    pos = torch.arange(total, device=cu.device)
    seg = torch.bucketize(pos, cu[1:], right=True) + 1
    return torch.where(pos < cu[-1], seg, torch.zeros_like(seg))
