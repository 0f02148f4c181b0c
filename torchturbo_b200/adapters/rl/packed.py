"""Packed-batch helpers for RL frameworks: shifted targets, per-token log-probabilities and entropies
(adapters/rl/packed.py:10-120 of the reference)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ...models.modules.loss import shift_labels_packed

IGNORE_INDEX = -100


def shifted_packed_tensor(x: torch.Tensor, cu_seq_lens: torch.Tensor, fill=0) -> torch.Tensor:
    """`out[t] = x[t + 1]` inside each document; the last token of every document (and padding) gets `fill`."""
    flat = x.reshape(-1)
    src = shift_labels_packed(torch.arange(flat.numel(), device=x.device).reshape(1, -1), cu_seq_lens, 1).reshape(-1)
    valid = src != IGNORE_INDEX
    out = torch.full_like(flat, fill)
    out[valid] = flat[src[valid]]
    return out.view_as(x)


def gather_logprobs_entropy(logits: torch.Tensor, targets: torch.Tensor, *, want_entropy: bool = True,
                            chunk: int = 4096):
    """logits [T, V], targets [T] (-100 = ignore) -> (logp [T], entropy [T] or None), fp32, computed in row chunks so
    the fp32 softmax of a large vocabulary is never materialised for the whole row."""
    T = logits.shape[0]
    lp = torch.zeros(T, dtype=torch.float32, device=logits.device)
    ent = torch.zeros(T, dtype=torch.float32, device=logits.device) if want_entropy else None
    for s in range(0, T, chunk):
        lg = logits[s:s + chunk].float()
        lsm = F.log_softmax(lg, dim=-1)
        tg = targets[s:s + chunk]
        ok = tg != IGNORE_INDEX
        lp[s:s + chunk] = torch.where(ok, lsm.gather(1, tg.clamp(min=0).unsqueeze(1)).squeeze(1), torch.zeros_like(lp[s:s + chunk]))
        if want_entropy:
            ent[s:s + chunk] = -(lsm.exp() * lsm).sum(-1)
    return lp, ent


def prepare_packed_mb_inputs(sequences: list[torch.Tensor], *, pad_to_multiple_of: int = 1, pad_token_id: int = 0) -> dict:
    """List of 1-D token tensors -> one packed row with boundaries (the engine's packed-batch contract)."""
    ids = torch.cat(sequences)
    lens = [int(s.numel()) for s in sequences]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    pad = (-ids.numel()) % pad_to_multiple_of
    if pad:
        ids = torch.cat([ids, ids.new_full((pad,), pad_token_id)])
        pos = torch.cat([pos, torch.arange(pad)])
    return {"input_ids": ids.unsqueeze(0), "position_ids": pos.unsqueeze(0), "cu_seq_lens_q": cu, "cu_seq_lens_k": cu.clone(),
            "max_length_q": max(lens), "max_length_k": max(lens)}
