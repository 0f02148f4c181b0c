"""Block-diffusion training batches for LLaDA2.

One training row is `[noisy | clean]`: the same token sequence twice, the first copy with a random subset of its
response tokens replaced by the mask token.  Attention is blockwise: with blocks of `block_size` tokens numbered
inside each sample,
    * noisy tokens see their own noisy block (both directions) and all *earlier* clean blocks,
    * clean tokens see clean blocks up to and including their own,
    * nothing crosses samples, and padding is never a key.
Only masked, non-pad positions of the noisy half carry labels (unshifted).  Noise is a function of the sample index
alone, so the ranks of a sequence-parallel group, which read the same index, build identical rows.

Same contract as models/llada2_moe/bd.py:227-450 of the reference (mask-ratio range, per-sample seeding, three mask
rules, first-fit-decreasing packing of short samples into one row); the mask is returned as a boolean `allow`
matrix `[2T, 2T]` plus the per-position structure (sample, segment, block) a fused kernel needs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch
from torch.utils.data import Dataset

IGNORE_INDEX = -100
SEG_NOISY, SEG_CLEAN, SEG_PAD = 0, 1, 2


def mask_noise(T: int, prompt_length: int, real_len: int, seed: int, low: float = 0.3, high: float = 0.8):
    """(move [T] bool, sigma): positions of the response (`prompt_length <= p < real_len`) masked with probability
    `sigma ~ U[low, high]`; deterministic in `seed`."""
    g = torch.Generator().manual_seed(int(seed))
    sigma = float(torch.rand(1, generator=g)) * (high - low) + low
    pos = torch.arange(T)
    move = (torch.rand(T, generator=g) < sigma) & (pos >= prompt_length) & (pos < real_len)
    return move, sigma


def block_diffusion_allow(sample: torch.Tensor, seg: torch.Tensor, block: torch.Tensor) -> torch.Tensor:
    """`allow[q, k]` from per-position sample ids (-1 = padding), segments and block numbers."""
    sq, sk = sample[:, None], sample[None, :]
    gq, gk = seg[:, None], seg[None, :]
    bq, bk = block[:, None], block[None, :]
    same = (sq == sk) & (sq >= 0)
    within = (bq == bk) & (gq == gk)
    noisy_sees_clean = (bq > bk) & (gq == SEG_NOISY) & (gk == SEG_CLEAN)
    clean_causal = (bq >= bk) & (gq == SEG_CLEAN) & (gk == SEG_CLEAN)
    return same & (within | noisy_sees_clean | clean_causal) & (gk != SEG_PAD)


@dataclass
class BDSample:
    input_ids: Sequence[int]
    prompt_length: int
    index: int = 0


def build_bd_row(samples: Sequence[BDSample], row_len: int, *, block_size: int = 32, mask_id: int, pad_id: int,
                 low: float = 0.3, high: float = 0.8) -> dict:
    """One `[noisy_0 | clean_0 | noisy_1 | clean_1 | ... | pad]` row of `row_len` tokens.  Every sample is padded to
    a whole number of blocks; `row_len` must fit `2 * sum(padded lengths)`."""
    ids, labels, pos, sample, seg, block = [], [], [], [], [], []
    for s_i, s in enumerate(samples):
        L = len(s.input_ids)
        T = (L + block_size - 1) // block_size * block_size
        toks = torch.full((T,), pad_id, dtype=torch.long)
        toks[:L] = torch.as_tensor(list(s.input_ids), dtype=torch.long)
        move, _ = mask_noise(T, s.prompt_length, L, s.index, low, high)
        noisy = torch.where(move, torch.full_like(toks, mask_id), toks)
        lab = torch.where(move & (toks != pad_id), toks, torch.full_like(toks, IGNORE_INDEX))
        ar = torch.arange(T)
        real = ar < L
        ids += [noisy, toks]
        labels += [lab, torch.full((T,), IGNORE_INDEX, dtype=torch.long)]
        pos += [ar, ar]
        sample += [torch.where(real, s_i, -1)] * 2
        seg += [torch.where(real, SEG_NOISY, SEG_PAD), torch.where(real, SEG_CLEAN, SEG_PAD)]
        block += [ar // block_size, ar // block_size]
    cat = lambda xs: torch.cat(xs) if xs else torch.zeros(0, dtype=torch.long)   # noqa: E731
    ids, labels, pos, sample, seg, block = (cat(x) for x in (ids, labels, pos, sample, seg, block))
    pad = row_len - ids.numel()
    if pad < 0:
        raise ValueError(f"samples need {ids.numel()} tokens but the row holds {row_len}")
    if pad:
        ids = torch.cat((ids, torch.full((pad,), pad_id, dtype=torch.long)))
        labels = torch.cat((labels, torch.full((pad,), IGNORE_INDEX, dtype=torch.long)))
        pos = torch.cat((pos, torch.arange(pad)))
        sample = torch.cat((sample, torch.full((pad,), -1, dtype=torch.long)))
        seg = torch.cat((seg, torch.full((pad,), SEG_PAD, dtype=torch.long)))
        block = torch.cat((block, torch.full((pad,), -2, dtype=torch.long)))
    return {"input_ids": ids.unsqueeze(0), "labels": labels.unsqueeze(0), "position_ids": pos.unsqueeze(0),
            "block_allow": block_diffusion_allow(sample, seg, block),
            "bd_structure": torch.stack((sample, seg, block))}


def first_fit_decreasing(lengths: Sequence[int], capacity: int, block_size: int = 32) -> list[list[int]]:
    """Bins of sample indices whose block-padded lengths sum to at most `capacity` (longest first, first fit)."""
    padded = [(i, (n + block_size - 1) // block_size * block_size) for i, n in enumerate(lengths)]
    bins: list[tuple[int, list[int]]] = []
    for i, n in sorted(padded, key=lambda t: (-t[1], t[0])):
        if n > capacity:
            continue                                   # longer than a row even alone: the caller truncates beforehand
        for b, (used, members) in enumerate(bins):
            if used + n <= capacity:
                bins[b] = (used + n, members + [i])
                break
        else:
            bins.append((n, [i]))
    return [m for _, m in bins]


class BDDataset(Dataset):
    """Rows of `2 * cutoff_len` tokens over pre-tokenised samples (`{"input_ids": [...], "prompt_length": n}`).
    With `pack=True` several short samples share one row."""

    def __init__(self, samples: Sequence[dict], cutoff_len: int, *, mask_id: int, pad_id: int, block_size: int = 32,
                 mask_low: float = 0.3, mask_high: float = 0.8, pack: bool = False):
        self.cutoff = (cutoff_len + block_size - 1) // block_size * block_size
        self.kw = dict(block_size=block_size, mask_id=mask_id, pad_id=pad_id, low=mask_low, high=mask_high)
        self.samples = [BDSample(list(s["input_ids"])[: self.cutoff], min(int(s.get("prompt_length", 0)), self.cutoff), i)
                        for i, s in enumerate(samples)]
        if pack:
            self.rows = first_fit_decreasing([len(s.input_ids) for s in self.samples], self.cutoff, block_size)
        else:
            self.rows = [[i] for i in range(len(self.samples))]

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int) -> dict:
        return build_bd_row([self.samples[j] for j in self.rows[i]], 2 * self.cutoff, **self.kw)
