"""Packed-sequence metadata built once per batch and reused by every layer.

`build_packed_params` does the single device-to-host read of `cu_seqlens`; a padded tail (tokens after
the last boundary) becomes an extra sequence so operators that must cover every token see a full
partition (ops/packed_params.py:24-120 in the reference).  Besides the chunk tables used by the
linear-attention operators it also prepares the 128-row query-tile table consumed by the varlen
flash-attention kernel.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..utils.functools import cache

CHUNK_SIZES = (16, 32, 64, 128, 1216)


@dataclass(frozen=True)
class PackedParams:
    cu_seqlens: torch.Tensor            # int64 on `device`, includes the padded tail when present
    cu_seqlens_list: list[int]
    chunk_indices: dict[str, torch.Tensor]  # str(chunk) -> int64 [n_chunks, 2] (sequence, chunk)
    chunk_indices_list: dict[str, list[int]]

    @property
    def num_sequences(self) -> int:
        return len(self.cu_seqlens_list) - 1

    @property
    def max_seqlen(self) -> int:
        o = self.cu_seqlens_list
        return max((b - a for a, b in zip(o[:-1], o[1:])), default=0)


def build_packed_params(cu_seqlens: torch.Tensor, chunk_sizes=CHUNK_SIZES, *, total_tokens: int | None = None,
                        device: torch.device | None = None) -> PackedParams:
    if cu_seqlens.ndim != 1:
        raise ValueError(f"cu_seqlens must be rank-1, got {tuple(cu_seqlens.shape)}")
    if cu_seqlens.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"cu_seqlens must be int32/int64, got {cu_seqlens.dtype}")
    device = device or cu_seqlens.device
    offsets = [int(v) for v in cu_seqlens.detach().cpu().tolist()]
    if total_tokens is not None and offsets[-1] < total_tokens:
        offsets.append(int(total_tokens))
    tensors, lists = {}, {}
    for cs in dict.fromkeys(chunk_sizes):
        flat: list[int] = []
        for s, (a, b) in enumerate(zip(offsets[:-1], offsets[1:])):
            for c in range((b - a + cs - 1) // cs):
                flat += [s, c]
        lists[str(cs)] = flat
        tensors[str(cs)] = torch.tensor(flat, dtype=torch.int64, device=device).reshape(-1, 2)
    return PackedParams(torch.tensor(offsets, dtype=torch.int64, device=device), offsets, tensors, lists)


@cache
def _cached(cu_seqlens, total_tokens, device, _version):
    return build_packed_params(cu_seqlens, total_tokens=total_tokens, device=device)


def get_packed_params(cu_seqlens: torch.Tensor | None, total_tokens: int, *, device=None) -> PackedParams | None:
    if cu_seqlens is None:
        return None
    device = device or cu_seqlens.device
    if torch.is_inference_mode_enabled() or cu_seqlens.is_inference():
        return build_packed_params(cu_seqlens, total_tokens=total_tokens, device=device)
    return _cached(cu_seqlens, total_tokens, device, cu_seqlens._version)
