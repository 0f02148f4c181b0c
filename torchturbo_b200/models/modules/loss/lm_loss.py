"""Language-model loss on packed batches.

Label preparation (engine/backends/fsdp2/backend.py:1821-1918 of the reference): stream 0 is the main
next-token stream, stream i >= 1 the i-th multi-token-prediction depth.  Labels are shifted left by `1 + i`,
targets that would cross the end of their document are masked, the normaliser is computed on the FULL
sequence, and only then are labels sliced to the sequence-parallel shard.

Two loss formulations with identical values:
  * `logits_loss`: cross entropy from materialised logits;
  * `chunk_loss` : fused lm_head + cross entropy from hidden states (on B200: per chunk a tcgen05 logits GEMM,
    an in-place CE-gradient kernel and two gradient GEMMs; fp32 logits are never materialised).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from ....ops import ops

IGNORE_INDEX = -100


_STAGING: dict[tuple, tuple[torch.Tensor, "torch.cuda.Event | None"]] = {}


def _to_device_async(host: torch.Tensor, device: torch.device) -> torch.Tensor:
    """Host -> device copy that does not block the host: staged through a cached pinned buffer (a copy from pageable
    memory waits for the stream).  The buffer is reused only after its previous copy has finished."""
    if device.type != "cuda":
        return host.to(device)
    key = (tuple(host.shape), host.dtype, device.index)
    buf, ev = _STAGING.get(key, (None, None))
    if buf is None:
        buf = torch.empty(host.shape, dtype=host.dtype, pin_memory=True)
    elif ev is not None:
        ev.synchronize()
    buf.copy_(host)
    out = buf.to(device, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(device))
    _STAGING[key] = (buf, ev)
    return out


def shift_labels_packed(labels: torch.Tensor, cu_seq_lens: torch.Tensor, shift: int = 1) -> torch.Tensor:
    """labels [1, T] -> shifted [1, T]: position t gets `labels[t + shift]` unless that target lies beyond the
    end of t's document (or t is padding after `cu[-1]`), in which case it gets -100.  The validity mask depends on
    the (host) boundaries only; it is built on the host and sent without blocking."""
    T = labels.shape[-1]
    flat = labels.reshape(-1)
    out = torch.full_like(flat, IGNORE_INDEX)
    if shift < T:
        out[: T - shift] = flat[shift:]
    cu = torch.as_tensor(cu_seq_lens).to(device="cpu", dtype=torch.long)
    pos = torch.arange(T)
    seg = torch.searchsorted(cu, pos, right=True)              # index of the boundary after pos
    seg_end = torch.where(seg < cu.numel(), cu[seg.clamp(max=cu.numel() - 1)], torch.zeros_like(pos))
    keep = _to_device_async(pos + shift < seg_end, labels.device)
    out = torch.where(keep, out, torch.full_like(out, IGNORE_INDEX))
    return out.view_as(labels)


@dataclass
class LossStream:
    labels: torch.Tensor        # [1, T_local] shifted, masked, sliced
    normalizer: torch.Tensor | float
    scale: float = 1.0
    name: str = "main"


def prepare_loss_labels(labels: torch.Tensor, cu_seq_lens: torch.Tensor, *, num_streams: int = 1,
                        stream_scales: Sequence[float] | None = None, num_items_in_batch: int | torch.Tensor | None = None,
                        sp_size: int = 1, sp_rank: int = 0, world_size: int = 1) -> list[LossStream]:
    """`labels` is the global (SP-padded) row.  Normaliser: `(num_items_in_batch // sp) * sp / world` when the
    trainer supplies a global token count, else `count(valid shifted labels over the full row) * sp`."""
    streams = []
    T = labels.shape[-1]
    local = T // sp_size
    for i in range(num_streams):
        sh = shift_labels_packed(labels, cu_seq_lens, 1 + i)
        if num_items_in_batch is not None:
            n = num_items_in_batch
            n = (torch.div(n, sp_size, rounding_mode="floor") if isinstance(n, torch.Tensor) else n // sp_size) * sp_size
            norm = n / world_size
        else:
            norm = (sh != IGNORE_INDEX).sum().clamp(min=1) * sp_size
        if sp_size > 1:
            sh = sh[..., sp_rank * local:(sp_rank + 1) * local].contiguous()
        scale = 1.0 if stream_scales is None else float(stream_scales[i])
        streams.append(LossStream(sh, norm, scale, "main" if i == 0 else f"mtp{i}"))
    return streams


def _finish(sums: list[torch.Tensor], streams: Sequence[LossStream]):
    comps, total = {}, None
    for s, st in zip(sums, streams):
        li = s / st.normalizer
        comps[st.name] = li.detach()
        if st.scale == 0.0:
            continue
        term = li * st.scale
        total = term if total is None else total + term
    if total is None:
        total = sums[0] * 0.0
    return total, comps


def logits_loss(logits: Sequence[torch.Tensor] | torch.Tensor, streams: Sequence[LossStream]):
    """`logits[i]`: [1, T_local, V] for stream i.  Returns (total, {stream name: loss})."""
    if isinstance(logits, torch.Tensor):
        logits = [logits]
    sums = [ops.cross_entropy_loss(lg.reshape(-1, lg.shape[-1]), st.labels.reshape(-1)) for lg, st in zip(logits, streams)]
    return _finish(sums, streams)


def chunk_loss(hidden: Sequence[torch.Tensor] | torch.Tensor, lm_head, streams: Sequence[LossStream],
               chunk_size: int = 1024):
    """`hidden[i]`: [1, T_local, H] for stream i; all streams share the output projection.  `lm_head` is either
    the head module (called with `labels=` so FSDP hooks run) or a plain `[V, H]` weight tensor."""
    if isinstance(hidden, torch.Tensor):
        hidden = [hidden]
    sums = []
    for h, st in zip(hidden, streams):
        if isinstance(lm_head, torch.nn.Module):
            sums.append(lm_head(h, labels=st.labels, chunk_size=chunk_size))
        else:
            sums.append(ops.linear_cross_entropy(h.reshape(-1, h.shape[-1]), lm_head, st.labels.reshape(-1),
                                                 chunk_size=chunk_size))
    return _finish(sums, streams)
