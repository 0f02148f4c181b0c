"""Packed-input contract checks and small helpers shared by the engine and adapters."""
from __future__ import annotations

import inspect
from typing import Any, Callable

import torch

from ..utils.fqn import match_fqn  # noqa: F401  (re-exported: plans and policies import it from here)

IGNORE_INDEX = -100


def validate_signature(function: Callable[..., Any], /, **expected_defaults: Any) -> None:
    """Require `function` to expose the given keyword parameters with exactly these defaults."""
    try:
        params = inspect.signature(function).parameters
    except (TypeError, ValueError) as e:
        raise TypeError(f"cannot inspect {function!r}") from e
    for name, default in expected_defaults.items():
        if name not in params:
            raise TypeError(f"{function!r} has no parameter {name!r}")
        if params[name].default != default:
            raise TypeError(f"{function!r}: parameter {name!r} must default to {default!r}")


def raise_if_evaluation_enabled(do_eval: bool, what: str = "evaluation") -> None:
    if do_eval:
        raise ValueError(f"{what} during training is not supported by the engine-managed loop")


def get_packed_boundaries(position_ids: torch.Tensor | None = None, sample_ids: torch.Tensor | None = None) -> torch.Tensor:
    """`cu_seq_lens` (int32, CPU) of one packed row from either neat-packing sample ids (1,1,2,2,2,0,0: zero =
    padding) or position resets (a new sequence starts wherever the position is 0)."""
    if sample_ids is not None:
        ids = sample_ids.reshape(-1).cpu()
        n = int((ids != 0).sum())
        ids = ids[:n]
        change = torch.nonzero(ids[1:] != ids[:-1]).reshape(-1) + 1
        cu = torch.cat([torch.zeros(1, dtype=torch.long), change, torch.tensor([n])])
        return cu.to(torch.int32)
    pos = position_ids.reshape(-1).cpu()
    starts = torch.nonzero(pos == 0).reshape(-1)
    if starts.numel() == 0 or starts[0] != 0:
        starts = torch.cat([torch.zeros(1, dtype=torch.long), starts])
    return torch.cat([starts, torch.tensor([pos.numel()])]).to(torch.int32)


def assert_packed_inputs(inputs: dict[str, Any]) -> None:
    """One flattened row `[1, T]` with `cu_seq_lens_q == cu_seq_lens_k` (int32, starts at 0, strictly
    increasing, last <= T), `max_length_q == max_length_k == max(diff(cu))` and no `attention_mask`."""
    ids = inputs.get("input_ids")
    if ids is None or ids.dim() != 2 or ids.shape[0] != 1:
        raise ValueError("packed batches carry input_ids of shape [1, T]")
    if inputs.get("attention_mask") is not None:
        raise ValueError("packed batches must not carry attention_mask")
    cu_q, cu_k = inputs.get("cu_seq_lens_q"), inputs.get("cu_seq_lens_k")
    if cu_q is None or cu_k is None:
        raise ValueError("packed batches need cu_seq_lens_q and cu_seq_lens_k")
    if cu_q.dtype != torch.int32 or cu_q.dim() != 1 or not torch.equal(cu_q.cpu(), cu_k.cpu()):
        raise ValueError("cu_seq_lens_q/k must be identical rank-1 int32 tensors")
    c = cu_q.cpu()
    if int(c[0]) != 0 or bool((c[1:] <= c[:-1]).any()) or int(c[-1]) > ids.shape[-1]:
        raise ValueError("cu_seq_lens must start at 0, increase strictly and end at or before T")
    mx = int((c[1:] - c[:-1]).max())
    if int(inputs.get("max_length_q", -1)) != mx or int(inputs.get("max_length_k", -1)) != mx:
        raise ValueError(f"max_length_q/k must equal the longest sequence ({mx})")
    labels = inputs.get("labels")
    if labels is not None and labels.shape != ids.shape:
        raise ValueError("labels must have the shape of input_ids")
    pos = inputs.get("position_ids")
    if pos is not None and pos.dim() == 2:
        p = pos.reshape(-1).cpu()
        if bool((p[c[:-1].long()] != 0).any()):
            raise ValueError("text positions must restart at 0 at every sequence boundary")
