"""ms-swift batches -> the engine's packed-row contract, on the host, before the trainer moves anything to the device.

Three shapes come out of swift's template collator:
  * packing / padding-free: one row that already concatenates the samples (optionally with `cu_seq_lens_*`), possibly
    with alignment padding on the left or right,
  * plain padded `[B, S]` batches with a 0/1 `attention_mask`,
  * RLHF (DPO) batches where the chosen samples come first and the rejected ones after them.
All of them leave here as one row whose valid prefix is described by `cu_seq_lens_q/k` + `max_length_q/k`, with the
first label of every sample masked (it has no in-sample predecessor) and binary `loss_scale` folded into the labels.
Same contract as adapters/msswift/inputs_bridging.py:21-330 of the reference.
"""
from __future__ import annotations

from itertools import accumulate
from typing import Any, Callable, Sequence

import torch

from ...engine.utils import assert_packed_inputs
from ...logging import get_logger
from ...utils.flash_attn_utils import get_unpad_data

logger = get_logger(__name__)
IGNORE_INDEX = -100
_ROW_KEYS = ("input_ids", "labels", "loss_scale", "position_ids", "text_position_ids", "mm_token_type_ids")


def _require_cpu(t: torch.Tensor, what: str) -> None:
    if t.device.type != "cpu":
        raise ValueError(f"{what} must be normalised on the host, before the device transfer")


def bridge_packed_inputs(inputs: dict[str, Any], *, sequence_lengths: Sequence[int], padding_side: str = "right") -> dict[str, Any]:
    """A row that already holds the samples back to back.  `sequence_lengths` are the original sample lengths: they,
    not position resets, separate real tokens from alignment padding.  Padding ends up at the tail."""
    ids = inputs["input_ids"]
    _require_cpu(ids, "packed swift inputs")
    total, valid = ids.shape[-1], sum(sequence_lengths)
    pad = total - valid
    if pad < 0 or not sequence_lengths or min(sequence_lengths) <= 0:
        raise ValueError("sample lengths must be positive and fit the collated row")
    if pad and padding_side == "left":
        for k in _ROW_KEYS:
            if inputs.get(k) is not None:
                inputs[k] = inputs[k].roll(-pad, dims=-1)
    want = torch.tensor([0, *accumulate(sequence_lengths)], dtype=torch.int32)
    for k in ("cu_seq_lens_q", "cu_seq_lens_k"):
        cu = inputs.get(k)
        if cu is not None:
            _require_cpu(cu, k)
            if pad:
                off = pad if padding_side == "left" else 0
                cu = cu[(cu >= off) & (cu <= off + valid)] - off
            if not torch.equal(cu.to(torch.int32), want):
                raise ValueError(f"{k} does not match the original sample boundaries")
        inputs[k] = want.clone()
    mx = max(sequence_lengths)
    for k in ("max_length_q", "max_length_k"):
        v = inputs.get(k, mx)
        inputs[k] = int(v) if isinstance(v, torch.Tensor) else v
    if inputs.get("labels") is not None:
        inputs["labels"][0, want[:-1].long()] = IGNORE_INDEX
    inputs.pop("attention_mask", None)
    assert_packed_inputs(inputs)
    return inputs


def bridge_unpacked_inputs(inputs: dict[str, Any]) -> dict[str, Any]:
    """A padded `[B, S]` batch: rows are flattened with the padding removed; every row is one sequence."""
    ids = inputs["input_ids"]
    _require_cpu(ids, "swift inputs")
    mask = inputs.pop("attention_mask")
    B, S = ids.shape
    if tuple(mask.shape) != (B, S):
        raise ValueError("attention_mask must match input_ids")
    keep, cu, mx = get_unpad_data((mask > 0).to(torch.int64))
    lens = (cu[1:] - cu[:-1]).tolist()
    text_pos = torch.cat([torch.arange(n) for n in lens]).unsqueeze(0)
    pos = inputs.get("position_ids")
    if pos is not None:
        inputs["position_ids"] = pos.flatten(1).index_select(1, keep).unsqueeze(1) if pos.dim() == 3 else \
            pos.flatten().index_select(0, keep).unsqueeze(0)
    elif inputs.get("mm_token_type_ids") is None:
        inputs["position_ids"] = text_pos          # multimodal batches must bring the template's rotary coordinates
    if inputs.get("text_position_ids") is not None:
        inputs["text_position_ids"] = text_pos
    for k in ("input_ids", "labels", "loss_scale", "mm_token_type_ids"):
        v = inputs.get(k)
        if v is not None:
            if tuple(v.shape[:2]) != (B, S):
                raise ValueError(f"{k} must align with the collated rows")
            inputs[k] = v.flatten(0, 1).index_select(0, keep).unsqueeze(0)
    if inputs.get("labels") is not None:
        inputs["labels"][0, cu[:-1].long()] = IGNORE_INDEX
    inputs["cu_seq_lens_q"], inputs["cu_seq_lens_k"] = cu, cu.clone()
    inputs["max_length_q"] = inputs["max_length_k"] = mx
    assert_packed_inputs(inputs)
    return inputs


def bake_loss_scale_into_labels(inputs: dict[str, Any]) -> dict[str, Any]:
    """Binary `loss_scale` (0 = skip) becomes -100 labels; the shifted cross entropy never reads `loss_scale`.
    Fractional weights cannot be expressed that way: they are dropped with a warning."""
    ls, labels = inputs.get("loss_scale"), inputs.get("labels")
    if ls is None or labels is None:
        return inputs
    ls = ls.reshape(labels.shape)
    off = ls <= 0
    if bool(((ls > 0) & (ls < 1)).any()):
        logger.warning_rank0("loss_scale holds fractional weights; only zero / positive is honoured")
    if bool(off.any()):
        inputs["labels"] = labels.masked_fill(off, IGNORE_INDEX)
    inputs.pop("loss_scale", None)
    return inputs


def bridge_swift_inputs(inputs: dict[str, Any], *, sequence_lengths: Sequence[int] | None = None,
                        padding_side: str = "right") -> dict[str, Any]:
    inputs = bake_loss_scale_into_labels(inputs)
    if sequence_lengths is not None:
        return bridge_packed_inputs(inputs, sequence_lengths=sequence_lengths, padding_side=padding_side)
    if inputs.get("attention_mask") is not None:
        return bridge_unpacked_inputs(inputs)
    if inputs.get("cu_seq_lens_q") is None:
        raise ValueError("a swift batch needs sample lengths, an attention mask or cu_seq_lens")
    assert_packed_inputs(inputs)
    return inputs


class SwiftInputCollator:
    """Runs swift's own collator, then normalises its result.  Sample lengths are taken from the raw samples before
    swift flattens and mutates the batch; DPO batches list all chosen samples, then all rejected ones."""

    def __init__(self, collator: Callable[[list], dict[str, Any]], template: Any):
        self.collator, self.template = collator, template

    def __call__(self, batch: list) -> dict[str, Any]:
        dpo = getattr(self.template, "mode", None) == "rlhf"
        lengths = None
        if getattr(self.template, "padding_free", False):
            samples = [s for g in batch for s in g] if isinstance(batch[0], list) else batch
            lengths = [len(s[f"{p}input_ids"]) for p in ("chosen_", "rejected_") for s in samples] if dpo else \
                [len(s["input_ids"]) for s in samples]
        side = getattr(self.template, "padding_side", "right") if getattr(self.template, "is_training", True) else "left"
        out = self.collator(batch)
        if dpo:
            return bridge_unpacked_inputs(out) if lengths is None else \
                bridge_packed_inputs(out, sequence_lengths=lengths, padding_side=side)
        return bridge_swift_inputs(out, sequence_lengths=lengths, padding_side=side)
