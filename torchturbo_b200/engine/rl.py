"""Packed-batch API for RL frameworks (`prepare_packed_micro_batch`, `forward_backward_batch`, `compute_logprobs`),
mixed into `TorchTurboEngine` (engine/core.py:1201-1470 of the reference).

An RL trainer hands the engine lists of token sequences plus per-token loss inputs; the engine packs them into the
packed-row contract, runs forward / backward per micro-batch with token-weighted normalisation across the data-parallel
group, and returns per-token log-probabilities (and entropies) in the original sequence layout."""
from __future__ import annotations

from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist

from ..adapters.rl.packed import gather_logprobs_entropy, prepare_packed_mb_inputs, shifted_packed_tensor
from ..adapters.rl.sp import gather_logprobs_and_shift


class RLMixin:
    def prepare_packed_micro_batch(self, sequences: Sequence[torch.Tensor], extras: dict[str, Sequence[torch.Tensor]] | None = None):
        """Pack sequences (1-D token tensors) into one row padded to a multiple of the SP size; per-token extras
        (advantages, old log-probs, masks) are concatenated and padded with zeros alike."""
        sp = self.backend.sp_size
        mb = prepare_packed_mb_inputs(list(sequences), pad_to_multiple_of=sp)
        T = mb["input_ids"].shape[-1]
        for k, vs in (extras or {}).items():
            flat = torch.cat([v.reshape(-1) for v in vs])
            if flat.numel() < T:
                flat = torch.cat([flat, flat.new_zeros(T - flat.numel())])
            mb[k] = flat.unsqueeze(0)
        return mb

    def _forward_microbatch(self, model, inputs: dict[str, Any]):
        keys = ("input_ids", "position_ids", "cu_seq_lens_q", "cu_seq_lens_k", "max_length_q", "max_length_k",
                "pixel_values", "image_grid_thw")
        model_in = {k: inputs[k] for k in keys if k in inputs}
        model_in = self.backend.prepare_inputs(model, model.on_prepare_inputs(model_in, source_inputs=inputs))
        self.backend._prepare_moe_runtime(model, model_in, 1.0)
        return model(**model_in)

    def _logprobs_and_entropy(self, model, mb: dict[str, Any], want_entropy: bool):
        be = self.backend
        out = self._forward_microbatch(model, mb)
        logits = out["logits"].reshape(-1, out["logits"].shape[-1])
        ids = mb["input_ids"].to(be.device)
        targets = shifted_packed_tensor(ids, mb["cu_seq_lens_q"], fill=-100).reshape(-1)
        T = targets.numel()
        lo, hi = (be.sp_rank * (T // be.sp_size), (be.sp_rank + 1) * (T // be.sp_size)) if be.sp_size > 1 else (0, T)
        lp, ent = gather_logprobs_entropy(logits, targets[lo:hi], want_entropy=want_entropy)
        return lp, ent, (targets != -100)

    @torch.no_grad()
    def compute_logprobs(self, model, micro_batches: Sequence[dict[str, Any]], want_entropy: bool = False):
        """Per-token log-prob of the next token for every micro-batch, gathered over the SP group: list of [T]."""
        model.eval()
        outs = []
        for mb in micro_batches:
            lp, ent, valid = self._logprobs_and_entropy(model, mb, want_entropy)
            lp = gather_logprobs_and_shift(lp, self.backend.sp_group, self.backend.sp_size)
            if want_entropy:
                ent = gather_logprobs_and_shift(ent, self.backend.sp_group, self.backend.sp_size)
            outs.append((lp, ent) if want_entropy else lp)
        model.train()
        return outs

    def forward_backward_batch(self, model, micro_batches: Sequence[dict[str, Any]],
                               loss_fn: Callable[[torch.Tensor, torch.Tensor | None, dict[str, Any]], torch.Tensor],
                               *, want_entropy: bool = False, loss_weight_key: str | None = "loss_mask"):
        """Forward + backward over the micro-batches of one optimizer step.  `loss_fn(logp, entropy, mb)` returns
        per-token losses on this rank's shard; they are normalised by the total loss weight of the global batch
        (all micro-batches, all DP ranks), so gradients do not depend on how the batch was split."""
        be = self.backend
        total_w = torch.zeros((), dtype=torch.float32, device=be.device)
        for mb in micro_batches:
            w = mb.get(loss_weight_key) if loss_weight_key else None
            total_w += (w.float().sum().to(be.device) if w is not None else
                        torch.tensor(float(int(mb["cu_seq_lens_q"][-1])), device=be.device))
        if dist.is_initialized() and be.dp_size > 1:
            dist.all_reduce(total_w, group=be.dp_group)
        total_w = total_w.clamp(min=1.0)
        mult = self._get_loss_multiplier()
        total = torch.zeros((), dtype=torch.float32, device=be.device)
        for mb in micro_batches:
            lp, ent, _ = self._logprobs_and_entropy(model, mb, want_entropy)
            per_tok = loss_fn(lp, ent, mb)
            T = mb["input_ids"].shape[-1]
            lo, hi = (be.sp_rank * (T // be.sp_size), (be.sp_rank + 1) * (T // be.sp_size)) if be.sp_size > 1 else (0, T)
            w = mb.get(loss_weight_key) if loss_weight_key else None
            if w is not None:
                per_tok = per_tok * w.reshape(-1)[lo:hi].to(per_tok.device).float()
            loss = per_tok.sum() / total_w * mult
            loss.backward()
            total += loss.detach()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(total)
            total /= mult
        return total

    def _get_loss_multiplier(self) -> float:
        """FSDP averages gradients over the world; a sum-normalised global loss therefore needs `world` back
        (each SP rank contributes its shard, each DP rank its samples)."""
        return float(self.backend.world_size)
