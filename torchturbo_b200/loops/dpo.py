"""Direct preference optimisation on packed batches.

One packed row holds `2N` segments: the N chosen answers followed by the N rejected ones (each with its prompt).
Policy and frozen reference model run the same row; per-token log-probabilities come from a full-vocabulary
log-softmax in fp32, are summed per segment, and feed the sigmoid / IPO / hinge preference losses.  Token weights
(IPO length normalisation, LD-DPO down-weighting of the tail beyond the shorter answer) are computed on the
global row *before* it is sharded for sequence parallelism, and the per-segment statistics of all SP ranks are
combined with a single all-reduce (adapters/msswift/trainer.py:479-668 and adapters/llamafactory_v0/trainer.py:590-797
of the reference).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..models.modules.loss import shift_labels_packed

IGNORE_INDEX = -100


@dataclass
class DPOConfig:
    beta: float = 0.1
    loss_type: str = "sigmoid"       # sigmoid | ipo | hinge
    label_smoothing: float = 0.0
    ld_alpha: float | None = None    # LD-DPO: weight of the tokens beyond min(len_chosen, len_rejected)
    sft_alpha: float = 0.0           # optional NLL regulariser on the chosen answers


def segment_token_weights(labels_shifted: torch.Tensor, cu: torch.Tensor, cfg: DPOConfig) -> torch.Tensor:
    """Per-token weights of the global row: 1 on valid targets, `ld_alpha` on the part of the longer answer that
    exceeds the shorter one (pair i = segments i and i + N)."""
    flat = labels_shifted.reshape(-1)
    w = (flat != IGNORE_INDEX).float()
    if cfg.ld_alpha is None:
        return w
    offs = cu.tolist()
    n = (len(offs) - 1) // 2
    for i in range(n):
        spans = [(offs[i], offs[i + 1]), (offs[i + n], offs[i + n + 1])]
        lens = [int((flat[a:b] != IGNORE_INDEX).sum()) for a, b in spans]
        short = min(lens)
        for (a, b), L in zip(spans, lens):
            if L > short:
                pos = torch.nonzero(flat[a:b] != IGNORE_INDEX).reshape(-1)[short:] + a
                w[pos] = cfg.ld_alpha
    return w


def segment_sums(values: torch.Tensor, offsets: list[int], lo: int, hi: int) -> torch.Tensor:
    """Sum of `values` (the local shard covering global positions [lo, hi)) per segment."""
    out = values.new_zeros(len(offsets) - 1)
    for s, (a, b) in enumerate(zip(offsets[:-1], offsets[1:])):
        a2, b2 = max(a, lo), min(b, hi)
        if b2 > a2:
            out[s] = values[a2 - lo:b2 - lo].sum()
    return out


def sequence_logps(engine, model, batch: dict, cfg: DPOConfig, *, grad: bool):
    """(per-segment summed log-prob [2N], per-segment valid-token count [2N]) for the packed row in `batch`."""
    be = engine.backend
    inputs = model.on_prepare_inputs(dict(batch), source_inputs=batch)
    inputs = be.prepare_inputs(model, inputs)
    labels = inputs.pop("labels").to(be.device)
    cu = inputs["cu_seq_lens_q"]
    shifted = shift_labels_packed(labels, cu, 1)
    weights = segment_token_weights(shifted, cu, cfg).to(be.device)
    T = shifted.shape[-1]
    sp, r = be.sp_size, be.sp_rank
    lo, hi = (r * (T // sp), (r + 1) * (T // sp)) if sp > 1 else (0, T)
    if inputs.get("position_ids") is None:
        inputs["position_ids"] = torch.arange(T, device=be.device).unsqueeze(0)
    be._prepare_moe_runtime(model, inputs, 1.0)
    with torch.set_grad_enabled(grad):
        out = model(**inputs)
        logits = out["logits"].reshape(-1, out["logits"].shape[-1])
        tgt = shifted.reshape(-1)[lo:hi]
        lsm = F.log_softmax(logits.float(), dim=-1)
        tok = lsm.gather(1, tgt.clamp(min=0).unsqueeze(1)).squeeze(1)
        tok = torch.where(tgt != IGNORE_INDEX, tok, torch.zeros_like(tok)) * weights[lo:hi]
    offs = cu.tolist()
    sums = segment_sums(tok, offs, lo, hi)
    counts = segment_sums((tgt != IGNORE_INDEX).float(), offs, lo, hi)
    if sp > 1:
        from ..models.modules.comm import all_reduce_sum_autograd

        stacked = torch.stack([sums, counts])
        stacked = all_reduce_sum_autograd(stacked, be.sp_group)
        sums, counts = stacked[0], stacked[1]
    return sums, counts


def dpo_loss(pol: torch.Tensor, ref: torch.Tensor, counts: torch.Tensor, cfg: DPOConfig):
    """pol / ref: [2N] summed log-probs (chosen first).  Returns (loss, metrics)."""
    n = pol.numel() // 2
    if cfg.loss_type == "ipo":
        pol, ref = pol / counts.clamp(min=1), ref / counts.clamp(min=1)
    pc, pr, rc, rr = pol[:n], pol[n:], ref[:n], ref[n:]
    logits = (pc - pr) - (rc - rr)
    if cfg.loss_type == "sigmoid":
        loss = -F.logsigmoid(cfg.beta * logits) * (1 - cfg.label_smoothing) - F.logsigmoid(-cfg.beta * logits) * cfg.label_smoothing
    elif cfg.loss_type == "ipo":
        loss = (logits - 1 / (2 * cfg.beta)) ** 2
    elif cfg.loss_type == "hinge":
        loss = torch.relu(1 - cfg.beta * logits)
    else:
        raise ValueError(f"unknown DPO loss_type {cfg.loss_type!r}")
    if cfg.sft_alpha:
        loss = loss - cfg.sft_alpha * pc / counts[:n].clamp(min=1)
    cr, rj = cfg.beta * (pc - rc).detach(), cfg.beta * (pr - rr).detach()
    return loss.mean(), {"rewards/chosen": cr.mean(), "rewards/rejected": rj.mean(),
                         "rewards/accuracies": (cr > rj).float().mean(), "rewards/margins": (cr - rj).mean()}


def dpo_step(engine, policy, reference, optimizer, batch: dict, cfg: DPOConfig, *, max_grad_norm: float = 1.0):
    """One optimizer step of DPO on one packed row.  `reference` is a second engine-built model (frozen, eval); when it
    is `None` the batch must carry precomputed `reference_logps` ([2N])."""
    if reference is not None:
        reference.eval()
        ref, _ = sequence_logps(engine, reference, batch, DPOConfig(cfg.beta, cfg.loss_type, ld_alpha=None), grad=False)
    else:
        ref = batch["reference_logps"].to(engine.backend.device)
    pol, counts = sequence_logps(engine, policy, batch, cfg, grad=True)
    loss, metrics = dpo_loss(pol, ref.detach(), counts, cfg)
    loss.backward()
    gnorm = engine.clip_grad_norm_(policy, max_grad_norm, optimizer)
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    return loss.detach(), gnorm, metrics


def build_reference_model(engine, model_name_or_path=None, *, policy=None, init_kwargs=None):
    """A frozen copy of the policy built by the same engine (same plan and sharding).  Without a checkpoint path the
    reference starts from the policy's current weights."""
    ref = engine.build_model(model_name_or_path, load_weights=model_name_or_path is not None, init_kwargs=init_kwargs)
    if model_name_or_path is None and policy is not None:
        with torch.no_grad():
            for (_, a), (_, b) in zip(ref.named_parameters(), policy.named_parameters()):
                la = a._local_tensor if hasattr(a, "_local_tensor") else a
                lb = b._local_tensor if hasattr(b, "_local_tensor") else b
                la.copy_(lb)
    for p in ref.parameters():
        p.requires_grad_(False)
    return ref.eval()
