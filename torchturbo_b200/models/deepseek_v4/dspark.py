"""DSpark block-draft training for DeepSeek-V4 (checkpoint namespace `mtp.*` when `dspark_block_size > 0`).

A DSpark draft predicts a BLOCK of `B` future tokens in one parallel pass.  Training samples anchor positions in the
packed row; for an anchor `a` the draft block is `[x_a, MASK, ..., MASK]` (B states at positions a .. a+B-1) and state
`j` is trained to predict token `x_{a+j+1}`.  Every draft stage is a DeepSeek-V4 block (hyper-connections, MoE / MLP)
whose attention sees only
  * the `sliding_window` positions of the TARGET model before the anchor (a projection of the concatenated hidden
    states of a few target layers: `main_proj` + `main_norm`, computed by the first stage), and
  * its own block, bidirectionally,
with the per-head attention sink of the family.  The last stage mixes the hyper-connection copies down, applies the
shared output head and adds a low-rank first-order transition bias (`markov_head`: embedding of the previous true
token times an output matrix); `confidence_head` predicts from the final state and that embedding how likely the
target model is to accept the drafted token.

Loss (all sums over the sampled draft rows, weights `exp(-j / gamma)` for state `j`, normalised by their sum):
    ce_alpha * CE(draft, true token) + l1_alpha * || softmax(draft) - softmax(target) ||_1
    + confidence_alpha * BCE(confidence logit, 1 - TV(draft, target))
The target distribution comes from the (detached) main model at the same positions.  The draft logits gradient is
produced chunk by chunk in the forward pass, so no `[rows, vocab]` probabilities are kept for backward.

Behavioural contract: models/deepseek_v4/mtp.py:97-260 (attention, heads, stage) and :442-504, :704-1000 (loss, anchor
sampling, objective) of the reference.  Sequence parallelism of the draft branch (the reference exchanges a halo of
context states) is not implemented: the branch runs when the sequence-parallel size is 1.
"""
from __future__ import annotations

from typing import Any, Callable

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import ops
from ..modules.transformer import RMSNorm
from .modeling import DeepseekV4Attention, DeepseekV4DecoderLayer, HyperConnection, HyperHead, rope_tables, rope_tail

LOSS_CHUNK_ROWS = 1024


class DraftBlockAttention(DeepseekV4Attention):
    """Same projections as the family's attention; keys = [context window before the anchor | own block]."""

    def forward(self, x, context, anchors, ctx_visible, block_ok, q_pos, ctx_pos):   # noqa: D102
        """x [N*B, H] draft states, context [T, H] projected target states, anchors [N] (index into the context),
        ctx_visible [N, W] (slot k = context index anchor - 1 - k), block_ok [N], q_pos [N*B], ctx_pos [T]."""
        N, W = ctx_visible.shape
        B = x.shape[0] // N
        hd, rd = self.head_dim, self.rd

        def rotated_kv(h, pos):
            cos, sin = rope_tables(pos, rd, self.theta)
            return rope_tail(self.kv_norm(ops.linear(h, self.wkv.weight)), cos, sin)

        cos_q, sin_q = rope_tables(q_pos, rd, self.theta)
        q = ops.linear(self.q_norm(ops.linear(x, self.wq_a.weight)), self.wq_b.weight).view(N * B, self.n_heads, hd)
        q = (q.float() * torch.rsqrt(q.float().square().mean(-1, keepdim=True) + self.eps)).to(x.dtype)
        q = rope_tail(q, cos_q, sin_q).view(N, B, self.n_heads, hd)
        ctx_kv = rotated_kv(context, ctx_pos)                                           # [T, hd]
        slots = (anchors[:, None] - 1 - torch.arange(W, device=x.device)[None, :]).clamp_(min=0)
        kv = torch.cat((ctx_kv[slots], rotated_kv(x, q_pos).view(N, B, hd)), dim=1)   # [N, W + B, hd] (one shared kv head)
        visible = torch.cat((ctx_visible, block_ok[:, None].expand(N, B)), dim=1)       # [N, W + B]
        logits = torch.einsum("nbhd,nkd->nbhk", q.float(), kv.float()) * self.scale
        logits = logits.masked_fill(~visible[:, None, None, :], float("-inf"))
        sink = self.attn_sink.float().view(1, 1, -1, 1).expand(N, B, self.n_heads, 1)
        probs = torch.softmax(torch.cat((logits, sink), dim=-1), dim=-1)[..., :-1]      # the sink takes mass, adds nothing
        o = torch.einsum("nbhk,nkd->nbhd", probs, kv.float()).to(x.dtype).reshape(N * B, self.n_heads, hd)
        o = rope_tail(o, cos_q, sin_q, inverse=True).reshape(N * B, self.n_groups, -1)
        wa = self.wo_a.weight.view(self.n_groups, self.o_rank, -1)
        o = torch.einsum("tgd,grd->tgr", o, wa.to(o.dtype))
        return ops.linear(o.reshape(N * B, -1), self.wo_b.weight)


class MarkovHead(nn.Module):
    """Low-rank first-order transition logits: `markov_w2(markov_w1[previous token])`."""

    def __init__(self, vocab: int, rank: int, dtype=None):
        super().__init__()
        self.markov_w1 = nn.Embedding(vocab, rank, dtype=dtype)
        self.markov_w2 = nn.Linear(rank, vocab, bias=False, dtype=dtype)

    def forward(self, previous_ids):
        e = self.markov_w1(previous_ids)
        return ops.linear(e, self.markov_w2.weight), e


class ConfidenceHead(nn.Module):
    def __init__(self, hidden: int, rank: int, dtype=None):
        super().__init__()
        self.proj = nn.Linear(hidden + rank, 1, bias=False, dtype=dtype)

    def forward(self, hidden, markov_embed):
        return F.linear(torch.cat((hidden, markov_embed.to(hidden.dtype)), -1), self.proj.weight).float().squeeze(-1)


class DSparkStage(DeepseekV4DecoderLayer):
    """One draft stage: a family block whose attention is the block-draft attention."""

    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__(config, layer_idx, dtype)
        self.self_attn = DraftBlockAttention(config, layer_idx, dtype)
        self.stage_idx = layer_idx - config.num_hidden_layers
        n_stages = int(config.dspark_num_layers)
        h, eps = config.hidden_size, config.rms_norm_eps
        if self.stage_idx == 0:
            self.main_proj = nn.Linear(h * len(config.dspark_target_layer_ids), h, bias=False, dtype=dtype)
            self.main_norm = RMSNorm(h, eps, dtype)
        if self.stage_idx == n_stages - 1:
            self.norm = RMSNorm(h, eps, dtype)
            self.markov_head = MarkovHead(config.vocab_size, config.dspark_markov_rank, dtype)
            self.confidence_head = ConfidenceHead(h, config.dspark_markov_rank, dtype)
            self.hc_head = HyperHead(h, config.hc_mult, config.hc_eps, eps)

    def forward(self, h, attn_args: dict, input_ids=None):   # noqa: D102
        y, post, comb = self.hc_attn.pre(h)
        a = self.self_attn(self.input_layernorm(y), **attn_args)
        h = HyperConnection.post(a, h, post, comb)
        y, post, comb = self.hc_ffn.pre(h)
        # the per-step padding mask the engine hands every MoE layer describes the main row, not the draft rows
        rt = getattr(self.mlp, "_runtime_inputs", None)
        if rt is not None and rt.padding_mask is not None:
            import dataclasses

            self.mlp.set_runtime_inputs(dataclasses.replace(rt, padding_mask=None))
        try:
            m = self.mlp(self.post_attention_layernorm(y), input_ids)
        finally:
            if rt is not None and rt.padding_mask is not None:
                self.mlp.set_runtime_inputs(rt)
        if isinstance(m, tuple):
            m = m[0]
        return HyperConnection.post(m, h, post, comb)


class _DraftLoss(torch.autograd.Function):
    """sum_rows w * (ce_alpha * CE + l1_alpha * L1(draft, target)); also the raw sums and 1 - TV per row."""

    @staticmethod
    def forward(ctx, logits, targets, weights, target_logits_fn: Callable[[int, int], torch.Tensor], ce_alpha, l1_alpha):
        R = logits.shape[0]
        grad = torch.empty_like(logits) if logits.requires_grad else None
        ce_sum = logits.new_zeros((), dtype=torch.float32)
        l1_sum = logits.new_zeros((), dtype=torch.float32)
        accept = logits.new_empty(R, dtype=torch.float32)
        for a in range(0, R, LOSS_CHUNK_ROWS):
            b = min(a + LOSS_CHUNK_ROWS, R)
            logp = torch.log_softmax(logits[a:b].float(), -1)
            p = logp.exp()
            q = torch.softmax(target_logits_fn(a, b).float(), -1)
            d = p - q
            l1 = d.abs().sum(-1)
            ce = -logp.gather(1, targets[a:b, None]).squeeze(1)
            w = weights[a:b]
            ce_sum += (ce * w).sum()
            l1_sum += (l1 * w).sum()
            accept[a:b] = (1.0 - 0.5 * l1).clamp(0.0, 1.0)
            if grad is not None:
                # d ||p - q||_1 / dz = p * (s - <p, s>), s = sign(p - q);  d CE / dz = p - onehot
                s = d.sign()
                g = p * (s - (p * s).sum(-1, keepdim=True)) * l1_alpha + p * ce_alpha
                g[torch.arange(b - a, device=g.device), targets[a:b]] -= ce_alpha
                grad[a:b] = (g * w[:, None]).to(grad.dtype)
        ctx.grad = grad
        ctx.mark_non_differentiable(ce_sum, l1_sum, accept)
        return ce_alpha * ce_sum + l1_alpha * l1_sum, ce_sum, l1_sum, accept

    @staticmethod
    def backward(ctx, g, *_):
        grad, ctx.grad = ctx.grad, None
        return (grad * g.to(grad.dtype) if grad is not None else None), None, None, None, None, None


def sample_anchors(labels: torch.Tensor, cu_seqlens, block: int, num_anchors: int, generator=None) -> torch.Tensor:
    """Positions `a` whose whole block of targets `a+1 .. a+block` lies inside `a`'s document and is supervised;
    at most `num_anchors` of them, sorted."""
    T = labels.numel()
    ok = torch.zeros(T, dtype=torch.bool, device=labels.device)
    sup = (labels.reshape(-1) != -100)
    bounds = [int(v) for v in cu_seqlens.tolist()]
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e - s > block:
            # every target of the block supervised: a sliding AND over `block` shifted copies
            good = torch.ones(e - s - block, dtype=torch.bool, device=labels.device)
            for j in range(1, block + 1):
                good &= sup[s + j:e - block + j]
            ok[s:e - block] = good
    cand = ok.nonzero().flatten()
    if cand.numel() > num_anchors:
        pick = torch.randperm(cand.numel(), generator=generator, device=cand.device)[:num_anchors]
        cand = cand[pick].sort().values
    return cand


class DSparkDraft(nn.Module):
    """The draft stages plus the training objective."""

    def __init__(self, config: Any, dtype=None):
        super().__init__()
        self.config = config
        self.block = int(config.dspark_block_size)
        L = config.num_hidden_layers
        self.stages = nn.ModuleList([DSparkStage(config, L + i, dtype) for i in range(int(config.dspark_num_layers))])
        self.metrics: dict[str, torch.Tensor] = {}

    def forward(self, *, embed: nn.Embedding, lm_head: nn.Module, target_hiddens: list[torch.Tensor], final_hidden: torch.Tensor,
                input_ids: torch.Tensor, labels: torch.Tensor, positions: torch.Tensor, cu_seqlens, train_cfg, expand,
                generator=None) -> torch.Tensor | None:
        """target_hiddens: [T, H] states of `dspark_target_layer_ids`; final_hidden [T, H] (normed output of the main
        model); labels unshifted [T].  Returns the weighted, normalised draft loss (None when no anchor fits)."""
        cfg, B = self.config, self.block
        ids, lab = input_ids.reshape(-1), labels.reshape(-1).to(input_ids.device)
        anchors = sample_anchors(lab, cu_seqlens, B, int(train_cfg.num_anchors), generator)
        N = anchors.numel()
        if N == 0:
            return None
        dev = ids.device
        W = int(cfg.sliding_window)
        offs = torch.arange(B, device=dev)
        rows = anchors[:, None] + offs[None, :]                                   # state j sits at position a + j
        block_ids = torch.full((N, B), int(cfg.dspark_mask_token_id), device=dev, dtype=ids.dtype)
        block_ids[:, 0] = ids[anchors]
        targets = ids[rows + 1].reshape(-1)                                        # state j predicts x_{a+j+1}
        previous = ids[rows].reshape(-1)                                           # teacher-forced previous token
        doc_start = torch.zeros(ids.numel(), dtype=torch.long, device=dev)
        bounds = [int(v) for v in cu_seqlens.tolist()]
        for s, e in zip(bounds[:-1], bounds[1:]):
            doc_start[s:e] = s
        slots = anchors[:, None] - 1 - torch.arange(W, device=dev)[None, :]
        ctx_visible = slots >= doc_start[anchors][:, None]
        attn_args = dict(anchors=anchors, ctx_visible=ctx_visible, block_ok=torch.ones(N, dtype=torch.bool, device=dev),
                         q_pos=positions.reshape(-1)[rows].reshape(-1), ctx_pos=positions.reshape(-1))
        first = self.stages[0]
        attn_args["context"] = first.main_norm(ops.linear(torch.cat([t.detach() for t in target_hiddens], -1), first.main_proj.weight))
        h = expand(embed(block_ids.reshape(-1)))
        for st in self.stages:
            h = st(h, attn_args, block_ids.reshape(-1))
        last = self.stages[-1]
        hidden = last.norm(last.hc_head(h))
        bias, m_embed = last.markov_head(previous)
        logits = lm_head(hidden).float() + bias.float()
        conf = last.confidence_head(hidden, m_embed)
        weights = torch.exp(-offs.float() / max(float(train_cfg.loss_decay_gamma), 1e-6)).repeat(N) if train_cfg.loss_decay_gamma > 0 \
            else torch.ones(N * B, device=dev)
        flat_rows = rows.reshape(-1)
        tgt_hidden = final_hidden.detach().reshape(-1, final_hidden.shape[-1])

        def target_logits(a: int, b: int):
            with torch.no_grad():
                return lm_head(tgt_hidden[flat_rows[a:b]])

        loss, ce_sum, l1_sum, accept = _DraftLoss.apply(logits, targets, weights, target_logits, float(train_cfg.ce_loss_alpha),
                                                        float(train_cfg.l1_loss_alpha))
        conf_loss = (F.binary_cross_entropy_with_logits(conf, accept, reduction="none") * weights).sum()
        norm = weights.sum().clamp_min(1e-6)
        total = (loss + float(train_cfg.confidence_loss_alpha) * conf_loss) / norm
        self.metrics = {"dspark/ce": (ce_sum / norm).detach(), "dspark/l1": (l1_sum / norm).detach(),
                        "dspark/confidence": (conf_loss / norm).detach(), "dspark/accept_rate": accept.mean().detach(),
                        "dspark/anchors": torch.tensor(float(N), device=dev)}
        return total

    def pop_metrics(self) -> dict[str, torch.Tensor]:
        m, self.metrics = self.metrics, {}
        return m
