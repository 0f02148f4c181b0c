"""DeepSeek-V4 decoder on packed rows.

What is specific to this family (models/deepseek_v4/modeling_deepseek_v4.py of the reference):
  * hyper-connections (`:1047-1195`): the residual stream holds `hc_mult` copies `[T, hc, D]`.  Before a sub-layer the
    copies are mixed down to one stream with data-dependent weights (`pre`), afterwards the output is written back
    to all copies (`post`) while the old copies are re-mixed by a doubly-stochastic matrix (`comb`, Sinkhorn
    normalised).  The head mixes the copies down once more.
  * attention (`:488-880`): every head attends to ONE shared key/value row per position (K == V, width `head_dim`,
    rotary on its last `qk_rope_head_dim` channels); q is low-rank and RMS-normalised per head without a weight;
    keys are the last `sliding_window` positions plus, in layers with `compress_ratio > 1`, rows of a compressed
    stream (every `ratio` tokens pooled by a learned gate, with overlap of the previous group when `ratio == 4`).
    Layers with `ratio == 4` pick `index_topk` compressed rows per query with an indexer, the others see all
    compressed rows that end before the query.  A per-head sink logit joins the softmax.  The output is rotated back
    and projected by a grouped low-rank pair (`wo_a` per head group, `wo_b`).
  * MoE gate (`:888-960`): `sqrtsoftplus` scores, bias-corrected selection, the first `num_hash_layers` layers route
    by a token-id table; experts clamp SwiGLU at `swiglu_limit`; one shared expert.
  * prediction depths reuse the block with `enorm`/`hnorm`/`eh_proj` (mtp.py).

The indexer's Hadamard rotation is omitted: it is the same orthonormal map on queries and keys, so every score is
unchanged.  Compression works per packed sequence (a group never spans two documents; the incomplete tail of a
document is not compressed).
"""
from __future__ import annotations

import math
import warnings
from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import ops
from ...ops.providers.native_linear_attention import _bounds
from ...ops.providers.native_sparse_attention import window_indices
from ..config import ModelConfig
from ..modules.attention.ulysses import all_gather_sp_with_grad_reduce
from ..modules.hybrid import roll_left_in_sequences
from ..modules.mixers import MixerContext
from ..modules.moe import MoELayer, MoELayerConfig
from ..modules.moe.moe import MoEAuxLossAutoScaler
from ..modules.transformer import CausalLMOutput, DenseMLP, RMSNorm
from ..qwen3.modeling import LMHead


class DeepseekV4Config(ModelConfig):
    model_type = "deepseek_v4"
    _defaults = dict(
        vocab_size=129280, hidden_size=4096, intermediate_size=4096, moe_intermediate_size=4096, num_hidden_layers=42,
        num_attention_heads=64, num_key_value_heads=1, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
        scoring_func="sqrtsoftplus", route_scale=1.0, aux_loss_alpha=0.001, q_lora_rank=1024, kv_lora_rank=512,
        qk_rope_head_dim=64, qk_nope_head_dim=448, v_head_dim=512, o_groups=8, o_lora_rank=1024, sliding_window=128,
        compress_ratios=None, rope_theta=10000.0, compress_rope_theta=40000.0, index_n_heads=64, index_head_dim=128,
        index_topk=512, hc_mult=4, hc_sinkhorn_iters=20, hc_eps=1e-6, swiglu_limit=0.0, num_hash_layers=0,
        num_mtp_layers=0, rms_norm_eps=1e-6, tie_word_embeddings=False, initializer_range=0.02, pad_token_id=0,
        torch_dtype="bfloat16", first_k_dense_replace=0, router_dtype="fp32", dsa_indexer_loss_coeff=0.0,
        # DSpark block-draft heads (0 = none): block length, draft stages, rank of the transition head, the target layers
        # whose states feed the draft context (default: the last one), the token id that fills the undrafted positions
        dspark_block_size=0, dspark_num_layers=1, dspark_markov_rank=64, dspark_target_layer_ids=None, dspark_mask_token_id=None,
    )

    def __init__(self, **kw):
        if "window_size" in kw:
            kw.setdefault("sliding_window", kw.pop("window_size"))
        # checkpoints state the number of prediction depths as `num_nextn_predict_layers`
        # (models/deepseek_v4/configuration_deepseek_v4.py:179 of the reference); `num_mtp_layers` is this package's name
        if kw.get("num_nextn_predict_layers") and not kw.get("num_mtp_layers"):
            kw["num_mtp_layers"] = kw["num_nextn_predict_layers"]
        if "dspark_noise_token_id" in kw and kw.get("dspark_mask_token_id") is None:
            kw["dspark_mask_token_id"] = kw["dspark_noise_token_id"]
        super().__init__(**kw)
        self.head_dim = self.qk_nope_head_dim + self.qk_rope_head_dim
        if not self.compress_ratios:
            self.compress_ratios = [1] * self.num_hidden_layers
        self.compress_ratios = list(self.compress_ratios)
        self.num_experts = self.n_routed_experts
        self.num_nextn_predict_layers = self.num_mtp_layers
        if not self.dspark_target_layer_ids:
            self.dspark_target_layer_ids = [self.num_hidden_layers - 1]
        self.dspark_target_layer_ids = [int(i) for i in self.dspark_target_layer_ids]
        if self.dspark_mask_token_id is None:
            self.dspark_mask_token_id = int(self.pad_token_id or 0)


# --------------------------------------------------------------------------------------------------
# rotary on interleaved pairs of the trailing channels
# --------------------------------------------------------------------------------------------------
def rope_tail(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotate the last `2 * cos.shape[-1]` channels of `[T, ..., D]` as (even, odd) pairs; `inverse` rotates back."""
    rd = 2 * cos.shape[-1]
    head, tail = x[..., :-rd], x[..., -rd:]
    t = tail.float().unflatten(-1, (rd // 2, 2))
    shape = (cos.shape[0],) + (1,) * (x.dim() - 2) + (rd // 2,)
    c, s = cos.view(shape), (-sin if inverse else sin).view(shape)
    a, b = t[..., 0], t[..., 1]
    rot = torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2).to(x.dtype)
    return torch.cat((head, rot), dim=-1)


def rope_tables(positions: torch.Tensor, rot_dim: int, theta: float):
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=positions.device) / rot_dim))
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


# --------------------------------------------------------------------------------------------------
# hyper-connections
# --------------------------------------------------------------------------------------------------
def sinkhorn_split(mixes, scale, base, hc: int, iters: int, eps: float):
    """mixes [T, (2 + hc) * hc] -> pre [T, hc], post [T, hc], comb [T, hc, hc] (rows = old copy, cols = new copy)."""
    pre, post, comb = mixes.split([hc, hc, hc * hc], dim=-1)
    pre = torch.sigmoid(pre * scale[0] + base[:hc]) + eps
    post = 2 * torch.sigmoid(post * scale[1] + base[hc:2 * hc])
    comb = (comb.unflatten(-1, (hc, hc)) * scale[2] + base[2 * hc:].view(hc, hc)).softmax(-1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(iters - 1):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    return pre, post, comb


class HyperConnection(nn.Module):
    """Mix-down / write-back pair around one sub-layer."""

    def __init__(self, hidden: int, hc: int, iters: int, eps: float, norm_eps: float):
        super().__init__()
        self.hc, self.iters, self.eps, self.norm_eps = hc, iters, eps, norm_eps
        mix = (2 + hc) * hc
        self.fn = nn.Parameter(torch.zeros(mix, hc * hidden, dtype=torch.float32))
        self.base = nn.Parameter(torch.zeros(mix, dtype=torch.float32))
        self.scale = nn.Parameter(torch.ones(3, dtype=torch.float32))

    def pre(self, x):
        """x [T, hc, D] -> (y [T, D], post, comb)"""
        flat = x.flatten(1).float()
        rs = torch.rsqrt(flat.square().mean(-1, keepdim=True) + self.norm_eps)
        pre, post, comb = sinkhorn_split(F.linear(flat, self.fn) * rs, self.scale, self.base, self.hc, self.iters, self.eps)
        y = (pre.unsqueeze(-1) * x.float()).sum(1)
        return y.to(x.dtype), post, comb

    @staticmethod
    def post(out, residual, post, comb):
        """new[h'] = post[h'] * out + sum_h comb[h, h'] * residual[h]"""
        y = post.unsqueeze(-1) * out.float().unsqueeze(1) + torch.einsum("thg,thd->tgd", comb, residual.float())
        return y.to(out.dtype)


class HyperHead(nn.Module):
    def __init__(self, hidden: int, hc: int, eps: float, norm_eps: float):
        super().__init__()
        self.eps, self.norm_eps = eps, norm_eps
        self.fn = nn.Parameter(torch.zeros(hc, hc * hidden, dtype=torch.float32))
        self.base = nn.Parameter(torch.zeros(hc, dtype=torch.float32))
        self.scale = nn.Parameter(torch.ones(1, dtype=torch.float32))

    def forward(self, x):
        flat = x.flatten(1).float()
        rs = torch.rsqrt(flat.square().mean(-1, keepdim=True) + self.norm_eps)
        pre = torch.sigmoid(F.linear(flat, self.fn) * rs * self.scale + self.base) + self.eps
        return (pre.unsqueeze(-1) * x.float()).sum(1).to(x.dtype)


# --------------------------------------------------------------------------------------------------
# compressed key/value stream
# --------------------------------------------------------------------------------------------------
class Compressor(nn.Module):
    """Gated pooling of every `ratio` consecutive tokens of a sequence into one row of width `head_dim`; with
    `ratio == 4` a group also pools the first half-channels of the previous group (overlap)."""

    def __init__(self, config: Any, ratio: int, head_dim: int, dtype=None):
        super().__init__()
        self.ratio, self.head_dim, self.rd = ratio, head_dim, config.qk_rope_head_dim
        self.overlap = ratio == 4
        c = 2 if self.overlap else 1
        self.ape = nn.Parameter(torch.zeros(ratio, c * head_dim, dtype=torch.float32))
        self.wkv = nn.Linear(config.hidden_size, c * head_dim, bias=False, dtype=torch.float32)
        self.wgate = nn.Linear(config.hidden_size, c * head_dim, bias=False, dtype=torch.float32)
        self.norm = RMSNorm(head_dim, config.rms_norm_eps, dtype)
        self.theta = config.compress_rope_theta

    def forward(self, x, cu_seqlens, positions):
        """x [T, H] (full sequence) -> (rows [Tc, head_dim], end [Tc]: global index after each group's last token,
        seq_of [Tc]); `None` when no sequence holds a whole group."""
        r, d = self.ratio, self.head_dim
        xf = x.float()
        kv_all, sc_all = self.wkv(xf), self.wgate(xf)
        rows, ends, seqs, first_pos = [], [], [], []
        for n, (a, b) in enumerate(_bounds(cu_seqlens, x.shape[0])):
            g = (b - a) // r
            if g == 0:
                continue
            kv = kv_all[a:a + g * r].view(g, r, -1)
            sc = sc_all[a:a + g * r].view(g, r, -1) + self.ape
            if self.overlap:
                kv2 = kv.new_zeros(g, 2 * r, d)
                sc2 = sc.new_full((g, 2 * r, d), float("-inf"))
                kv2[:, r:], sc2[:, r:] = kv[..., d:], sc[..., d:]
                kv2[1:, :r], sc2[1:, :r] = kv[:-1, :, :d], sc[:-1, :, :d]
                kv, sc = kv2, sc2
            rows.append((kv * sc.softmax(dim=1)).sum(1))
            ends.append(a + r * torch.arange(1, g + 1, device=x.device))
            seqs.append(torch.full((g,), n, device=x.device))
            first_pos.append(positions[a:a + g * r:r])
        if not rows:
            return None
        out = self.norm(torch.cat(rows).to(x.dtype))
        cos, sin = rope_tables(torch.cat(first_pos), self.rd, self.theta)
        return rope_tail(out, cos, sin), torch.cat(ends), torch.cat(seqs)


class Indexer(nn.Module):
    def __init__(self, config: Any, ratio: int, dtype=None):
        super().__init__()
        self.n_heads, self.head_dim, self.topk = config.index_n_heads, config.index_head_dim, config.index_topk
        self.rd = config.qk_rope_head_dim
        self.wq_b = nn.Linear(config.q_lora_rank, self.n_heads * self.head_dim, bias=False, dtype=dtype)
        self.weights_proj = nn.Linear(config.hidden_size, self.n_heads, bias=False, dtype=dtype)
        self.compressor = Compressor(config, ratio, self.head_dim, dtype)

    def _queries(self, x_full, qr_local, cos, sin, q_rows):
        Tl = qr_local.shape[0]
        q = ops.linear(qr_local, self.wq_b.weight).view(Tl, self.n_heads, self.head_dim)
        q = rope_tail(q, cos, sin)
        w = ops.linear(x_full[q_rows], self.weights_proj.weight).float() * (self.head_dim ** -0.5 * self.n_heads ** -0.5)
        return q, w

    @torch.no_grad()
    def forward(self, x_full, qr_local, cos, sin, cu_seqlens, positions_full, q_rows):
        """Selected rows of the compressed stream per local query: [T_local, topk] (-1 padded), or None."""
        comp = self.compressor(x_full, cu_seqlens, positions_full)
        if comp is None:
            return None
        k, ends, seq_of = comp
        q, w = self._queries(x_full, qr_local, cos, sin, q_rows)
        sc = (torch.relu(torch.einsum("thd,cd->thc", q.float(), k.float())) * w.unsqueeze(-1)).sum(1)     # [Tl, Tc]
        visible = visible_compressed(q_rows, ends, seq_of, cu_seqlens, x_full.shape[0])
        sc = sc.masked_fill(~visible, float("-inf"))
        kk = min(self.topk, sc.shape[1])
        val, idx = sc.topk(kk, dim=-1)
        return idx.masked_fill(~torch.isfinite(val), -1).to(torch.int32)

    def kl_loss(self, x_full, qr_local, cos, sin, cu_seqlens, positions_full, q_rows, sel, q_main, ckv_main, scale):
        """Trains the indexer towards the main attention: KL(target || indexer) over the selected rows, where the
        target is the main attention's softmax over the visible compressed rows summed over heads, taken at the
        selected rows and normalised to 1, and the indexer side is the softmax of its scores over the same rows.
        Averaged over the queries that selected anything.  The target carries no gradient; the indexer's inputs are
        detached by the caller, so only indexer parameters (its compressor included) receive gradient.
        (DSAIndexerLoss / LiLoss, models/deepseek_v4/modeling_deepseek_v4.py:250-381 in the reference.)"""
        k, ends, seq_of = self.compressor(x_full, cu_seqlens, positions_full)
        valid = sel >= 0
        safe = sel.clamp_min(0).long()
        q, w = self._queries(x_full, qr_local, cos, sin, q_rows)
        s = (torch.relu(torch.einsum("thd,tkd->thk", q.float(), k.float()[safe])) * w.unsqueeze(-1)).sum(1)   # [Tl, K]
        p = torch.softmax(s.masked_fill(~valid, torch.finfo(torch.float32).min), dim=-1).masked_fill(~valid, 0.0)
        with torch.no_grad():
            visible = visible_compressed(q_rows, ends, seq_of, cu_seqlens, x_full.shape[0])
            a = torch.einsum("thd,cd->thc", q_main.float(), ckv_main.float()) * scale
            a = a.masked_fill(~visible[:, None, :], torch.finfo(torch.float32).min)
            a = torch.softmax(a, dim=-1).masked_fill(~visible[:, None, :], 0.0).sum(1)                       # [Tl, Tc]
            t = a.gather(1, safe).masked_fill(~valid, 0.0)
            t = t / t.sum(-1, keepdim=True).clamp_min(1e-12)
        kl = torch.where(t > 0, t * (t.clamp_min(1e-30).log() - (p + 1e-10).log()), torch.zeros_like(t)).sum()
        return kl / valid.any(-1).sum().clamp_min(1)


def visible_compressed(q_rows, ends, seq_of, cu_seqlens, T):
    """[Tq, Tc] True where the compressed row ends at or before the query and lies in the query's sequence."""
    seq_q = torch.zeros(T, dtype=torch.long, device=q_rows.device)
    for n, (a, b) in enumerate(_bounds(cu_seqlens, T)):
        seq_q[a:b] = n
    sq = seq_q[q_rows]
    return (ends[None, :] <= (q_rows[:, None] + 1)) & (seq_of[None, :] == sq[:, None])


# --------------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------------
class DeepseekV4Attention(nn.Module):
    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        c = config
        self.n_heads, self.head_dim, self.rd = c.num_attention_heads, c.head_dim, c.qk_rope_head_dim
        self.n_groups, self.o_rank, self.eps = c.o_groups, c.o_lora_rank, c.rms_norm_eps
        self.window = c.sliding_window
        self.ratio = c.compress_ratios[layer_idx] if layer_idx < len(c.compress_ratios) else 1
        self.wq_a = nn.Linear(c.hidden_size, c.q_lora_rank, bias=False, dtype=dtype)
        self.q_norm = RMSNorm(c.q_lora_rank, self.eps, dtype)
        self.wq_b = nn.Linear(c.q_lora_rank, self.n_heads * self.head_dim, bias=False, dtype=dtype)
        self.wkv = nn.Linear(c.hidden_size, self.head_dim, bias=False, dtype=dtype)
        self.kv_norm = RMSNorm(self.head_dim, self.eps, dtype)
        self.wo_a = nn.Linear(self.n_heads * self.head_dim // self.n_groups, self.n_groups * self.o_rank, bias=False, dtype=dtype)
        self.wo_b = nn.Linear(self.n_groups * self.o_rank, c.hidden_size, bias=False, dtype=dtype)
        self.attn_sink = nn.Parameter(torch.zeros(self.n_heads, dtype=torch.float32))
        self.compressor = Compressor(c, self.ratio, self.head_dim, dtype) if self.ratio > 1 else None
        self.indexer = Indexer(c, self.ratio, dtype) if self.ratio == 4 else None
        self.theta = c.compress_rope_theta if self.ratio > 1 else c.rope_theta
        self.scale = self.head_dim ** -0.5
        self.indexer_loss_coeff = float(getattr(c, "dsa_indexer_loss_coeff", 0.0) or 0.0)
        self.last_indexer_loss: torch.Tensor | None = None

    def forward(self, x, ctx: MixerContext):
        """x [T_local, H].  Under sequence parallelism the shared key/value stream and the layer input (for the
        compressed stream) are gathered over the group; queries stay local."""
        Tl = x.shape[0]
        sp, r = ctx.sp_size, ctx.sp_rank
        pos_full = ctx.extras["positions_full"]
        q_rows = torch.arange(r * Tl, (r + 1) * Tl, device=x.device)
        cos_f, sin_f = rope_tables(pos_full, self.rd, self.theta)
        cos, sin = cos_f[q_rows], sin_f[q_rows]
        qr = self.q_norm(ops.linear(x, self.wq_a.weight))
        q = ops.linear(qr, self.wq_b.weight).view(Tl, self.n_heads, self.head_dim)
        q = (q.float() * torch.rsqrt(q.float().square().mean(-1, keepdim=True) + self.eps)).to(x.dtype)
        q = rope_tail(q, cos, sin)
        kv = rope_tail(self.kv_norm(ops.linear(x, self.wkv.weight)), cos, sin)
        x_full = x
        if sp > 1:
            kv = all_gather_sp_with_grad_reduce(kv, 0, ctx.sp_group, sp)
            if self.ratio > 1:
                x_full = all_gather_sp_with_grad_reduce(x, 0, ctx.sp_group, sp)
        T = kv.shape[0]
        idx = window_indices(T, self.window, ctx.cu_seqlens, x.device)[q_rows]
        keys = kv
        index_loss = None
        if self.compressor is not None:
            comp = self.compressor(x_full, ctx.cu_seqlens, pos_full)
            if comp is not None:
                ckv, ends, seq_of = comp
                if self.indexer is not None:
                    sel = self.indexer(x_full.detach(), qr.detach(), cos, sin, ctx.cu_seqlens, pos_full, q_rows)
                    if sel is not None and self.training and self.indexer_loss_coeff > 0 and torch.is_grad_enabled():
                        index_loss = self.indexer.kl_loss(x_full.detach(), qr.detach(), cos, sin, ctx.cu_seqlens, pos_full,
                                                          q_rows, sel, q.detach(), ckv.detach(), self.scale)
                        self.last_indexer_loss = index_loss.detach()
                else:
                    vis = visible_compressed(q_rows, ends, seq_of, ctx.cu_seqlens, T)
                    ar = torch.arange(ckv.shape[0], device=x.device, dtype=torch.int32)
                    sel = torch.where(vis, ar[None, :], torch.full_like(ar, -1)[None, :])
                if sel is not None:
                    idx = torch.cat((idx, torch.where(sel >= 0, sel + T, sel)), dim=-1)
                    keys = torch.cat((kv, ckv), dim=0)
        kh = keys.unsqueeze(1)
        o = ops.sparse_attention(q, kh, kh, idx, scale=self.scale, sinks=self.attn_sink)
        o = rope_tail(o, cos, sin, inverse=True)
        o = o.reshape(Tl, self.n_groups, -1)
        wa = self.wo_a.weight.view(self.n_groups, self.o_rank, -1)
        o = torch.einsum("tgd,grd->tgr", o, wa.to(o.dtype))
        out = ops.linear(o.reshape(Tl, -1), self.wo_b.weight)
        if index_loss is not None:
            out = MoEAuxLossAutoScaler.apply(out, index_loss * self.indexer_loss_coeff)
        return out


# --------------------------------------------------------------------------------------------------
# MoE
# --------------------------------------------------------------------------------------------------
def moe_layer_config(c, layer_idx: int, ep_size=1, engine_config=None, params_dtype=None) -> MoELayerConfig:
    return MoELayerConfig(
        hidden_size=c.hidden_size, moe_ffn_hidden_size=c.moe_intermediate_size, num_moe_experts=c.n_routed_experts,
        moe_router_topk=c.num_experts_per_tok, expert_model_parallel_size=ep_size,
        params_dtype=params_dtype or torch.float32, init_method_std=c.initializer_range,
        moe_shared_expert_intermediate_size=(c.moe_intermediate_size * (c.n_shared_experts or 0)) or None,
        moe_aux_loss_coeff=engine_config.moe.aux_loss_coeff if engine_config is not None else 0.0,
        moe_z_loss_coeff=engine_config.moe.z_loss_coeff if engine_config is not None else 0.0,
        moe_router_topk_scaling_factor=c.route_scale, moe_router_score_function=c.scoring_func,
        moe_router_pre_softmax=c.scoring_func == "softmax", moe_router_dtype=c.router_dtype,
        moe_router_enable_expert_bias=c.scoring_func != "softmax" and layer_idx >= c.num_hash_layers,
        moe_swiglu_limit=c.swiglu_limit or None, num_hash_layers=c.num_hash_layers, vocab_size=c.vocab_size,
    )


class DeepseekV4MoE(MoELayer):
    """Hash layers (`layer_idx < num_hash_layers`) route by a persistent token-id table `tid2eid [vocab, k]`."""

    def __init__(self, config: MoELayerConfig, hash_layer: bool = False, **kw):
        super().__init__(config, **kw)
        self.hash_layer = hash_layer
        if hash_layer:
            del self.router.tid2eid                                     # plain attribute placeholder -> buffer
            self.router.register_buffer("tid2eid", self._hash_table(config), persistent=True)

    @staticmethod
    def _hash_table(config: MoELayerConfig) -> torch.Tensor:
        """Seeded token-id -> expert table for models built without a checkpoint (a checkpoint brings its own)."""
        g = torch.Generator(device="cpu").manual_seed(1234)
        with torch.device("cpu"):
            table = torch.stack([torch.randperm(config.num_moe_experts, generator=g)[: config.moe_router_topk]
                                 for _ in range(config.vocab_size)]) if config.vocab_size <= 4096 else \
                torch.randint(0, config.num_moe_experts, (config.vocab_size, config.moe_router_topk), generator=g)
        return table.to(torch.int32)

    def reset_buffers_after_materialize(self) -> None:
        """A model constructed on the meta device gets its table here, once the buffer has real storage."""
        if self.hash_layer:
            with torch.no_grad():
                self.router.tid2eid.copy_(self._hash_table(self.config).to(self.router.tid2eid.device))

    def forward(self, hidden_states, input_ids=None):
        return super().forward(hidden_states, input_ids)[0]


def replace_v4_moe(original_module, hf_config, sp_info, ep_info, engine_config, **kwargs):
    if not isinstance(original_module, MoELayer):
        return original_module
    ps = list(original_module.parameters())
    li = getattr(original_module.router, "layer_number", 0) or 0
    hashed = getattr(original_module.router, "tid2eid", None) is not None
    return DeepseekV4MoE(moe_layer_config(hf_config, li, ep_info["ep_size"], engine_config, ps[0].dtype if ps else None),
                         hash_layer=hashed, ep_group=ep_info["ep_group"], sp_group=sp_info["sp_group"], layer_number=li)


# --------------------------------------------------------------------------------------------------
# decoder
# --------------------------------------------------------------------------------------------------
class DeepseekV4DecoderLayer(nn.Module):
    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        c = config
        self.layer_idx = layer_idx
        self.self_attn = DeepseekV4Attention(c, layer_idx, dtype)
        li = min(layer_idx, c.num_hidden_layers - 1)
        if c.n_routed_experts and layer_idx >= c.first_k_dense_replace:
            self.mlp = DeepseekV4MoE(moe_layer_config(c, layer_idx, 1, None, dtype or torch.float32),
                                     hash_layer=layer_idx < c.num_hash_layers, layer_number=layer_idx)
        else:
            self.mlp = DenseMLP(c.hidden_size, c.intermediate_size, dtype)
        self.input_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype)
        self.hc_attn = HyperConnection(c.hidden_size, c.hc_mult, c.hc_sinkhorn_iters, c.hc_eps, c.rms_norm_eps)
        self.hc_ffn = HyperConnection(c.hidden_size, c.hc_mult, c.hc_sinkhorn_iters, c.hc_eps, c.rms_norm_eps)
        del li

    def forward(self, h, ctx: MixerContext):
        """h [T, hc, D] -> [T, hc, D]"""
        y, post, comb = self.hc_attn.pre(h)
        a = self.self_attn(self.input_layernorm(y), ctx)
        h = HyperConnection.post(a, h, post, comb)
        y, post, comb = self.hc_ffn.pre(h)
        m = self.mlp(self.post_attention_layernorm(y), ctx.input_ids)
        return HyperConnection.post(m, h, post, comb)


class DeepseekV4Model(nn.Module):
    def __init__(self, config: Any, dtype=None):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList([DeepseekV4DecoderLayer(config, i, dtype) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)
        self.hc_head = HyperHead(config.hidden_size, config.hc_mult, config.hc_eps, config.rms_norm_eps)
        self.sp_group, self.sp_size, self.sp_rank = None, 1, 0

    def set_sequence_parallel(self, group, size: int, rank: int | None = None) -> None:
        if rank is None:
            rank = torch.distributed.get_rank(group) if (size > 1 and group is not None) else 0
        self.sp_group, self.sp_size, self.sp_rank = group, size, rank

    def context(self, Tl, position_ids, cu, max_len, input_ids, device) -> MixerContext:
        T = Tl * self.sp_size
        if position_ids is None or position_ids.numel() != T:
            # positions restart at every document start; rebuilt from the (global) boundaries
            pos = torch.arange(T, device=device)
            if cu is not None:
                start = torch.zeros(T, dtype=torch.long, device=device)
                for a, b in _bounds(cu, T):
                    start[a:b] = a
                pos = pos - start
        else:
            pos = position_ids.reshape(-1).to(device)
        if cu is None:
            cu, max_len = torch.tensor([0, T], dtype=torch.int32), T
        ids = input_ids.reshape(-1) if input_ids is not None else None
        if ids is not None and self.sp_size > 1 and ids.numel() == T:
            ids = ids[self.sp_rank * Tl:(self.sp_rank + 1) * Tl]
        dummy = torch.zeros(Tl, 0, device=device)
        return MixerContext(dummy, dummy, cu, max_len, self.sp_group, self.sp_size, self.sp_rank, ids,
                            {"positions_full": pos})

    def expand(self, emb):
        return emb.unsqueeze(1).expand(-1, self.config.hc_mult, -1).contiguous()

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, cu_seq_lens_q=None, max_length_q=None,
                global_position_ids=None, return_context=False, collect_layers=None, **_):
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        e = inputs_embeds.reshape(-1, inputs_embeds.shape[-1])
        ctx = self.context(e.shape[0], global_position_ids if global_position_ids is not None else position_ids,
                           cu_seq_lens_q, max_length_q, input_ids, e.device)
        h = self.expand(e)
        keep = set(collect_layers or ())
        kept: dict[int, torch.Tensor] = {}
        for i, layer in enumerate(self.layers):
            h = layer(h, ctx)
            if i in keep:
                kept[i] = h.float().mean(1).to(h.dtype)      # the hyper-connection copies of a layer, averaged
        out = self.norm(self.hc_head(h)).unsqueeze(0)
        if collect_layers is not None:
            ctx.extras["layer_states"] = kept
        return (out, ctx, h) if return_context else out


class DeepseekV4NextN(nn.Module):
    """Prediction depth (models/deepseek_v4/mtp.py:32-102 of the reference): every hyper-connection copy of the
    incoming stream `[T, hc, H]` (the last decoder layer's output, or the previous depth's) is normalised and
    projected, the projected embedding of the tokens shifted one step further is added to all copies, the result runs
    through a decoder layer of its own, and the depth's own head mix and norm give the hidden state for the shared
    head.  `eh_proj [H, 2H]` holds the checkpoint's `e_proj` (columns 0..H) and `h_proj` (columns H..2H).
    Returns (stream for the next depth, hidden state for the head)."""

    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        h, eps = config.hidden_size, config.rms_norm_eps
        self.enorm, self.hnorm = RMSNorm(h, eps, dtype), RMSNorm(h, eps, dtype)
        self.eh_proj = nn.Linear(2 * h, h, bias=False, dtype=dtype)
        self.block = DeepseekV4DecoderLayer(config, layer_idx, dtype)
        self.hc_head = HyperHead(h, config.hc_mult, config.hc_eps, eps)
        self.norm = RMSNorm(h, eps, dtype)

    def forward(self, emb, stream, ctx):
        T, hc, H = stream.shape
        w = self.eh_proj.weight
        x = ops.linear(self.hnorm(stream.reshape(T * hc, H)), w[:, H:].contiguous()).view(T, hc, H)
        x = x + ops.linear(self.enorm(emb), w[:, :H].contiguous()).unsqueeze(1)
        y = self.block(x, ctx)
        return y, self.norm(self.hc_head(y))


class DeepseekV4ForCausalLMBase(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        from ..qwen3_5.modeling import as_dtype, init_hybrid_weights

        self.config = config
        dtype = as_dtype(getattr(config, "dtype", None) or getattr(config, "torch_dtype", None))
        self.model = DeepseekV4Model(config, dtype)
        self.lm_head = LMHead(config.hidden_size, config.vocab_size, bias=False, dtype=dtype)
        n = int(config.num_mtp_layers or 0)
        self.mtp = nn.ModuleList([DeepseekV4NextN(config, config.num_hidden_layers + i, dtype) for i in range(n)]) if n else None
        self.dspark = None
        if int(getattr(config, "dspark_block_size", 0) or 0) > 0:
            from .dspark import DSparkDraft

            self.dspark = DSparkDraft(config, dtype)
        if not any(p.is_meta for p in self.parameters()):
            init_hybrid_weights(self, config.initializer_range)
            self.init_family_parameters()
        self.tie_weights()

    def init_family_parameters(self) -> None:
        std = self.config.initializer_range
        with torch.no_grad():
            for m in self.modules():
                if isinstance(m, (HyperConnection, HyperHead)):
                    nn.init.normal_(m.fn, std=std)
                    m.base.zero_()
                    m.scale.fill_(1.0)
                elif isinstance(m, Compressor):
                    nn.init.normal_(m.ape, std=std)
                elif isinstance(m, DeepseekV4Attention):
                    nn.init.normal_(m.attn_sink, std=std)

    def tie_weights(self) -> None:
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.embed_tokens.weight

    @property
    def all_tied_weights_keys(self):
        return {"lm_head.weight": "model.embed_tokens.weight"} if getattr(self.config, "tie_word_embeddings", False) else {}

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, cu_seq_lens_q=None, cu_seq_lens_k=None,
                max_length_q=None, max_length_k=None, skip_lm_head=False, global_input_ids=None,
                global_position_ids=None, dspark_labels=None, dspark_config=None, **kw):
        draft = (self.dspark is not None and self.training and dspark_labels is not None and dspark_config is not None
                 and input_ids is not None)
        if draft and self.model.sp_size > 1:
            # the draft branch needs a halo of context states from the neighbouring sequence shards, which is not built:
            # say so once instead of training the main model only without notice
            if not getattr(self, "_warned_dspark_sp", False):
                self._warned_dspark_sp = True
                warnings.warn("DSpark draft heads are not trained under sequence parallelism (sp_size "
                              f"{self.model.sp_size}): the draft loss is left out of this run", RuntimeWarning, stacklevel=2)
            draft = False
        hidden, ctx, stream = self.model(input_ids=input_ids, position_ids=position_ids, inputs_embeds=inputs_embeds,
                                    cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q,
                                    global_position_ids=global_position_ids, return_context=True,
                                    collect_layers=self.config.dspark_target_layer_ids if draft else None)
        out = CausalLMOutput(hidden_states=hidden)
        if draft:
            states = ctx.extras["layer_states"]
            out["dspark_loss"] = self.dspark(
                embed=self.model.embed_tokens, lm_head=self.lm_head, expand=self.model.expand,
                target_hiddens=[states[i] for i in self.config.dspark_target_layer_ids], final_hidden=hidden[0],
                input_ids=input_ids, labels=dspark_labels, positions=ctx.extras["positions_full"], cu_seqlens=ctx.cu_seqlens,
                train_cfg=dspark_config)
        ids = global_input_ids if global_input_ids is not None else input_ids
        if self.mtp is not None and self.training and ids is not None:
            m = self.model
            Tl = hidden.shape[1]
            cur, outs, roll = stream, [], ids
            for layer in self.mtp:
                roll = roll_left_in_sequences(roll, ctx.cu_seqlens, getattr(self.config, "pad_token_id", 0) or 0)
                emb = m.embed_tokens(roll).reshape(-1, cur.shape[-1])
                if m.sp_size > 1 and emb.shape[0] != Tl:
                    emb = emb[m.sp_rank * Tl:(m.sp_rank + 1) * Tl]
                cur, head_in = layer(emb, cur, ctx)
                outs.append(head_in.unsqueeze(0))
            out["mtp_hidden_states"] = outs
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
            if out.get("mtp_hidden_states"):
                out["mtp_logits"] = [self.lm_head(h) for h in out["mtp_hidden_states"]]
        return out
