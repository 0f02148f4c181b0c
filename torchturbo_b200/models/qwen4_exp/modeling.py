"""Qwen4-Exp: hybrid decoder (gated delta rule / sparse softmax attention) with low-rank gated residual streams,
per-layer lexical embeddings, MoE feed-forward blocks and a Qwen-VL vision tower.

Family-specific mechanisms (models/qwen4_exp/modeling_qwen4_exp.py and qsa.py / ple.py of the reference):
  * gated residual (`:979-1010`): the residual is `hc_count` streams `[T, hc * H]`; a sub-layer reads a mix of the
    group-normalised streams (weights from a low-rank bottleneck, mean over streams) and its output is injected
    into every stream with a per-token, per-stream weight `2 * sigmoid(.)`.
  * QSA attention (`:650-760`, qsa.py:30-156): softmax-attention layers see, per query, the `indexer_budget` tokens
    of the best-scoring complete key blocks of `indexer_compress_ratio` tokens (score = sum over indexer heads of
    `relu(q_h . mean-pooled, normalised, rotated block key)`), plus the causal tail after the last complete block.
    Selection is shared by all heads; queries stay local under sequence parallelism and keys / values are gathered.
  * PLE (`ple.py`): hashed n-gram rows gated into every stream on linear-attention layers named by `ple_layer_ids`.
"""
from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import ops
from ...ops.providers.native_linear_attention import _bounds
from ..config import ModelConfig
from ..modules.attention.ulysses import all_gather_sp_with_grad_reduce
from ..modules.hybrid import MRotaryEmbedding
from ..modules.mixers import GatedAttention, GatedDeltaNet, MixerContext, apply_partial_rope
from ..modules.moe import MoELayer
from ..modules.transformer import CausalLMOutput, RMSNorm
from ..qwen3.modeling import LMHead
from ..qwen3_5.modeling import Qwen3_5Config, as_dtype, init_hybrid_weights
from ..qwen3_5_moe.model import Qwen3_5MoeTextConfig, moe_layer_config
from ..qwen3_vl.modeling import VisionTower
from .ple import GroupRMSNorm, PLELayer


class Qwen4ExpTextConfig(Qwen3_5MoeTextConfig):
    model_type = "qwen4_exp_text"
    _defaults = dict(hc_count=4, hc_lowrank=320, ple_layer_ids=None, ple_embed_dim=None, ple_conv_kernel_size=4, ngram_size=3,
                     heads_per_ngram=8, ngram_vocab_size_base=20_000_000, make_ngram_vocab_size_divisible_by=128, seed=0,
                     indexer_n_heads=None, indexer_kv_heads=1, indexer_head_dim=None, indexer_budget=None,
                     indexer_compress_ratio=None, eos_token_id=0)

    def __init__(self, **kw):
        super().__init__(**kw)
        self.ple_layer_ids = sorted(set(self.ple_layer_ids or []))
        self.ple_embed_dim = self.ple_embed_dim or self.hidden_size
        if self.hc_count <= 1:
            raise ValueError("hc_count must be at least 2")
        if self.indexer_budget:
            if self.indexer_kv_heads != 1:
                raise ValueError("QSA requires indexer_kv_heads=1")
            if self.indexer_budget % self.indexer_compress_ratio:
                raise ValueError("indexer_budget must be a multiple of indexer_compress_ratio")
        for lid in self.ple_layer_ids:
            if not 1 <= lid <= self.num_hidden_layers or self.layer_types[lid - 1] != "linear_attention":
                raise ValueError(f"ple_layer_ids entry {lid} must name a linear-attention layer (1-based)")


class Qwen4ExpConfig(Qwen3_5Config):
    model_type = "qwen4_exp"
    text_config_class = Qwen4ExpTextConfig
    _mirrored_extra = ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "shared_expert_intermediate_size")


class GatedResidual(nn.Module):
    def __init__(self, config: Any, dtype=None, use_combine: bool = True):
        super().__init__()
        self.hc, self.H = config.hc_count, config.hidden_size
        n = self.hc * self.H
        self.hc_norm = GroupRMSNorm(n, self.H, config.rms_norm_eps, dtype)
        self.input_mix_weight_down = nn.Linear(n, config.hc_lowrank, bias=False, dtype=dtype)
        self.input_mix_weight_up = nn.Linear(config.hc_lowrank, n, bias=False, dtype=dtype)
        self.block_inject_weight = nn.Linear(n, self.hc, bias=False, dtype=dtype) if use_combine else None

    def forward(self, streams):
        """streams [T, hc*H] -> (sub-layer input [T, H], injection weights [T, hc])"""
        normed = self.hc_norm(streams)
        mix = torch.sigmoid(F.linear(F.silu(F.linear(normed, self.input_mix_weight_down.weight) / self.hc),
                                     self.input_mix_weight_up.weight))
        x = (mix.view(-1, self.hc, self.H) * normed.view(-1, self.hc, self.H)).mean(1)
        if self.block_inject_weight is None:
            return x, None
        inject = 2 * torch.sigmoid(F.linear(normed, self.block_inject_weight.weight) / self.hc)
        return x, inject

    @staticmethod
    def inject(streams, out, weights):
        return streams + (out.unsqueeze(1) * weights.unsqueeze(-1).to(out.dtype)).flatten(1)


class QSAIndexer(nn.Module):
    def __init__(self, config: Any, dtype=None):
        super().__init__()
        c = config
        self.n_heads, self.head_dim = c.indexer_n_heads, c.indexer_head_dim
        self.budget, self.ratio = c.indexer_budget, c.indexer_compress_ratio
        self.block_topk = self.budget // self.ratio
        self.index_qk_proj = nn.Linear(c.hidden_size, (self.n_heads + 1) * self.head_dim, bias=False, dtype=dtype)
        self.q_layernorm = RMSNorm(self.head_dim, c.rms_norm_eps, dtype, one_plus_weight=True)
        self.k_layernorm = RMSNorm(self.head_dim, c.rms_norm_eps, dtype, one_plus_weight=True)

    @torch.no_grad()
    def forward(self, x, ctx: MixerContext) -> torch.Tensor:
        """Selected key rows per local query: int32 [T_local, budget + ratio - 1] (global rows, -1 = unused)."""
        Tl, r = x.shape[0], self.ratio
        qk = ops.linear(x, self.index_qk_proj.weight)
        q = self.q_layernorm(qk[:, : self.n_heads * self.head_dim].reshape(Tl, self.n_heads, self.head_dim).contiguous())
        q = apply_partial_rope(q, ctx.cos, ctx.sin)
        raw = qk[:, self.n_heads * self.head_dim:]
        cos, sin = ctx.cos, ctx.sin
        if ctx.sp_size > 1:
            packed = torch.cat((raw.float(), cos, sin), -1)
            full = packed.new_empty(ctx.sp_size * Tl, packed.shape[1])
            torch.distributed.all_gather_into_tensor(full, packed.contiguous(), group=ctx.sp_group)
            raw, cos, sin = full[:, : self.head_dim].to(raw.dtype), full[:, self.head_dim: self.head_dim + cos.shape[1]], \
                full[:, self.head_dim + cos.shape[1]:]
        T = raw.shape[0]
        off = ctx.sp_rank * Tl
        out = torch.full((Tl, self.budget + r - 1), -1, dtype=torch.int32, device=x.device)
        tail = torch.arange(r - 1, device=x.device)
        blk = torch.arange(r, device=x.device)
        for a, b in _bounds(ctx.cu_seqlens, T):
            qa, qb = max(a, off), min(b, off + Tl)
            if qa >= qb:
                continue
            pos = torch.arange(qa, qb, device=x.device) - a                       # position inside the sample
            complete = (pos + 1) // r                                             # complete blocks visible to the query
            nb = (qb - a) // r
            n_sel = torch.zeros_like(complete)
            rows = out[qa - off:qb - off]
            if nb:
                pooled = self.k_layernorm(raw[a:a + nb * r].view(nb, r, -1).float().mean(1).to(raw.dtype))
                bk = apply_partial_rope(pooled.unsqueeze(1), cos[a:a + nb * r:r], sin[a:a + nb * r:r])[:, 0]
                sc = torch.relu(torch.einsum("thd,bd->thb", q[qa - off:qb - off].float(), bk.float())).sum(1) / math.sqrt(self.head_dim)
                vis = torch.arange(nb, device=x.device)[None, :] < complete[:, None]
                sc = sc.masked_fill(~vis, torch.finfo(sc.dtype).min)
                k = min(self.block_topk, nb)
                ids = sc.topk(k, dim=-1).indices
                ok = ids < complete[:, None]
                n_sel = ok.sum(1)
                # valid blocks first, so the tail can be written right after them
                order = torch.argsort((~ok).to(torch.int8), dim=1, stable=True)
                ids, ok = ids.gather(1, order), ok.gather(1, order)
                tok = (a + ids.unsqueeze(-1) * r + blk).to(torch.int32).masked_fill(~ok.unsqueeze(-1), -1).flatten(1)
                rows[:, : tok.shape[1]] = tok
            t0 = complete * r
            tail_len = pos + 1 - t0
            ids_t = torch.where(tail[None, :] < tail_len[:, None], a + t0[:, None] + tail[None, :], -1).to(torch.int32)
            dest = n_sel[:, None] * r + tail[None, :]
            rows.scatter_(1, dest, ids_t)
        return out


class QSAAttention(GatedAttention):
    """Gated softmax attention over the indexer's selection (all heads share it)."""

    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__(config, layer_idx, dtype)
        self.indexer = QSAIndexer(config, dtype) if getattr(config, "indexer_budget", None) else None

    def forward(self, x, ctx: MixerContext):
        if self.indexer is None:
            return super().forward(x, ctx)
        T = x.shape[0]
        sel = self.indexer(x.detach(), ctx)
        qg = self._lin(x, self.q_proj).view(T, self.n_q, -1)
        q, gate = qg[..., : self.head_dim], qg[..., self.head_dim:].reshape(T, -1)
        k = self._lin(x, self.k_proj).view(T, self.n_kv, self.head_dim)
        v = self._lin(x, self.v_proj).view(T, self.n_kv, self.head_dim)
        q, k = self.q_norm(q.contiguous()), self.k_norm(k)
        q, k = apply_partial_rope(q, ctx.cos, ctx.sin), apply_partial_rope(k, ctx.cos, ctx.sin)
        if ctx.sp_size > 1:
            k = all_gather_sp_with_grad_reduce(k.contiguous(), 0, ctx.sp_group, ctx.sp_size)
            v = all_gather_sp_with_grad_reduce(v.contiguous(), 0, ctx.sp_group, ctx.sp_size)
        out = ops.sparse_attention(q, k, v, sel, scale=self.scale).reshape(T, -1)
        return self._lin(out * torch.sigmoid(gate), self.o_proj)


class Qwen4ExpDecoderLayer(nn.Module):
    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        c = config
        self.layer_idx, self.layer_type = layer_idx, c.layer_types[layer_idx]
        if self.layer_type == "linear_attention":
            self.linear_attn = GatedDeltaNet(c, layer_idx, dtype)
        else:
            self.self_attn = QSAAttention(c, layer_idx, dtype)
        self.input_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, one_plus_weight=True)
        self.post_attention_layernorm = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, one_plus_weight=True)
        self.mlp = _Qwen4MoE(moe_layer_config(c, 1, None, dtype or torch.float32), layer_number=layer_idx)
        pli = c.ple_layer_ids.index(layer_idx + 1) if (layer_idx + 1) in c.ple_layer_ids else None
        self.ple = PLELayer(c, layer_idx, pli, dtype) if pli is not None else None
        self.attn_hyper_connection = GatedResidual(c, dtype)
        self.mlp_hyper_connection = GatedResidual(c, dtype)

    def forward(self, streams, ctx: MixerContext):
        if self.ple is not None:
            ex = ctx.extras
            streams = streams + self.ple(streams, ex["ple_rows"][self.ple.ple_layer_index], ex["segment_ids"],
                                         ctx.sp_group, ctx.sp_size, ctx.sp_rank)
        x, w = self.attn_hyper_connection(streams)
        mixer = self.linear_attn if self.layer_type == "linear_attention" else self.self_attn
        streams = GatedResidual.inject(streams, mixer(self.input_layernorm(x), ctx), w)
        x, w = self.mlp_hyper_connection(streams)
        return GatedResidual.inject(streams, self.mlp(self.post_attention_layernorm(x), ctx.input_ids), w)


class _Qwen4MoE(MoELayer):
    def forward(self, hidden_states, input_ids=None):
        return super().forward(hidden_states, input_ids)[0]


class Qwen4ExpTextModel(nn.Module):
    def __init__(self, config: Any, dtype=None):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList([Qwen4ExpDecoderLayer(config, i, dtype) for i in range(config.num_hidden_layers)])
        self.final_hyper_connection = GatedResidual(config, dtype, use_combine=False)
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype, one_plus_weight=True)
        rot = int(config.head_dim * getattr(config, "partial_rotary_factor", 1.0))
        self.rotary_emb = MRotaryEmbedding(rot, config.rope_theta, getattr(config, "mrope_section", None),
                                           getattr(config, "mrope_interleaved", True))
        self.sp_group, self.sp_size, self.sp_rank = None, 1, 0

    def set_sequence_parallel(self, group, size: int, rank: int | None = None) -> None:
        if rank is None:
            rank = torch.distributed.get_rank(group) if (size > 1 and group is not None) else 0
        self.sp_group, self.sp_size, self.sp_rank = group, size, rank

    def ple_inputs(self, global_ids: torch.Tensor, cu, Tl: int, device):
        """Hash on the host once per step; per PLE layer, the local rows of the table go to the device."""
        ids = global_ids.reshape(-1).cpu()
        T = ids.numel()
        seg = torch.zeros(T, dtype=torch.long)
        for n, (a, b) in enumerate(zip(cu.tolist()[:-1], cu.tolist()[1:])):
            seg[a:b] = n + 1
        lo, hi = self.sp_rank * Tl, (self.sp_rank + 1) * Tl
        rows = {}
        for layer in self.layers:
            if layer.ple is not None:
                ctx_len = layer.ple.hasher.ngram_size - 1
                a = max(lo - ctx_len, 0)
                emb = layer.ple.lookup(ids[a:hi], seg[a:hi], device)
                rows[layer.ple.ple_layer_index] = emb[lo - a:]
        return rows, seg

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, cu_seq_lens_q=None, max_length_q=None,
                global_input_ids=None, **_):
        if inputs_embeds is None:
            inputs_embeds = self.embed_tokens(input_ids)
        e = inputs_embeds.reshape(-1, inputs_embeds.shape[-1])
        Tl = e.shape[0]
        T = Tl * self.sp_size
        if position_ids is None:
            position_ids = torch.arange(self.sp_rank * Tl, (self.sp_rank + 1) * Tl, device=e.device)
        elif position_ids.dim() == 3:
            position_ids = position_ids.reshape(3, -1)[:, -Tl:]
        else:
            position_ids = position_ids.reshape(-1)[-Tl:]
        cos, sin = self.rotary_emb(position_ids.to(e.device))
        if cu_seq_lens_q is None:
            cu_seq_lens_q, max_length_q = torch.tensor([0, T], dtype=torch.int32), T
        ids_g = global_input_ids if global_input_ids is not None else input_ids
        extras = {}
        if any(l.ple is not None for l in self.layers):
            if ids_g is None or ids_g.numel() != T:
                raise ValueError("lexical embeddings need the token ids of the whole row (`global_input_ids`)")
            extras["ple_rows"], extras["segment_ids"] = self.ple_inputs(ids_g, cu_seq_lens_q, Tl, e.device)
        ids_l = ids_g.reshape(-1)[self.sp_rank * Tl:(self.sp_rank + 1) * Tl] if ids_g is not None else None
        ctx = MixerContext(cos, sin, cu_seq_lens_q, max_length_q, self.sp_group, self.sp_size, self.sp_rank, ids_l, extras)
        streams = e.repeat(1, self.config.hc_count)
        for layer in self.layers:
            streams = layer(streams, ctx)
        x, _ = self.final_hyper_connection(streams)
        return self.norm(x).unsqueeze(0)


class Qwen4ExpInner(nn.Module):
    def __init__(self, config, dtype=None):
        super().__init__()
        self.visual = VisionTower(config.vision_config, dtype)
        self.language_model = Qwen4ExpTextModel(config.text_config, dtype)


class Qwen4ExpForConditionalGenerationBase(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        self.config = config
        dtype = as_dtype(config.dtype)
        tc = config.text_config
        self.model = Qwen4ExpInner(config, dtype)
        self.lm_head = LMHead(tc.hidden_size, tc.vocab_size, bias=False, dtype=dtype)
        if not any(p.is_meta for p in self.parameters()):
            init_hybrid_weights(self, config.initializer_range)

    def tie_weights(self) -> None:
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.language_model.embed_tokens.weight

    @property
    def all_tied_weights_keys(self):
        return {"lm_head.weight": "model.language_model.embed_tokens.weight"} \
            if getattr(self.config, "tie_word_embeddings", False) else {}

    def fuse_media(self, input_ids, pixel_values, grid):
        emb = self.model.language_model.embed_tokens(input_ids)
        visual = self.model.visual
        if pixel_values is None or pixel_values.shape[0] == 0:        # no media in this rank's row
            v_in, g = visual.dummy_inputs(emb.device, emb.dtype)
            return emb + 0.0 * visual(v_in, grid_thw=g).sum()
        feats = visual(pixel_values, grid_thw=grid)
        mask = input_ids == self.config.image_token_id
        n = int(mask.sum())
        if n == 0:
            return emb + 0.0 * feats.sum()
        if n != feats.shape[0]:
            raise ValueError(f"{n} media placeholder tokens but {feats.shape[0]} media features")
        return emb.masked_scatter(mask.unsqueeze(-1), feats.to(emb.dtype))

    def forward(self, input_ids=None, position_ids=None, pixel_values=None, image_grid_thw=None, inputs_embeds=None,
                cu_seq_lens_q=None, cu_seq_lens_k=None, max_length_q=None, max_length_k=None, skip_lm_head=False, **kw):
        if inputs_embeds is None:
            inputs_embeds = self.fuse_media(input_ids, pixel_values, image_grid_thw)
        hidden = self.model.language_model(inputs_embeds=inputs_embeds, position_ids=position_ids,
                                           cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q,
                                           global_input_ids=input_ids)
        out = CausalLMOutput(hidden_states=hidden)
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
        return out
