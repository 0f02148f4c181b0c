"""`glm_moe_dsa`: GLM MoE with dynamic sparse attention: DeepSeek-V3 style MLA + MoE decoder in which every query
attends only to the `index_topk` keys picked by a light-weight indexer (a few small heads scoring
`sum_h w_h relu(q_h . k)` over the causal prefix).  "full" layers run their own indexer, "shared" layers reuse the
selection of the previous full layer (models/glm_moe_dsa/modeling_glm_moe_dsa.py:63-144,185-358 of the reference).

Sequence parallelism gathers heads for the sparse attention as Ulysses does; the selection is per token and shared by
all heads, so indexer keys and the selected indices are all-gathered across the group (they are small).
The reference fuses this path only on Ascend (glm_moe_dsa/model.py:89-100); here `ops.lightning_indexer` and
`ops.sparse_attention` are ordinary operators."""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn

from ...engine.metrics.flops import MlaLLMFlops
from ...ops import ops
from ...parallel import FSDPPlanSpec
from ..base import TurboModel
from ..bailing_hybrid.model import HybridTurboMixin
from ..modules.attention.ulysses import gather_heads_scatter_seq, gather_seq_scatter_heads
from ..modules.deepseek import (DeepseekV3Config, DeepseekV3ForCausalLMBase, DeepseekV3Model, DeepseekWeightConverter,
                                deepseek_plan)
from ..modules.hybrid import MIXERS
from ..modules.mixers import MixerContext, MLAttention, apply_partial_rope
from ..registry import register_model


class GlmMoeDsaConfig(DeepseekV3Config):
    model_type = "glm_moe_dsa"
    _defaults = dict(vocab_size=154880, hidden_size=6144, intermediate_size=12288, moe_intermediate_size=2048,
                     num_hidden_layers=78, num_attention_heads=64, num_key_value_heads=64, kv_lora_rank=512, q_lora_rank=2048,
                     qk_rope_head_dim=64, v_head_dim=256, qk_nope_head_dim=192, n_group=1, topk_group=1, rms_norm_eps=1e-5,
                     index_topk=2048, index_head_dim=128, index_n_heads=32, indexer_types=None, index_topk_pattern=None,
                     index_topk_freq=1, index_skip_topk_offset=2, mlp_layer_types=None, rope_interleave=False)

    def __init__(self, **kw):
        rp = kw.pop("rope_parameters", None) or {}
        if "rope_theta" in rp:
            kw.setdefault("rope_theta", rp["rope_theta"])
        super().__init__(**kw)
        n = self.num_hidden_layers
        if self.indexer_types is None:
            if self.index_topk_pattern:
                self.indexer_types = [{"F": "full", "S": "shared"}[c] for c in self.index_topk_pattern]
            else:
                f, off = max(self.index_topk_freq, 1), self.index_skip_topk_offset
                self.indexer_types = ["full" if (max(i - off + 1, 0) % f) == 0 else "shared" for i in range(n)]
        if len(self.indexer_types) < n:
            raise ValueError("`indexer_types` must list one entry per layer")
        if self.mlp_layer_types is None:
            self.mlp_layer_types = ["dense"] * min(3, n) + ["sparse"] * max(n - 3, 0)
        self.first_k_dense_replace = next((i for i, t in enumerate(self.mlp_layer_types) if t == "sparse"), n)


class DsaIndexer(nn.Module):
    def __init__(self, config: Any, dtype=None):
        super().__init__()
        self.n_heads, self.head_dim, self.topk = config.index_n_heads, config.index_head_dim, config.index_topk
        self.d_rope = config.qk_rope_head_dim
        self.wq_b = nn.Linear(config.q_lora_rank, self.n_heads * self.head_dim, bias=False, dtype=dtype)
        self.wk = nn.Linear(config.hidden_size, self.head_dim, bias=False, dtype=dtype)
        self.k_norm = nn.LayerNorm(self.head_dim, eps=1e-6, dtype=dtype)
        self.weights_proj = nn.Linear(config.hidden_size, self.n_heads, bias=False, dtype=dtype)

    @torch.no_grad()
    def forward(self, x, q_resid, ctx: MixerContext) -> torch.Tensor:
        """Selected key rows `[T_local, topk]` (global row numbers)."""
        T = x.shape[0]
        q = ops.linear(q_resid, self.wq_b.weight).view(T, self.n_heads, self.head_dim)
        k = self.k_norm(ops.linear(x, self.wk.weight)).view(T, 1, self.head_dim)
        q, k = apply_partial_rope(q, ctx.cos, ctx.sin), apply_partial_rope(k, ctx.cos, ctx.sin)   # rotary part first
        w = ops.linear(x, self.weights_proj.weight).float() * (self.n_heads ** -0.5)
        k = k[:, 0]
        offset = 0
        if ctx.sp_size > 1:
            full = k.new_empty(ctx.sp_size * T, self.head_dim)
            dist.all_gather_into_tensor(full, k.contiguous(), group=ctx.sp_group)
            k, offset = full, ctx.sp_rank * T
        return ops.lightning_indexer(q, k, w, self.topk, cu_seqlens=ctx.cu_seqlens, scale=self.head_dim ** -0.5,
                                     q_offset=offset)


class DsaAttention(MLAttention):
    """MLA whose softmax runs over the indexer's selection.  A layer with an indexer files its selection under its own
    layer index in `ctx.extras["dsa_topk"]`; a shared layer reads the entry of the nearest earlier layer with an
    indexer.  Keyed by layer, the entries are still the right ones when activation checkpointing replays a layer in
    the backward pass, long after later layers have filed theirs."""

    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__(config, layer_idx, dtype)
        kinds = config.indexer_types
        self.shared = (kinds[layer_idx] if layer_idx < len(kinds) else "full") == "shared"
        self.indexer = None if self.shared else DsaIndexer(config, dtype)
        self.source_layer = layer_idx if not self.shared else next(
            (i for i in range(min(layer_idx, len(kinds)) - 1, -1, -1) if kinds[i] != "shared"), None)

    def forward(self, x, ctx: MixerContext):
        T = x.shape[0]
        if ctx.extras is None:
            ctx.extras = {}
        if self.q_lora:
            q_resid = self.q_a_layernorm(ops.linear(x, self.q_a_proj.weight))
            q = ops.linear(q_resid, self.q_b_proj.weight)
        else:
            q_resid = x
            q = ops.linear(x, self.q_proj.weight)
        if self.indexer is not None:
            sel = self.indexer(x, q_resid, ctx)
            if ctx.sp_size > 1:
                full = sel.new_empty(ctx.sp_size * T, sel.shape[1])
                dist.all_gather_into_tensor(full, sel.contiguous(), group=ctx.sp_group)
                sel = full
            ctx.extras.setdefault("dsa_topk", {})[self.layer_idx] = sel
        sel = ctx.extras.get("dsa_topk", {}).get(self.source_layer)
        if sel is None:
            raise ValueError("a shared sparse-attention layer needs the selection of an earlier full layer")
        q = q.view(T, self.n_heads, self.d_qk)
        ckv = ops.linear(x, self.kv_a_proj_with_mqa.weight)
        c, k_rope = ckv[:, : self.kv_lora], ckv[:, self.kv_lora:].reshape(T, 1, self.d_rope)
        kv = ops.linear(self.kv_a_layernorm(c.contiguous()), self.kv_b_proj.weight).view(T, self.n_heads, self.d_nope + self.d_v)
        q_rope = apply_partial_rope(q[..., self.d_nope:].contiguous(), ctx.cos, ctx.sin, self.rope_interleaved)
        k_rope = apply_partial_rope(k_rope.contiguous(), ctx.cos, ctx.sin, self.rope_interleaved)
        q = torch.cat((q[..., : self.d_nope], q_rope), -1)
        k = torch.cat((kv[..., : self.d_nope], k_rope.expand(T, self.n_heads, self.d_rope)), -1)
        v = kv[..., self.d_nope:].contiguous()
        sp = ctx.sp_size
        if sp > 1:
            q, k, v = (gather_seq_scatter_heads(t.contiguous(), ctx.sp_group, sp) for t in (q, k, v))
        out = ops.sparse_attention(q, k, v, sel, scale=self.scale)
        if sp > 1:
            out = gather_heads_scatter_seq(out.contiguous(), ctx.sp_group, sp)
        return ops.linear(out.reshape(T, self.n_heads * self.d_v), self.o_proj.weight)


MIXERS["dsa"] = DsaAttention


class GlmMoeDsaModel(DeepseekV3Model):
    mixer = "dsa"


class GlmMoeDsaForCausalLMBase(DeepseekV3ForCausalLMBase):
    model_cls = GlmMoeDsaModel


@register_model("glm_moe_dsa")
class TurboGlmMoeDsaForCausalLM(HybridTurboMixin, TurboModel, GlmMoeDsaForCausalLMBase):
    config_class = GlmMoeDsaConfig

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        plan = deepseek_plan("model")
        plan.plan["model.embed_tokens"] = FSDPPlanSpec(standalone_world_shard=True)
        plan.plan["lm_head"] = FSDPPlanSpec(standalone_world_shard=True)
        return plan

    def get_weight_converter(self, parallel_context, model_path=None):
        return DeepseekWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return MlaLLMFlops
