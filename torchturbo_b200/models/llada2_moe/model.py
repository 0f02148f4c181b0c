"""`llada2_moe`: LLaDA2 block-diffusion language model: a GQA + MoE decoder that is trained as a masked-diffusion
denoiser on `[noisy | clean]` rows under a blockwise attention mask instead of a causal one.

Architecture as models/llada2_moe/modeling_llada2_moe.py:438-560,765-800 of the reference: fused `query_key_value`
projection, per-head RMSNorm on q and k, rotary on half of each head, `dense` output projection; MoE with sigmoid
group-limited routing, scaled weights, an expert bias and shared experts; `first_k_dense_replace` dense blocks.
`is_diffusion_model` routes training through `engine.compute_diffusion_loss` and the block-diffusion dataset
(models/llada2_moe/model.py:20-195, bd.py of the reference).  Under sequence parallelism the row is sliced like any
other input while the block mask stays global: attention gathers the sequence and scatters heads (Ulysses), so every
rank applies the full mask to its heads."""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ...engine.metrics.flops import MoELLMFlops
from ...ops import ops
from ...parallel import FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec
from ..bailing_hybrid.model import HybridTurboMixin, _ForwardOnlyMoE
from ..base import TurboModel
from ..config import ModelConfig
from ..modules.attention.ulysses import gather_heads_scatter_seq, gather_seq_scatter_heads, repeat_kv
from ..modules.hybrid import MIXERS, HybridModel, MRotaryEmbedding
from ..modules.mixers import MixerContext, apply_partial_rope
from ..modules.moe import MoELayer, MoELayerConfig
from ..modules.transformer import CausalLMOutput, DenseMLP, RMSNorm
from ..qwen3.modeling import LMHead
from ..qwen3_5.modeling import as_dtype, init_hybrid_weights
from ..registry import register_model
from ..weight_converter import BaseWeightConverter


class LLaDA2MoeConfig(ModelConfig):
    model_type = "llada2_moe"
    _defaults = dict(
        vocab_size=157184, hidden_size=2048, intermediate_size=5120, num_hidden_layers=20, num_attention_heads=16,
        num_key_value_heads=4, head_dim=None, use_qkv_bias=False, use_qk_norm=True, use_bias=False, rms_norm_eps=1e-6,
        tie_word_embeddings=False, initializer_range=0.02, rope_theta=600000.0, pad_token_id=156892, mask_token_id=156895,
        num_experts=256, num_shared_experts=1, num_experts_per_tok=8, n_group=8, topk_group=4, routed_scaling_factor=2.5,
        moe_intermediate_size=512, first_k_dense_replace=1, partial_rotary_factor=0.5, torch_dtype="bfloat16",
        moe_router_enable_expert_bias=True, score_function="sigmoid", router_dtype="fp32",
    )


def moe_layer_config(c, ep_size=1, engine_config=None, params_dtype=None) -> MoELayerConfig:
    groups = c.n_group if (c.n_group or 0) > 1 else None
    return MoELayerConfig(
        hidden_size=c.hidden_size, moe_ffn_hidden_size=c.moe_intermediate_size, num_moe_experts=c.num_experts,
        moe_router_topk=c.num_experts_per_tok, expert_model_parallel_size=ep_size,
        params_dtype=params_dtype or torch.float32, init_method_std=c.initializer_range,
        moe_shared_expert_intermediate_size=(c.moe_intermediate_size * (c.num_shared_experts or 0)) or None,
        moe_aux_loss_coeff=engine_config.moe.aux_loss_coeff if engine_config is not None else 0.0,
        moe_z_loss_coeff=engine_config.moe.z_loss_coeff if engine_config is not None else 0.0,
        moe_router_num_groups=groups, moe_router_group_topk=c.topk_group if groups else None,
        moe_router_topk_scaling_factor=c.routed_scaling_factor, moe_router_score_function=c.score_function,
        moe_router_dtype=c.router_dtype, moe_router_enable_expert_bias=bool(c.moe_router_enable_expert_bias),
    )


class BlockDiffusionAttention(nn.Module):
    """GQA attention under the row's block mask (`ctx.extras["block_allow"]`); causal packed attention when no mask
    is given (plain language-model use)."""

    def __init__(self, config: Any, layer_idx: int, dtype=None):
        super().__init__()
        self.n_q, self.n_kv, self.head_dim = config.num_attention_heads, config.num_key_value_heads, config.head_dim
        H = config.hidden_size
        self.query_key_value = nn.Linear(H, (self.n_q + 2 * self.n_kv) * self.head_dim, bias=config.use_qkv_bias, dtype=dtype)
        self.dense = nn.Linear(self.n_q * self.head_dim, H, bias=config.use_bias, dtype=dtype)
        if config.use_qk_norm:
            self.query_layernorm = RMSNorm(self.head_dim, config.rms_norm_eps, dtype)
            self.key_layernorm = RMSNorm(self.head_dim, config.rms_norm_eps, dtype)
        else:
            self.query_layernorm = self.key_layernorm = None
        self.scale = self.head_dim ** -0.5

    def forward(self, x, ctx: MixerContext):
        T, D = x.shape[0], self.head_dim
        qkv = ops.linear(x, self.query_key_value.weight)
        if self.query_key_value.bias is not None:
            qkv = qkv + self.query_key_value.bias
        q, k, v = qkv.split([self.n_q * D, self.n_kv * D, self.n_kv * D], dim=-1)
        q, k, v = q.reshape(T, self.n_q, D), k.reshape(T, self.n_kv, D), v.reshape(T, self.n_kv, D)
        if self.query_layernorm is not None:
            q, k = self.query_layernorm(q.contiguous()), self.key_layernorm(k.contiguous())
        q, k = apply_partial_rope(q, ctx.cos, ctx.sin), apply_partial_rope(k, ctx.cos, ctx.sin)
        allow = (ctx.extras or {}).get("block_allow")
        sp = ctx.sp_size
        if sp > 1:
            if self.n_q % sp:
                raise ValueError(f"{self.n_q} attention heads do not divide by sp={sp}")
            rep = max(sp // self.n_kv, 1) if self.n_kv % sp else 1
            k, v = repeat_kv(k, rep), repeat_kv(v, rep)
            q, k, v = (gather_seq_scatter_heads(t.contiguous(), ctx.sp_group, sp) for t in (q, k, v))
        if allow is not None:
            out = ops.masked_attention(q, k, v, allow, scale=self.scale)
        else:
            # a diffusion LM has no causal default: without a block mask every token of a packed segment sees the whole
            # segment (`is_causal = False` in models/llada2_moe/modeling_llada2_moe.py:466 of the reference)
            out = ops.attention(q, k, v.contiguous(), ctx.cu_seqlens, ctx.max_seqlen, causal=False, scale=self.scale)
        if sp > 1:
            out = gather_heads_scatter_seq(out.contiguous(), ctx.sp_group, sp)
        y = ops.linear(out.reshape(T, self.n_q * D), self.dense.weight)
        return y if self.dense.bias is None else y + self.dense.bias


MIXERS["block_diffusion_attention"] = BlockDiffusionAttention


class LLaDA2MoeModel(HybridModel):
    def mixer_kind(self, i: int) -> str:
        return "block_diffusion_attention"

    def make_mlp(self, i: int, dtype) -> nn.Module:
        c = self.config
        if c.num_experts and i >= c.first_k_dense_replace:
            return _ForwardOnlyMoE(moe_layer_config(c, 1, None, dtype or torch.float32), layer_number=i)
        return DenseMLP(c.hidden_size, c.intermediate_size, dtype)

    def make_rotary(self, config):
        return MRotaryEmbedding(int(config.head_dim * config.partial_rotary_factor), config.rope_theta)


class LLaDA2MoeModelLMBase(nn.Module):
    def __init__(self, config: Any):
        super().__init__()
        self.config = config
        dtype = as_dtype(getattr(config, "dtype", None) or getattr(config, "torch_dtype", None))
        self.model = LLaDA2MoeModel(config, dtype)
        self.lm_head = LMHead(config.hidden_size, config.vocab_size, bias=False, dtype=dtype)
        if not any(p.is_meta for p in self.parameters()):
            init_hybrid_weights(self, config.initializer_range)
        self.tie_weights()

    def tie_weights(self) -> None:
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.embed_tokens.weight

    @property
    def all_tied_weights_keys(self):
        return {"lm_head.weight": "model.embed_tokens.weight"} if getattr(self.config, "tie_word_embeddings", False) else {}

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, block_allow=None, cu_seq_lens_q=None,
                cu_seq_lens_k=None, max_length_q=None, max_length_k=None, skip_lm_head=False, **kw):
        extras = {"block_allow": block_allow} if block_allow is not None else {}
        hidden = self.model(input_ids=input_ids, position_ids=position_ids, inputs_embeds=inputs_embeds,
                            cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q, **extras)
        out = CausalLMOutput(hidden_states=hidden)
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
        return out


def replace_moe_only(original_module, hf_config, sp_info, ep_info, engine_config, **kwargs):
    if not isinstance(original_module, MoELayer):
        return original_module
    ps = list(original_module.parameters())
    return _ForwardOnlyMoE(moe_layer_config(hf_config, ep_info["ep_size"], engine_config, ps[0].dtype if ps else None),
                           ep_group=ep_info["ep_group"], sp_group=sp_info["sp_group"],
                           layer_number=getattr(original_module.router, "layer_number", None))


class LLaDA2WeightConverter(BaseWeightConverter):
    hf_shared_expert_name = "shared_experts"
    extra_renames = (
        (r"^model\.embed_tokens\.", "model.word_embeddings."),
        (r"\.self_attn\.", ".attention."),
        (r"\.mlp\.router\.expert_bias$", ".mlp.gate.expert_bias"),
    )


@register_model("llada2_moe")
class TurboLLaDA2MoeForCausalLM(HybridTurboMixin, TurboModel, LLaDA2MoeModelLMBase):
    config_class = LLaDA2MoeConfig
    is_diffusion_model = True

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        from torch.distributed.tensor import Shard

        return FSDPParallelPlan(plan={
            "model.layers.*.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
            "model.layers.*.mlp": FSDPPlanSpec(replace_module=replace_moe_only),
            "model.layers.*": FSDPPlanSpec(activation_checkpoint=True),
            "model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
            "lm_head": FSDPPlanSpec(standalone_world_shard=True),
        }, sp_size=1, ep_size=1)

    def on_prepare_inputs(self, inputs, *, source_inputs=None):
        """Diffusion rows carry their structure in `block_allow`, not in packed boundaries."""
        if inputs.get("block_allow") is not None:
            return inputs
        return super().on_prepare_inputs(inputs, source_inputs=source_inputs)

    def get_weight_converter(self, parallel_context, model_path=None):
        return LLaDA2WeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return MoELLMFlops
