"""DeepSeek-V3 style decoder used by several families (Kimi-K2.5 text model, GLM-MoE, DeepSeek-V4 base blocks):
multi-head latent attention in every layer, `first_k_dense_replace` dense blocks followed by MoE blocks with sigmoid
scores, group-limited top-k, a selection-only score correction bias, scaled normalised weights and shared experts.
Checkpoint names follow models/kimi_k25/modeling_deepseek.py of the reference (`self_attn.q_a_proj`, `mlp.gate`,
`mlp.experts.<e>.*`, `mlp.shared_experts.*`)."""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..qwen3.modeling import LMHead
from ..weight_converter import BaseWeightConverter
from .hybrid import HybridDecoderLayer, HybridModel, MRotaryEmbedding, NextNPredictLayer, run_nextn_layers
from .moe import MoELayer, MoELayerConfig
from .transformer import CausalLMOutput, DenseMLP


class DeepseekV3Config(ModelConfig):
    model_type = "deepseek_v3"
    _defaults = dict(
        vocab_size=129280, hidden_size=7168, intermediate_size=18432, moe_intermediate_size=2048, num_hidden_layers=61,
        num_nextn_predict_layers=0, num_attention_heads=128, num_key_value_heads=128, n_shared_experts=1,
        n_routed_experts=256, routed_scaling_factor=2.5, kv_lora_rank=512, q_lora_rank=1536, qk_rope_head_dim=64,
        v_head_dim=128, qk_nope_head_dim=128, n_group=8, topk_group=4, num_experts_per_tok=8, first_k_dense_replace=3,
        norm_topk_prob=True, scoring_func="sigmoid", rms_norm_eps=1e-6, rope_theta=10000.0, rope_scaling=None,
        rope_interleave=True, attention_bias=False, tie_word_embeddings=False, initializer_range=0.02,
        torch_dtype="bfloat16", pad_token_id=0, router_dtype="fp32",
    )

    def __init__(self, **kw):
        super().__init__(**kw)
        self.qk_head_dim = self.qk_nope_head_dim + self.qk_rope_head_dim
        self.head_dim = self.qk_rope_head_dim
        self.num_experts = self.n_routed_experts


def deepseek_moe_config(c, ep_size=1, engine_config=None, params_dtype=None) -> MoELayerConfig:
    groups = c.n_group if (getattr(c, "n_group", None) or 0) > 1 else None
    return MoELayerConfig(
        hidden_size=c.hidden_size, moe_ffn_hidden_size=c.moe_intermediate_size, num_moe_experts=c.n_routed_experts,
        moe_router_topk=c.num_experts_per_tok, expert_model_parallel_size=ep_size,
        params_dtype=params_dtype or torch.float32, init_method_std=getattr(c, "initializer_range", 0.02),
        moe_shared_expert_intermediate_size=(c.moe_intermediate_size * (c.n_shared_experts or 0)) or None,
        moe_aux_loss_coeff=engine_config.moe.aux_loss_coeff if engine_config is not None else 0.0,
        moe_z_loss_coeff=engine_config.moe.z_loss_coeff if engine_config is not None else 0.0,
        moe_router_num_groups=groups, moe_router_group_topk=c.topk_group if groups else None,
        moe_router_topk_scaling_factor=c.routed_scaling_factor, moe_router_score_function=c.scoring_func,
        moe_router_pre_softmax=c.scoring_func == "softmax", moe_router_dtype=getattr(c, "router_dtype", None),
        moe_router_enable_expert_bias=c.scoring_func == "sigmoid",
        num_hash_layers=int(getattr(c, "num_hash_layers", 0) or 0), vocab_size=c.vocab_size,
    )


class DeepseekMoE(MoELayer):
    """`replace_module` target and the in-model block: forward returns the tensor only."""

    def forward(self, hidden_states, input_ids=None):
        return super().forward(hidden_states, input_ids)[0]


def replace_deepseek_moe(original_module, hf_config, sp_info, ep_info, engine_config, **kwargs):
    if not isinstance(original_module, MoELayer):
        return original_module
    c = getattr(hf_config, "text_config", hf_config)
    ps = list(original_module.parameters())
    return DeepseekMoE(deepseek_moe_config(c, ep_info["ep_size"], engine_config, ps[0].dtype if ps else None),
                       ep_group=ep_info["ep_group"], sp_group=sp_info["sp_group"],
                       layer_number=getattr(original_module.router, "layer_number", None))


class DeepseekV3Model(HybridModel):
    mixer = "mla"

    def mixer_kind(self, i: int) -> str:
        return self.mixer

    def make_mlp(self, i: int, dtype) -> nn.Module:
        c = self.config
        if c.n_routed_experts and i >= c.first_k_dense_replace:
            return DeepseekMoE(deepseek_moe_config(c, 1, None, dtype or torch.float32), layer_number=i)
        return DenseMLP(c.hidden_size, c.intermediate_size, dtype)

    def make_rotary(self, config):
        return MRotaryEmbedding(config.qk_rope_head_dim, config.rope_theta)

    def make_nextn_layer(self, i: int, dtype) -> nn.Module:
        return NextNPredictLayer(self.config, HybridDecoderLayer(self.config, i, self.mixer, self.make_mlp(i, dtype), dtype), dtype)


class DeepseekV3ForCausalLMBase(nn.Module):
    model_cls = DeepseekV3Model

    def __init__(self, config: Any):
        super().__init__()
        from ..qwen3_5.modeling import as_dtype, init_hybrid_weights

        self.config = config
        dtype = as_dtype(getattr(config, "dtype", None) or getattr(config, "torch_dtype", None))
        self.model = self.model_cls(config, dtype)
        self.lm_head = LMHead(config.hidden_size, config.vocab_size, bias=False, dtype=dtype)
        n = int(getattr(config, "num_nextn_predict_layers", 0) or 0)
        self.mtp = nn.ModuleList([self.model.make_nextn_layer(config.num_hidden_layers + i, dtype) for i in range(n)]) if n else None
        if not any(p.is_meta for p in self.parameters()):
            init_hybrid_weights(self, config.initializer_range)
        self.tie_weights()

    def tie_weights(self) -> None:
        if getattr(self.config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.embed_tokens.weight

    @property
    def all_tied_weights_keys(self):
        return {"lm_head.weight": "model.embed_tokens.weight"} if getattr(self.config, "tie_word_embeddings", False) else {}

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None, cu_seq_lens_q=None, cu_seq_lens_k=None,
                max_length_q=None, max_length_k=None, skip_lm_head=False, global_input_ids=None, **extras):
        hidden, ctx = self.model(input_ids=input_ids, position_ids=position_ids, inputs_embeds=inputs_embeds,
                                 cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q, return_context=True, **extras)
        out = CausalLMOutput(hidden_states=hidden)
        ids = global_input_ids if global_input_ids is not None else input_ids
        if self.mtp is not None and self.training and ids is not None:
            m, sp_slice = self.model, None
            if m.sp_size > 1:
                Tl = hidden.shape[1]
                sp_slice = lambda e: e[m.sp_rank * Tl:(m.sp_rank + 1) * Tl]       # noqa: E731
            hs = run_nextn_layers(self.mtp, ids, hidden[0], m.embed_tokens, ctx, getattr(self.config, "pad_token_id", 0) or 0,
                                  sp_slice)
            out["mtp_hidden_states"] = [h.unsqueeze(0) for h in hs]
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
            if out.get("mtp_hidden_states"):
                out["mtp_logits"] = [self.lm_head(h) for h in out["mtp_hidden_states"]]
        return out


class DeepseekWeightConverter(BaseWeightConverter):
    hf_shared_expert_name = "shared_experts"

    def __init__(self, model, parallel_context=None, model_path=None):
        super().__init__(model, parallel_context, model_path)
        c = getattr(self.config, "text_config", self.config)
        self.num_experts = getattr(c, "n_routed_experts", 0) or 0
        self.num_local_experts = self.num_experts // self.ep_size if self.num_experts else 0


def deepseek_plan(prefix: str = "model", checkpoint: bool = True):
    from torch.distributed.tensor import Shard

    from ...parallel import FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec

    plan = {
        f"{prefix}.layers.*.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
        f"{prefix}.layers.*.mlp": FSDPPlanSpec(replace_module=replace_deepseek_moe),
    }
    if checkpoint:
        plan[f"{prefix}.layers.*"] = FSDPPlanSpec(activation_checkpoint=True)
    return FSDPParallelPlan(plan=plan, sp_size=1, ep_size=1)
