"""Bailing-MoE v3 (Ling 3.0) hybrid decoder: groups of Kimi-delta-attention layers closed by one multi-head latent
attention layer, a dense first block followed by MoE blocks with sigmoid, group-limited, bias-corrected routing and
shared experts, optional next-token-prediction depths.

Layer kinds follow models/bailing_hybrid/modeling_bailing_moe_v3.py:1086-1105 of the reference: layer `i` is softmax
(MLA) when `(i + 1) % layer_group_size == 0` or `i` lies in the incomplete last group, linear (KDA) otherwise.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..modules.hybrid import HybridDecoderLayer, HybridModel, NextNPredictLayer, run_nextn_layers
from ..modules.moe import MoELayer, MoELayerConfig
from ..modules.transformer import CausalLMOutput, DenseMLP
from ..qwen3.modeling import LMHead
from ..qwen3_5.modeling import as_dtype, init_hybrid_weights


class BailingMoeV3Config(ModelConfig):
    model_type = "bailing_hybrid"
    _defaults = dict(
        vocab_size=157184, hidden_size=2048, intermediate_size=5120, num_hidden_layers=20, num_attention_heads=16,
        num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, rope_theta=600000.0, rope_scaling=None,
        use_qkv_bias=False, use_bias=False, tie_word_embeddings=False, initializer_range=0.02, pad_token_id=156892,
        num_experts=256, num_shared_experts=1, num_experts_per_tok=8, n_group=8, topk_group=4, moe_intermediate_size=512,
        moe_shared_expert_intermediate_size=512, first_k_dense_replace=1, num_nextn_predict_layers=0,
        mtp_loss_scaling_factor=0, moe_router_enable_expert_bias=True, routed_scaling_factor=1.0, layer_group_size=5,
        kv_lora_rank=512, q_lora_rank=None, qk_rope_head_dim=64, v_head_dim=128, qk_nope_head_dim=128,
        rope_interleave=True, scoring_func="sigmoid", router_dtype="fp32", gated_attention_proj_granularity_type=None,
        no_kda_lora=False, kda_safe_gate=False, kda_lower_bound=None, short_conv_kernel_size=4, torch_dtype="bfloat16",
        expert_swiglu_limit_list=None, share_expert_swiglu_limit_list=None,
    )

    def __init__(self, **kw):
        super().__init__(**kw)
        self.qk_head_dim = self.qk_nope_head_dim + self.qk_rope_head_dim
        self.mtp_num_hidden_layers = self.num_nextn_predict_layers


def moe_layer_config(c, ep_size=1, engine_config=None, params_dtype=None) -> MoELayerConfig:
    return MoELayerConfig(
        hidden_size=c.hidden_size, moe_ffn_hidden_size=c.moe_intermediate_size, num_moe_experts=c.num_experts,
        moe_router_topk=c.num_experts_per_tok, expert_model_parallel_size=ep_size,
        params_dtype=params_dtype or torch.float32, init_method_std=getattr(c, "initializer_range", 0.02),
        moe_shared_expert_intermediate_size=(c.moe_shared_expert_intermediate_size * c.num_shared_experts) or None,
        moe_aux_loss_coeff=engine_config.moe.aux_loss_coeff if engine_config is not None else 0.0,
        moe_z_loss_coeff=engine_config.moe.z_loss_coeff if engine_config is not None else 0.0,
        moe_router_num_groups=c.n_group, moe_router_group_topk=c.topk_group,
        moe_router_topk_scaling_factor=c.routed_scaling_factor, moe_router_score_function=c.scoring_func,
        moe_router_dtype=c.router_dtype, moe_router_enable_expert_bias=bool(c.moe_router_enable_expert_bias),
    )


class BailingModel(HybridModel):
    def mixer_kind(self, i: int) -> str:
        g, n = self.config.layer_group_size, self.config.num_hidden_layers
        return "mla" if ((i + 1) % g == 0 or i >= n // g * g) else "kda"

    def make_mlp(self, i: int, dtype) -> nn.Module:
        c = self.config
        if c.num_experts and i >= c.first_k_dense_replace:
            return MoELayer(moe_layer_config(c, 1, None, dtype or torch.float32), layer_number=i)
        return DenseMLP(c.hidden_size, c.intermediate_size, dtype)

    def make_rotary(self, config):
        from ..modules.hybrid import MRotaryEmbedding

        return MRotaryEmbedding(config.qk_rope_head_dim, config.rope_theta)

    def make_nextn_layer(self, i: int, dtype) -> nn.Module:
        block = HybridDecoderLayer(self.config, i, "mla", self.make_mlp(i, dtype), dtype)
        return NextNPredictLayer(self.config, block, dtype)


class BailingMoeV3ForCausalLMBase(nn.Module):
    model_cls = BailingModel

    def __init__(self, config: Any):
        super().__init__()
        self.config = config
        dtype = as_dtype(getattr(config, "dtype", None) or getattr(config, "torch_dtype", None))
        self.model = self.model_cls(config, dtype)
        self.lm_head = LMHead(config.hidden_size, config.vocab_size, bias=False, dtype=dtype)
        n_mtp = int(getattr(config, "num_nextn_predict_layers", 0) or 0)
        self.mtp = nn.ModuleList([self.model.make_nextn_layer(config.num_hidden_layers + i, dtype) for i in range(n_mtp)]) \
            if n_mtp else None
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
                max_length_q=None, max_length_k=None, skip_lm_head=False, global_input_ids=None, **kw):
        hidden, ctx = self.model(input_ids=input_ids, position_ids=position_ids, inputs_embeds=inputs_embeds,
                                 cu_seq_lens_q=cu_seq_lens_q, max_length_q=max_length_q, return_context=True)
        out = CausalLMOutput(hidden_states=hidden)
        ids = global_input_ids if global_input_ids is not None else input_ids
        if self.mtp is not None and self.training and ids is not None:
            m = self.model
            sp_slice = None
            if m.sp_size > 1:
                Tl = hidden.shape[1]
                if ids.shape[-1] == Tl:
                    raise ValueError("prediction depths under sequence parallelism need the global row (`global_input_ids`)")
                sp_slice = lambda e: e[m.sp_rank * Tl:(m.sp_rank + 1) * Tl]       # noqa: E731
            hs = run_nextn_layers(self.mtp, ids, hidden[0], m.embed_tokens, ctx, getattr(self.config, "pad_token_id", 0) or 0,
                                  sp_slice)
            out["mtp_hidden_states"] = [h.unsqueeze(0) for h in hs]
        if not skip_lm_head:
            out["logits"] = self.lm_head(hidden)
            if out.get("mtp_hidden_states"):
                out["mtp_logits"] = [self.lm_head(h) for h in out["mtp_hidden_states"]]
        return out
