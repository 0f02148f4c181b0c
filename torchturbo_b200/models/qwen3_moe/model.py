"""`qwen3_moe`: Qwen3-MoE causal LM (e.g. Qwen3-30B-A3B: 128 SwiGLU experts, top-8, normalised top-k
probabilities) with expert parallelism.

Plan (same decisions as models/qwen3_moe/parallel_plan.py:46-70 of the reference): expert containers are
sharded on the expert-data-parallel mesh, every `mlp` is rebuilt as an EP-aware `MoELayer`, embeddings and
`lm_head` are standalone world-sharded units, and no layer asks for activation checkpointing.  Routing
applies the softmax to the selected logits when `norm_topk_prob` is set (`pre_softmax = not norm_topk_prob`).
"""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ...engine.metrics.flops import MoELLMFlops
from ...parallel import FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec
from ..base import TurboModel
from ..modules.moe import MoELayer, MoELayerConfig
from ..modules.transformer import DecoderLayer, DenseMLP
from ..qwen3.modeling import Qwen3Config, Qwen3ForCausalLMBase, Qwen3Model
from ..registry import register_model
from ..weight_converter import BaseWeightConverter


class Qwen3MoeConfig(Qwen3Config):
    model_type = "qwen3_moe"
    _defaults = dict(
        hidden_size=2048, intermediate_size=6144, num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
        num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True, decoder_sparse_step=1,
        mlp_only_layers=(), router_aux_loss_coef=0.001, output_router_logits=False, shared_expert_intermediate_size=None,
    )


def moe_layer_config(hf_config: Any, ep_size: int = 1, engine_config=None, params_dtype=None) -> MoELayerConfig:
    aux = engine_config.moe.aux_loss_coeff if engine_config is not None else 0.0
    z = engine_config.moe.z_loss_coeff if engine_config is not None else 0.0
    return MoELayerConfig(
        hidden_size=hf_config.hidden_size, moe_ffn_hidden_size=hf_config.moe_intermediate_size,
        num_moe_experts=hf_config.num_experts, moe_router_topk=hf_config.num_experts_per_tok,
        expert_model_parallel_size=ep_size, params_dtype=params_dtype or torch.float32,
        init_method_std=getattr(hf_config, "initializer_range", 0.02),
        moe_shared_expert_intermediate_size=getattr(hf_config, "shared_expert_intermediate_size", None),
        moe_aux_loss_coeff=aux, moe_z_loss_coeff=z,
        moe_router_pre_softmax=not getattr(hf_config, "norm_topk_prob", True),
        moe_token_dispatcher_transport=getattr(hf_config, "moe_token_dispatcher_transport", "auto"),
    )


class Qwen3MoeLayerWrapper(MoELayer):
    """`replace_module` target of the plan: rebuilds a layer's MoE block for the actual EP / SP groups."""

    def __init__(self, original_module, hf_config, sp_info, ep_info, engine_config, **kwargs):
        dtype = next(original_module.parameters()).dtype if any(True for _ in original_module.parameters()) else None
        cfg = moe_layer_config(hf_config, ep_info["ep_size"], engine_config, dtype)
        super().__init__(cfg, ep_group=ep_info["ep_group"], sp_group=sp_info["sp_group"],
                         layer_number=getattr(original_module, "layer_number", None))

    def forward(self, hidden_states, input_ids=None):
        out, _ = super().forward(hidden_states, input_ids)
        return out


class Qwen3MoeModel(Qwen3Model):
    def _make_layer(self, config, i, dtype):
        sparse = (i not in tuple(getattr(config, "mlp_only_layers", ()) or ())) and config.num_experts > 0 and \
            (i + 1) % max(getattr(config, "decoder_sparse_step", 1), 1) == 0
        if sparse:
            mlp = MoELayer(moe_layer_config(config, 1, None, dtype or torch.float32), layer_number=i)
        else:
            mlp = DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        return DecoderLayer(config, i, mlp, dtype)


def _is_moe(model, fqn_pattern="model.layers.*.mlp"):
    return True


def get_parallel_plan() -> FSDPParallelPlan:
    from torch.distributed.tensor import Shard

    return FSDPParallelPlan(
        plan={
            "model.layers.*.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
            "model.layers.*.mlp": FSDPPlanSpec(replace_module=Qwen3MoeLayerWrapper),
            "model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
            "lm_head": FSDPPlanSpec(standalone_world_shard=True),
        },
        sp_size=1, ep_size=1,
    )


@register_model("qwen3_moe")
class TurboQwen3MoeForCausalLM(TurboModel, Qwen3ForCausalLMBase):
    config_class = Qwen3MoeConfig
    model_cls = Qwen3MoeModel

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def on_materialized(self) -> None:
        # the reference rebuilds inv_freq in bf16 for this family (models/qwen3_moe/model.py:53-72); the
        # table is tiny, so fp32 is kept and only rounded through bf16 to stay bit-compatible
        rot = self.model.rotary_emb
        rot.inv_freq_dtype = torch.float32
        rot.reset(self.model.embed_tokens.weight.device)
        self.tie_weights()

    def get_weight_converter(self, parallel_context, model_path=None):
        return BaseWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return MoELLMFlops

    def get_optimizer_recipe(self, optimizer_name: str):
        from ...engine.optimizers.muon import default_decoder_muon_recipe

        if optimizer_name == "muon":
            return default_decoder_muon_recipe(self)
        return super().get_optimizer_recipe(optimizer_name)
