"""`qwen3_5_moe`: the Qwen3.5 hybrid decoder with MoE feed-forward blocks (routed experts plus a sigmoid-gated shared
expert) behind the vision tower, and its checkpoint layout with 3-D fused expert tensors.

Plan (models/qwen3_5_moe/parallel_plan.py:62-103 of the reference): expert containers `Shard(0)` on the expert data
parallel mesh, every `mlp` (prediction layers included) rebuilt as an EP-aware MoE layer that keeps the shared
expert, the rest as in the dense model."""
from __future__ import annotations

import torch
import torch.nn as nn

from ...engine.metrics.flops import VLMFlops
from ...parallel import FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec
from ..base import TurboVLMModel
from ..modules.moe import MoELayer, MoELayerConfig
from ..qwen3_5.model import Qwen3_5TurboMixin, get_parallel_plan as dense_plan
from ..qwen3_5.modeling import (Qwen3_5Config, Qwen3_5ForConditionalGenerationBase, Qwen3_5Inner, Qwen3_5TextConfig,
                                Qwen3_5TextModel)
from ..registry import register_model
from ..weight_converter import FusedExpertWeightConverter


class Qwen3_5MoeTextConfig(Qwen3_5TextConfig):
    model_type = "qwen3_5_moe_text"
    _defaults = dict(hidden_size=2048, num_hidden_layers=40, num_attention_heads=16, num_key_value_heads=2, head_dim=256,
                     num_experts=256, num_experts_per_tok=8, moe_intermediate_size=512, shared_expert_intermediate_size=512,
                     norm_topk_prob=True, router_aux_loss_coef=0.001, mlp_only_layers=(), decoder_sparse_step=1,
                     intermediate_size=5632)


class Qwen3_5MoeConfig(Qwen3_5Config):
    model_type = "qwen3_5_moe"
    text_config_class = Qwen3_5MoeTextConfig
    _mirrored_extra = ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "shared_expert_intermediate_size")


def moe_layer_config(tc, ep_size=1, engine_config=None, params_dtype=None) -> MoELayerConfig:
    return MoELayerConfig(
        hidden_size=tc.hidden_size, moe_ffn_hidden_size=tc.moe_intermediate_size, num_moe_experts=tc.num_experts,
        moe_router_topk=tc.num_experts_per_tok, expert_model_parallel_size=ep_size,
        params_dtype=params_dtype or torch.float32, init_method_std=getattr(tc, "initializer_range", 0.02),
        moe_shared_expert_intermediate_size=getattr(tc, "shared_expert_intermediate_size", None) or None,
        moe_shared_expert_gate=True,
        moe_aux_loss_coeff=engine_config.moe.aux_loss_coeff if engine_config is not None else 0.0,
        moe_z_loss_coeff=engine_config.moe.z_loss_coeff if engine_config is not None else 0.0,
        moe_router_pre_softmax=not getattr(tc, "norm_topk_prob", True),
    )


class Qwen3_5MoeLayerWrapper(MoELayer):
    """`replace_module` target: the same block rebuilt for the real EP / SP groups."""

    def __init__(self, original_module, hf_config, sp_info, ep_info, engine_config, **kwargs):
        tc = getattr(hf_config, "text_config", hf_config)
        ps = list(original_module.parameters())
        cfg = moe_layer_config(tc, ep_info["ep_size"], engine_config, ps[0].dtype if ps else None)
        super().__init__(cfg, ep_group=ep_info["ep_group"], sp_group=sp_info["sp_group"],
                         layer_number=getattr(original_module, "layer_number", None))

    def forward(self, hidden_states, input_ids=None):
        return super().forward(hidden_states, input_ids)[0]


class Qwen3_5MoeTextModel(Qwen3_5TextModel):
    def make_mlp(self, i: int, dtype) -> nn.Module:
        c = self.config
        dense = i in tuple(getattr(c, "mlp_only_layers", ()) or ()) or (i + 1) % max(getattr(c, "decoder_sparse_step", 1), 1)
        if dense or not c.num_experts:
            return super().make_mlp(i, dtype)
        return MoELayer(moe_layer_config(c, 1, None, dtype or torch.float32), layer_number=i)


class Qwen3_5MoeInner(Qwen3_5Inner):
    text_model_cls = Qwen3_5MoeTextModel


def get_parallel_plan(with_vision: bool = True, prefix: str = "model.language_model") -> FSDPParallelPlan:
    from torch.distributed.tensor import Shard

    base = dense_plan(with_vision).plan
    plan = {
        f"{prefix}.layers.*.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
        f"{prefix}.layers.*.mlp": FSDPPlanSpec(replace_module=Qwen3_5MoeLayerWrapper),
        "mtp.layers.*.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
        "mtp.layers.*.mlp": FSDPPlanSpec(replace_module=Qwen3_5MoeLayerWrapper),
    }
    plan.update(base)
    return FSDPParallelPlan(plan=plan, sp_size=1, ep_size=1)


@register_model("qwen3_5_moe")
class TurboQwen3_5MoeForConditionalGeneration(Qwen3_5TurboMixin, TurboVLMModel, Qwen3_5ForConditionalGenerationBase):
    config_class = Qwen3_5MoeConfig
    inner_cls = Qwen3_5MoeInner

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan(True)

    def get_weight_converter(self, parallel_context, model_path=None):
        return FusedExpertWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return VLMFlops
