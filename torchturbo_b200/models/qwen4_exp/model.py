"""`qwen4_exp`: Qwen4-Exp vision-language MoE with gated residual streams, sparse (QSA) attention and per-layer
lexical embeddings.

Plan (models/qwen4_exp/parallel_plan.py and model.py:132-295 of the reference): experts on the expert-data-parallel
mesh with MoE blocks rebuilt EP-aware, layers and tower blocks checkpointed, tower world-sharded with vision
balancing, embeddings and head as standalone units.  The n-gram tables are frozen and excluded from sharding and
from the optimizer; `on_materialized` can move them into node-shared CPU memory so that one copy serves every rank
of a node.  Sequence-parallel slicing happens at the language model entry; QSA gathers keys / values over the group
and the lexical convolution exchanges halos."""
from __future__ import annotations

import os

from ...engine.metrics.flops import VLMFlops
from ...parallel import FSDPPlanSpec
from ..base import TurboVLMModel
from ..modules.moe import MoELayer
from ..qwen3_5.model import Qwen3_5TurboMixin
from ..qwen3_5_moe.model import get_parallel_plan as moe_plan, moe_layer_config
from ..registry import register_model
from ..weight_converter import FusedExpertWeightConverter
from .modeling import Qwen4ExpConfig, Qwen4ExpForConditionalGenerationBase, _Qwen4MoE


def replace_moe(original_module, hf_config, sp_info, ep_info, engine_config, **kwargs):
    if not isinstance(original_module, MoELayer):
        return original_module
    tc = getattr(hf_config, "text_config", hf_config)
    ps = list(original_module.parameters())
    return _Qwen4MoE(moe_layer_config(tc, ep_info["ep_size"], engine_config, ps[0].dtype if ps else None),
                     ep_group=ep_info["ep_group"], sp_group=sp_info["sp_group"],
                     layer_number=getattr(original_module.router, "layer_number", None))


def get_parallel_plan():
    plan = moe_plan(True)
    plan.plan["model.language_model.layers.*.mlp"] = FSDPPlanSpec(replace_module=replace_moe)
    plan.plan.pop("mtp.layers.*.mlp", None)
    plan.plan.pop("mtp.layers.*.mlp.experts", None)
    plan.plan.pop("mtp.layers.*", None)
    plan.plan["model.language_model.layers.*.ple.ngram_embedding"] = FSDPPlanSpec(no_shard=True)
    return plan


@register_model("qwen4_exp")
class TurboQwen4ExpForConditionalGeneration(Qwen3_5TurboMixin, TurboVLMModel, Qwen4ExpForConditionalGenerationBase):
    config_class = Qwen4ExpConfig

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def on_materialized(self) -> None:
        super().on_materialized()
        if os.environ.get("TORCHTURBO_PLE_NODE_SHARED", "0") == "1":
            from ..modules.cpu_resident import NodeSharedCPUResidentParameter

            for layer in self.model.language_model.layers:
                if layer.ple is not None:
                    emb = layer.ple.ngram_embedding
                    emb.weight = NodeSharedCPUResidentParameter(emb.weight.detach(), requires_grad=False)

    def get_weight_converter(self, parallel_context, model_path=None):
        return FusedExpertWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return VLMFlops
