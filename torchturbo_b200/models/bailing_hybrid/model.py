"""`bailing_hybrid`: Ling-3.0 / BailingMoeV3 (MLA + KDA + MoE) causal LM.

Plan (models/bailing_hybrid/parallel_plan.py:19-91 of the reference): every layer checkpointed, expert containers
`Shard(0)` on the expert-data-parallel mesh, MoE blocks rebuilt EP-aware with sigmoid group-limited routing, expert
bias and fp32 router; the dense first block is left alone.  Muon recipe with MLA QK-clip as in
models/bailing_moe_v3_vl/optimizer_recipe.py:20-72."""
from __future__ import annotations

import torch.nn as nn

from ...engine.metrics.flops import MlaLLMFlops
from ...parallel import FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec
from ..base import TurboModel
from ..modules.moe import MoELayer
from ..registry import register_model
from ..weight_converter import BaseWeightConverter
from .modeling import BailingMoeV3Config, BailingMoeV3ForCausalLMBase, moe_layer_config


def replace_moe_only(original_module, hf_config, sp_info, ep_info, engine_config, **kwargs):
    """`replace_module` target that leaves dense blocks untouched."""
    if not isinstance(original_module, MoELayer):
        return original_module
    c = getattr(hf_config, "text_config", hf_config)
    ps = list(original_module.parameters())
    layer = _ForwardOnlyMoE(moe_layer_config(c, ep_info["ep_size"], engine_config, ps[0].dtype if ps else None),
                            ep_group=ep_info["ep_group"], sp_group=sp_info["sp_group"],
                            layer_number=getattr(original_module.router, "layer_number", None))
    return layer


class _ForwardOnlyMoE(MoELayer):
    def forward(self, hidden_states, input_ids=None):
        return super().forward(hidden_states, input_ids)[0]


class BailingWeightConverter(BaseWeightConverter):
    """Checkpoint names of this family: `model.word_embeddings`, one `attention` attribute for both mixer kinds with
    the output projection called `dense` on MLA layers, `mlp.gate.expert_bias`, plural `shared_experts`."""

    hf_shared_expert_name = "shared_experts"
    extra_renames = (
        (r"^model\.embed_tokens\.", "model.word_embeddings."),
        (r"\.self_attn\.o_proj\.", ".attention.dense."),
        (r"\.(self_attn|linear_attn)\.", ".attention."),
        (r"\.mlp\.router\.expert_bias$", ".mlp.gate.expert_bias"),
        (r"^mtp\.(\d+)\.block\.", r"model.mtp.\1."),
        (r"^mtp\.(\d+)\.", r"model.mtp.\1."),
    )


def get_parallel_plan(prefix: str = "model") -> FSDPParallelPlan:
    from torch.distributed.tensor import Shard

    return FSDPParallelPlan(
        plan={
            f"{prefix}.layers.*.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
            f"{prefix}.layers.*.mlp": FSDPPlanSpec(replace_module=replace_moe_only),
            f"{prefix}.layers.*": FSDPPlanSpec(activation_checkpoint=True),
            "mtp.*.block.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
            "mtp.*.block.mlp": FSDPPlanSpec(replace_module=replace_moe_only),
            "mtp.*": FSDPPlanSpec(activation_checkpoint=True),
        },
        sp_size=1, ep_size=1,
    )


class HybridTurboMixin:
    """Engine hooks shared by the text-only hybrid families built on `HybridModel`."""

    def get_decoder(self) -> nn.Module:
        return self.model

    def on_parallelized(self, parallel_context) -> None:
        sp = parallel_context["sp"]
        self.get_decoder().set_sequence_parallel(sp["sp_group"], sp["sp_size"], sp["sp_rank"])

    def on_materialized(self) -> None:
        self.get_decoder().rotary_emb.reset(self.lm_head.weight.device)
        self.tie_weights()

    def on_prepare_inputs(self, inputs, *, source_inputs=None):
        inputs = super().on_prepare_inputs(inputs, source_inputs=source_inputs)
        if getattr(self, "mtp", None) is not None:
            inputs.setdefault("global_input_ids", inputs["input_ids"])    # stays global when `input_ids` is SP-sliced
        return inputs


@register_model("bailing_hybrid")
class TurboBailingMoeV3ForCausalLM(HybridTurboMixin, TurboModel, BailingMoeV3ForCausalLMBase):
    config_class = BailingMoeV3Config

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def get_weight_converter(self, parallel_context, model_path=None):
        return BailingWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return MlaLLMFlops

    def get_optimizer_recipe(self, optimizer_name: str):
        from ...engine.optimizers.muon import default_decoder_muon_recipe

        if optimizer_name == "muon":
            return default_decoder_muon_recipe(self)
        return super().get_optimizer_recipe(optimizer_name)
