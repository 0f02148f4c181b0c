"""`deepseek_v4`: hyper-connected decoder with shared-KV sliding-window + compressed sparse attention and a
`sqrtsoftplus` / hash-routed MoE.

Plan (models/deepseek_v4/parallel_plan.py:9-20,96-131 of the reference): layers and prediction depths checkpointed,
experts on the expert-data-parallel mesh with MoE blocks rebuilt EP-aware, and the small fp32 parameters that every
rank needs whole (`hc_*` mixers, `attn_sink`) kept out of FSDP sharding (`no_shard`, gradients averaged over the
world).  Sequence parallelism gathers the shared key/value stream over the group instead of trading heads
(models/deepseek_v4/model.py:251-569)."""
from __future__ import annotations

from ...engine.metrics.flops import MlaLLMFlops
from ...parallel import FSDPParallelPlan, FSDPPlacementSpec, FSDPPlanSpec
from ..bailing_hybrid.model import HybridTurboMixin
from ..base import TurboModel
from ..modules.deepseek import DeepseekWeightConverter
from ..registry import register_model
from .modeling import DeepseekV4Config, DeepseekV4ForCausalLMBase, replace_v4_moe

NO_SHARD_PARAMETERS = ("hc_attn.fn", "hc_attn.base", "hc_attn.scale", "hc_ffn.fn", "hc_ffn.base", "hc_ffn.scale",
                       "hc_head.fn", "hc_head.base", "hc_head.scale", "attn_sink")


def get_parallel_plan() -> FSDPParallelPlan:
    from torch.distributed.tensor import Shard

    plan = {
        "model.layers.*.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
        "model.layers.*.mlp": FSDPPlanSpec(replace_module=replace_v4_moe),
        "model.layers.*": FSDPPlanSpec(activation_checkpoint=True),
        "mtp.*.block.mlp.experts": FSDPPlanSpec(placement=FSDPPlacementSpec(Shard(0), "edp")),
        "mtp.*.block.mlp": FSDPPlanSpec(replace_module=replace_v4_moe),
        "mtp.*": FSDPPlanSpec(activation_checkpoint=True),
        "model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
        "lm_head": FSDPPlanSpec(standalone_world_shard=True),
    }
    for leaf in ("hc_attn", "hc_ffn"):
        plan[f"model.layers.*.{leaf}"] = FSDPPlanSpec(no_shard=True)
        plan[f"mtp.*.block.{leaf}"] = FSDPPlanSpec(no_shard=True)
    plan["model.hc_head"] = FSDPPlanSpec(no_shard=True)
    plan["mtp.*.hc_head"] = FSDPPlanSpec(no_shard=True)
    return FSDPParallelPlan(plan=plan, sp_size=1, ep_size=1)


@register_model("deepseek_v4")
class TurboDeepseekV4ForCausalLM(HybridTurboMixin, TurboModel, DeepseekV4ForCausalLMBase):
    config_class = DeepseekV4Config

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def on_materialized(self) -> None:
        self.tie_weights()

    def on_prepare_inputs(self, inputs, *, source_inputs=None):
        inputs = TurboModel.on_prepare_inputs(self, inputs, source_inputs=source_inputs)
        inputs.setdefault("global_input_ids", inputs["input_ids"])
        if inputs.get("position_ids") is not None:
            inputs.setdefault("global_position_ids", inputs["position_ids"])
        return inputs

    def get_weight_converter(self, parallel_context, model_path=None):
        return DeepseekWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return MlaLLMFlops
