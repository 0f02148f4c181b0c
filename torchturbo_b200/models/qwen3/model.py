"""`qwen3`: dense Qwen3 causal LM as a Turbo model.

The reference registry has no dense Qwen3 entry (it only wraps the MoE variant), yet its dense benchmark
shapes need one; this package provides it natively."""
from __future__ import annotations

from ...engine.metrics.flops import LLMFlops
from ...parallel import FSDPParallelPlan, FSDPPlanSpec
from ..base import TurboModel
from ..registry import register_model
from ..weight_converter import BaseWeightConverter
from .modeling import Qwen3Config, Qwen3ForCausalLMBase


def get_parallel_plan() -> FSDPParallelPlan:
    return FSDPParallelPlan(
        plan={
            "model.layers.*": FSDPPlanSpec(activation_checkpoint=True),
            "model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
            "lm_head": FSDPPlanSpec(standalone_world_shard=True),
        },
        sp_size=1, ep_size=1,
    )


@register_model("qwen3")
class TurboQwen3ForCausalLM(TurboModel, Qwen3ForCausalLMBase):
    config_class = Qwen3Config

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan()

    def on_materialized(self) -> None:
        self.model.rotary_emb.reset(self.model.embed_tokens.weight.device)
        self.tie_weights()

    def get_weight_converter(self, parallel_context, model_path=None):
        return BaseWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return LLMFlops

    def get_optimizer_recipe(self, optimizer_name: str):
        from ...engine.optimizers.muon import default_decoder_muon_recipe

        if optimizer_name == "muon":
            return default_decoder_muon_recipe(self)
        return super().get_optimizer_recipe(optimizer_name)
