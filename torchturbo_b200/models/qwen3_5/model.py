"""`qwen3_5`: dense hybrid (gated delta rule + gated attention) vision-language model.

Plan (same decisions as models/qwen3_5/parallel_plan.py:8-25 of the reference): decoder layers, ViT blocks and
prediction layers are checkpointed, `model.visual` is one world-sharded unit with vision balancing, and sequence
parallel slicing happens at the language model entry on `inputs_embeds` / `position_ids`."""
from __future__ import annotations

from ...engine.metrics.flops import VLMFlops
from ...parallel import FSDPParallelPlan, FSDPPlanSpec, VisionBalanceMode, VisionBalanceSpec
from ..base import TurboVLMModel
from ..modules.vision import GridVisionBalanceIO
from ..registry import register_model
from ..weight_converter import BaseWeightConverter
from .modeling import Qwen3_5Config, Qwen3_5ForConditionalGenerationBase


def get_parallel_plan(with_vision: bool = True) -> FSDPParallelPlan:
    plan = {
        "model.language_model.layers.*": FSDPPlanSpec(activation_checkpoint=True),
        "mtp.layers.*": FSDPPlanSpec(activation_checkpoint=True),
        "model.language_model.embed_tokens": FSDPPlanSpec(standalone_world_shard=True),
        "lm_head": FSDPPlanSpec(standalone_world_shard=True),
    }
    if with_vision:
        plan["model.visual.blocks.*"] = FSDPPlanSpec(activation_checkpoint=True)
        plan["model.visual"] = FSDPPlanSpec(standalone_world_shard=True, vision_balance=VisionBalanceSpec(
            mode=VisionBalanceMode.PATCH_SQ, io=GridVisionBalanceIO(2)))
    return FSDPParallelPlan(plan=plan, sp_size=1, ep_size=1)


class Qwen3_5TurboMixin:
    """Engine hooks shared by the dense and MoE Qwen3.5 classes."""

    multimodal_input_keys = ("pixel_values", "image_grid_thw")

    def get_norm(self):
        return self.model.language_model.norm

    def get_input_embeddings(self):
        return self.model.language_model.embed_tokens

    def get_language_model(self):
        return self.model.language_model

    def get_sequence_parallel_input_slicing_spec(self):
        from ..modules.attention.ulysses import SequenceParallelInputSlicingSpec

        lm = self.model.language_model
        return SequenceParallelInputSlicingSpec(lm, type(lm).forward)

    def on_parallelized(self, parallel_context) -> None:
        sp = parallel_context["sp"]
        self.model.language_model.set_sequence_parallel(sp["sp_group"], sp["sp_size"], sp["sp_rank"])

    def on_materialized(self) -> None:
        self.model.language_model.rotary_emb.reset(self.lm_head.weight.device)
        self.tie_weights()

    def get_weight_converter(self, parallel_context, model_path=None):
        return BaseWeightConverter(self, parallel_context, model_path)

    def get_flops_class(self):
        return VLMFlops


@register_model("qwen3_5")
class TurboQwen3_5ForConditionalGeneration(Qwen3_5TurboMixin, TurboVLMModel, Qwen3_5ForConditionalGenerationBase):
    config_class = Qwen3_5Config

    @classmethod
    def get_default_parallel_plan(cls, **kwargs):
        return get_parallel_plan(True)
